#!/usr/bin/env python
"""Benchmark of the triangle-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one forward + backward pass of fused triangle attention over one batch of
synthetic input: the headline shape B=1, H=4, L1=L2=768, D=32, bf16 (workload ``ns_l768``),
811.75 GFLOP per step by the metric's model (4*B*H*L1*L2^2*D forward, 2.5x that backward).
With N > 1 (launched by torchrun, one rank per GPU) the problem is split heads first, L1 rows second:
ranks that own different heads exchange nothing (a head's dBias is complete on its rank); ranks that
share a head own blocks of its L1 rows and all-reduce its float32 dBias among themselves over NCCL
(N = 8 at H = 4: pairs). The value is whole-problem FLOPs / max-over-ranks device time (total work
fixed: strong scaling).

Prints ONE JSON line on rank 0 (see the keys below). ``--impl reference`` times the CPU
restatement of the reference's naive path (oracle/) on the host cores instead, on rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "flash-triangle-attention_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402

WORKLOAD = "ns_l768"
METRIC = "fwd+bwd TFLOP/s, fused triangle attention B=1 H=4 L=768 D=32 bf16"
# DRAM bytes (read + write) of ONE launch of the backward kernel at the full workload, from the
# one-pass ncu capture of that launch (dram__bytes_read.sum + dram__bytes_write.sum).
BWD_KERNEL_DRAM_BYTES = 1228830208 + 1208799488
# L1 rows per block of the end-to-end leg (host tensors streamed through the GPU)
E2E_BLOCK_ROWS = int(os.environ.get("FTA_E2E_BLOCK_ROWS", "128"))


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured (burst)"
    return 1590.0, 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v == "Active"})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def cpu_reference_rate(target_seconds=12.0):
    """Times the CPU restatement of the reference's naive path (oracle/, numpy + BLAS, all host
    threads) on a bounded sample of the workload: the first rows of L1 of every head, sized to
    about ``target_seconds``. Returns (TFLOP/s, cores, sample description, seconds)."""
    import workloads
    from oracle import tt_attn_oracle as npo
    w = workloads.WORKLOADS[WORKLOAD]
    try:
        from threadpoolctl import threadpool_info
        cores = max([p.get("num_threads", 1) for p in threadpool_info()] + [1])
    except Exception:
        cores = os.cpu_count() or 1
    rng = np.random.Generator(np.random.PCG64(w.seed))

    def sample(rows):
        sh = (w.B, w.H, rows, w.L2, w.D)
        q, k, v, do = (rng.standard_normal(sh, dtype=np.float32) for _ in range(4))
        bias = rng.standard_normal((w.B, w.H, w.L2, w.L2), dtype=np.float32)
        t0 = time.perf_counter()
        npo.forward_backward(q, k, v, bias, do, w.sm_scale)
        return time.perf_counter() - t0

    sample(1)  # warm-up (BLAS thread pool, page faults)
    t2 = sample(2)
    rows = int(max(2, min(w.L1, round(2 * target_seconds / max(t2, 1e-4)))))
    t = sample(rows)
    flops = 3.5 * 4.0 * w.B * w.H * rows * w.L2 * w.L2 * w.D
    desc = f"{rows} of {w.L1} L1 rows x {w.H} heads of {WORKLOAD}, fp32 numpy/BLAS restatement, fwd+bwd"
    return flops / t / 1e12, cores, desc, t


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import workloads
    w = workloads.WORKLOADS[WORKLOAD]
    vals, secs = [], []
    cores, desc = 1, ""
    for it in range(args.warmup + args.steps):
        v, cores, desc, t = cpu_reference_rate(target_seconds=3.0)
        if it >= args.warmup:
            vals.append(v)
            secs.append(t)
    value = float(np.mean(vals))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.mean(secs)) * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "B": w.B, "H": w.H, "L1": w.L1, "L2": w.L2, "D": w.D,
                   "note": "reference = naive PyTorch path restated in numpy (the reference module "
                           "itself is Python and is not shipped); each step is a bounded sample"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--rows", type=int, default=0,
                    help="restrict the workload to its first ROWS L1 rows (a small case for ncu captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import torch.distributed as dist

    import _cabi
    import flash_tt_attn as fta
    import workloads
    from _cabi import FtaProblem, t4, t5

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(3, args.warmup)

    w = workloads.WORKLOADS[WORKLOAD]
    if args.rows > 0:
        w = w.with_rows(min(args.rows, w.L1))
    # heads first (no exchange between ranks that own different heads), L1 rows second (ranks that
    # share a head all-reduce its float32 dBias among themselves)
    heads, rows, peers = fta.shard_plan(w.H, w.L1, rank, world)
    nrows = rows.stop - rows.start
    dt = torch.bfloat16
    x = workloads.make_inputs(w, rows)
    host = {k: torch.from_numpy(np.ascontiguousarray(x[k][:, heads])).to(dt).pin_memory()
            for k in ("q", "k", "v", "do", "bias")}
    d = {k: v.to(dev) for k, v in host.items()}
    L = _cabi.lib()
    B, H, L2, D = w.B, heads.stop - heads.start, w.L2, w.D  # H: heads of this rank
    row_shards = len(peers)
    grp = None
    if world > 1 and row_shards > 1:
        # every rank takes part in the creation of every subgroup
        for g0 in range(0, world, row_shards):
            g_ = dist.new_group(list(range(g0, g0 + row_shards)))
            if g0 == peers[0]:
                grp = g_
    prob = FtaProblem(B, H, nrows, L2, D, _cabi.FTA_BF16)
    o = torch.empty_like(d["q"])
    lse = torch.empty(3, B, H, nrows, L2, dtype=torch.float32, device=dev)
    delta = torch.empty(B, H, nrows, L2, dtype=torch.float32, device=dev)
    dq, dk, dv = (torch.empty_like(d["q"]) for _ in range(3))
    db = torch.empty_like(d["bias"])
    db32 = torch.empty(B, H, L2, L2, dtype=torch.float32, device=dev)
    ws_bytes = int(L.fta_bwd_workspace_bytes(prob))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2
    stream = torch.cuda.current_stream().cuda_stream
    scale = w.sm_scale
    sharded = grp is not None

    def step():
        _cabi.check(L.fta_forward(prob, t5(d["q"]), t5(d["k"]), t5(d["v"]), t4(d["bias"]), scale, t5(o),
                                  lse.data_ptr(), status.data_ptr(), stream), "fta_forward")
        _cabi.check(L.fta_bwd_preprocess(prob, t5(o), t5(d["do"]), delta.data_ptr(), stream), "fta_bwd_preprocess")
        _cabi.check(L.fta_backward(prob, t5(d["q"]), t5(d["k"]), t5(d["v"]), t4(d["bias"]), t5(d["do"]),
                                   lse.data_ptr(), delta.data_ptr(), scale, t5(dq), t5(dk), t5(dv),
                                   db32.data_ptr(), None if sharded else db.data_ptr(), ws.data_ptr(), ws_bytes,
                                   status.data_ptr(), stream), "fta_backward")
        if sharded:
            dist.all_reduce(db32, group=grp)
            _cabi.check(L.fta_dbias_cast(db32.data_ptr(), db.data_ptr(), db32.numel(), prob.dtype, stream),
                        "fta_dbias_cast")

    launches_per_step = 6 + (1 if sharded else 0)  # fwd, preprocess, transpose, bwd, dq finalise, dbias finalise (+cast)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    barrier()

    # ---- timed region: K steps, each bracketed by CUDA events on the launching stream; L2 is
    # flushed (a 256 MB write) between steps, outside the events. Backward-kernel events too.
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    step_ms, fwd_ms, bwdk_ms = [], [], []
    barrier()
    wall0 = time.perf_counter()
    # The host only enqueues: events are recorded on the stream around every step and read after
    # the loop, so the GPU always has the next launches queued (with a synchronise per step the
    # host's launch sequence would sit exposed between the short kernels of a multi-GPU shard).
    evs = []
    for it in range(args.steps):
        flush.zero_()
        e0, e1, ef, k0, k1 = (torch.cuda.Event(enable_timing=True) for _ in range(5))
        k0.record()  # creates the underlying cudaEvent_t handles (re-recorded inside fta_backward)
        k1.record()
        L.fta_profile_backward_kernel(k0.cuda_event, k1.cuda_event)
        e0.record()
        _cabi.check(L.fta_forward(prob, t5(d["q"]), t5(d["k"]), t5(d["v"]), t4(d["bias"]), scale, t5(o),
                                  lse.data_ptr(), status.data_ptr(), stream), "fta_forward")
        ef.record()
        _cabi.check(L.fta_bwd_preprocess(prob, t5(o), t5(d["do"]), delta.data_ptr(), stream), "fta_bwd_preprocess")
        _cabi.check(L.fta_backward(prob, t5(d["q"]), t5(d["k"]), t5(d["v"]), t4(d["bias"]), t5(d["do"]),
                                   lse.data_ptr(), delta.data_ptr(), scale, t5(dq), t5(dk), t5(dv),
                                   db32.data_ptr(), None if sharded else db.data_ptr(), ws.data_ptr(), ws_bytes,
                                   status.data_ptr(), stream), "fta_backward")
        if sharded:
            dist.all_reduce(db32, group=grp)
            _cabi.check(L.fta_dbias_cast(db32.data_ptr(), db.data_ptr(), db32.numel(), prob.dtype, stream),
                        "fta_dbias_cast")
        e1.record()
        evs.append((e0, e1, ef, k0, k1))
    torch.cuda.synchronize()
    for e0, e1, ef, k0, k1 in evs:
        step_ms.append(e0.elapsed_time(e1))
        fwd_ms.append(e0.elapsed_time(ef))
        bwdk_ms.append(k0.elapsed_time(k1))
    barrier()
    wall = time.perf_counter() - wall0
    L.fta_profile_backward_kernel(None, None)
    clocks = sampler.stop() if rank == 0 else None
    if int(status.item()) != 0:
        raise SystemExit(f"device status 0x{int(status.item()):x}: a bounded device-side wait ran out")

    total_ms = float(np.sum(step_ms))
    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    flops_step = w.flops_fwd() + w.flops_bwd()  # whole problem, all ranks
    value = flops_step * args.steps / (total_ms * 1e-3) / 1e12

    # ---- end to end through the public API with HOST buffers: pinned inputs copied to the device,
    # attention + backward, outputs and gradients copied back, every step.
    e2e_steps = max(1, min(args.steps, 5))
    out_host = {k: torch.empty_like(host["q"]).pin_memory() for k in ("o", "dq", "dk", "dv")}
    db_host = torch.empty_like(host["bias"]).pin_memory()
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = sum(v.numel() * v.element_size() for v in out_host.values()) + db_host.numel() * db_host.element_size()

    out_host["dbias"] = db_host

    def e2e_step():
        # the library's host-memory entry point: blocks of L1 rows double-buffered through the GPU,
        # copies in / kernels / copies out on three streams
        fta.attention_fwd_bwd_streamed(host, scale, out_host, block_rows=E2E_BLOCK_ROWS, device=dev, group=grp)

    if args.no_e2e:
        e2e_steps = 0
    else:
        for _ in range(3):  # untimed: first touches of the pinned buffers, allocator, streams
            e2e_step()
    barrier()
    e2e_ms = []
    for _ in range(e2e_steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_step()
        e1.record()
        torch.cuda.synchronize()
        e2e_ms.append(e0.elapsed_time(e1))
    barrier()
    te = torch.tensor([float(np.sum(e2e_ms))], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_value = flops_step * e2e_steps / (float(te.item()) * 1e-3) / 1e12 if e2e_steps else None
    fta.check_device_status(dev)

    if rank == 0:
        peak_tf, peak_gbs, peak_kind = _peaks()
        bwd_kernel_ms = float(np.mean(bwdk_ms))
        bwd_flops_rank = 2.5 * 4.0 * B * H * nrows * L2 * L2 * D
        achieved = bwd_flops_rank / (bwd_kernel_ms * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD if args.rows <= 0 else f"{WORKLOAD}[first {w.L1} rows]", "B": B, "H": w.H,
                       "L1": w.L1, "L2": L2, "D": D, "heads_per_gpu": H, "rows_per_gpu": nrows,
                       "parallelism": (f"{world // row_shards} head shard(s) x {row_shards} L1-row shard(s); "
                                       f"dBias all-reduce among {row_shards} rank(s)"),
                       "l2": "flushed between steps (256 MB write outside the events)",
                       "fwd_ms": float(np.mean(fwd_ms)), "bwd_kernel_ms": bwd_kernel_ms,
                       "frac_of_bf16_peak": value / (peak_tf * world), "peak": f"{peak_tf} TFLOP/s {peak_kind}",
                       "wall_ms_per_step_incl_flush": wall / args.steps * 1e3},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h), "steps": e2e_steps},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "roofline": {"kernel": "fta_bwd_kernel", "bound": "tensor", "achieved": achieved, "peak": peak_tf,
                         "unit": "TFLOP/s", "frac": achieved / peak_tf, "traffic": BWD_KERNEL_DRAM_BYTES,
                         "peak_kind": peak_kind},
        }
        if world == 1 and not args.no_cpu_baseline:
            v, cores, desc, _ = cpu_reference_rate()
            line["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
