#!/usr/bin/env python
"""Benchmark of the triangle-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|triton] [--shard heads|rows]

One "step" = one forward + backward pass of fused triangle attention over one batch of
synthetic input: the headline shape B=1, H=4, L1=L2=768, D=32, bf16 (workload ``ns_l768``),
811.75 GFLOP per step by the metric's model (4*B*H*L1*L2^2*D forward, 2.5x that backward).

With N > 1 (launched by torchrun, one rank per GPU) the problem is split over the ranks and the
total work stays fixed (strong scaling). Two partitions are timed in the same run:
  heads (default, the headline ``value``): heads first, L1 rows second - ranks that own different
        heads exchange nothing; ranks that share a head all-reduce its float32 dBias among themselves;
  rows  (``rows_only`` in the line; the headline with ``--shard rows``): every rank owns a block of
        L1 rows of ALL heads and the float32 dBias (B,H,L2,L2) is all-reduced among all N ranks.
The value is whole-problem FLOPs / max-over-ranks device time.

Prints ONE JSON line on rank 0. ``--impl reference`` times the reference project's own CPU path
(its naive PyTorch function from baseline/_ref, else the CPU restatement in oracle/) on the host
cores, rank 0 only. ``--impl triton`` times the reference's Triton kernels beside this library on
one GPU at the fp16 shapes they can run; the default N = 1 run carries the same table as
``triton_ref``.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

os.environ.setdefault("TRITON_ALLOW_NON_CONSTEXPR_GLOBALS", "1")  # the reference's module needs it (Triton >= 3)

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "flash-triangle-attention_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402

WORKLOAD = "ns_l768"
METRIC = "fwd+bwd TFLOP/s, fused triangle attention B=1 H=4 L=768 D=32 bf16"
# DRAM bytes (read + write) of ONE launch of the backward kernel at the full workload on one GPU,
# from the one-pass ncu capture of that launch (dram__bytes_read.sum + dram__bytes_write.sum,
# profiles/bwd_kernel_ns_l768_dram.md); a rank that owns a fraction of the rows and heads moves that
# fraction of it.
BWD_KERNEL_DRAM_BYTES = 1152078848 + 1059723264
# L1 rows per block of the end-to-end leg (host tensors streamed through the GPU)
E2E_BLOCK_ROWS = int(os.environ.get("FTA_E2E_BLOCK_ROWS", "96"))


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured (burst)"
    return 1590.0, 6650.0, "fallback"


try:
    _ALL_CORES = os.sched_getaffinity(0)  # before any binding to the GPU's NUMA node
except AttributeError:
    _ALL_CORES = None


def host_cores() -> int:
    """Cores this process may use; the CPU arm runs on all of them (the GPU arm's NUMA binding undone)."""
    if _ALL_CORES is None:
        return os.cpu_count() or 1
    try:
        os.sched_setaffinity(0, _ALL_CORES)
    except OSError:
        pass
    return len(os.sched_getaffinity(0))


def base_config(world: int, shard: str) -> dict:
    """The description of the workload, identical for every arm at the same N and partition."""
    import workloads
    w = workloads.WORKLOADS[WORKLOAD]
    return {"workload": WORKLOAD, "B": w.B, "H": w.H, "L1": w.L1, "L2": w.L2, "D": w.D, "n_gpus": world,
            "shard": shard, "l2": "flushed between steps (256 MB write outside the events)"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc, self.first = index, [], None, 0

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

    def wait_first_sample(self, timeout_s=3.0):
        """nvidia-smi takes a good part of a second to initialise (and perturbs launches while it does):
        callers start it ahead of the warm-up and begin timing once it delivers samples."""
        t0 = time.perf_counter()
        while self.proc is not None and not self.rows and time.perf_counter() - t0 < timeout_s:
            time.sleep(0.02)

    def mark_region_start(self):
        self.first = len(self.rows)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = self.rows[self.first:] or self.rows  # samples taken from the start of the timed region on
        sm = [float(r[1]) for r in rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v == "Active"})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# --------------------------------------------------------------------------------------------
# CPU arm: the reference's own CPU path on the host cores
# --------------------------------------------------------------------------------------------
def _available_host_bytes() -> int:
    try:
        import psutil
        return int(psutil.virtual_memory().available)
    except Exception:
        return 0


def cpu_naive_sample():
    """The reference project's own CPU path, once: its naive function ``reference_tt_attn``
    (flash_tt_attn.py:845-864, taken unmodified from baseline/_ref) with torch autograd, float32, all
    host threads, on ONE of the workload's heads - the function needs L1 == L2 and materialises the
    (L,L,L) logits, so a head is the smallest sample of the workload it can run. None when the copy of
    the reference is absent or the host lacks the memory for about ten logits-sized tensors."""
    import workloads
    import ref_compare
    w = workloads.WORKLOADS[WORKLOAD]
    cores = host_cores()
    need = 10 * 4 * w.L2 * w.L2 * w.L2
    if not (ref_compare.available() and w.L1 == w.L2 and _available_host_bytes() > need + (8 << 30)):
        return None
    import torch
    torch.set_num_threads(cores)
    fn = ref_compare.load_naive_fn()
    g = torch.Generator().manual_seed(w.seed)
    L, D = w.L2, w.D
    q, k, v = (torch.randn(1, 1, L, L, D, generator=g).requires_grad_() for _ in range(3))
    do = torch.randn(1, 1, L, L, D, generator=g)
    b = torch.randn(1, 1, L, L, generator=g).requires_grad_()
    t0 = time.perf_counter()
    o = fn(q, k, v, b, w.sm_scale)
    o.backward(do)
    t = time.perf_counter() - t0
    flops = 3.5 * 4.0 * L * L * L * D
    return {"value": flops / t / 1e12, "cores": cores, "kind": "reference", "seconds": t,
            "sample": f"1 of {w.H} heads of {WORKLOAD} (B1 H1 L{L} D{D}), the reference's own reference_tt_attn "
                      f"+ torch autograd, float32, fwd+bwd, {cores} threads"}


def cpu_port_sample(target_seconds=12.0):
    """The numpy/BLAS restatement of the reference's naive path (oracle/) on the first rows of every
    head, sized to about ``target_seconds``, all host threads (set explicitly: a launcher's
    OMP_NUM_THREADS=1 must not shrink it)."""
    import contextlib
    import workloads
    from oracle import tt_attn_oracle as npo
    w = workloads.WORKLOADS[WORKLOAD]
    cores = host_cores()
    try:
        from threadpoolctl import threadpool_limits
        limiter = threadpool_limits(limits=cores)
    except Exception:
        limiter = contextlib.nullcontext()
    rng = np.random.Generator(np.random.PCG64(w.seed))

    def sample(rows):
        sh = (w.B, w.H, rows, w.L2, w.D)
        q, k, v, do = (rng.standard_normal(sh, dtype=np.float32) for _ in range(4))
        bias = rng.standard_normal((w.B, w.H, w.L2, w.L2), dtype=np.float32)
        t0 = time.perf_counter()
        npo.forward_backward(q, k, v, bias, do, w.sm_scale)
        return time.perf_counter() - t0

    with limiter:
        sample(1)  # warm-up (BLAS thread pool, page faults)
        t2 = sample(2)
        rows = int(max(2, min(w.L1, round(2 * target_seconds / max(t2, 1e-4)))))
        t = sample(rows)
    flops = 3.5 * 4.0 * w.B * w.H * rows * w.L2 * w.L2 * w.D
    return {"value": flops / t / 1e12, "cores": cores, "kind": "port", "seconds": t,
            "sample": f"{rows} of {w.L1} L1 rows x {w.H} heads of {WORKLOAD}, float32 numpy/BLAS restatement of the "
                      f"reference's naive path, fwd+bwd, {cores} threads"}


# A sample of the reference's own function is one whole head (it cannot run less); where that takes
# longer than this, the timed steps use the restatement instead and the one probe is reported beside
# them, so that a run of K steps stays within minutes.
NAIVE_STEP_LIMIT_S = 6.0


def cpu_reference_rate(target_seconds=12.0):
    """The CPU baseline of the N = 1 line: (sample dict, probe dict or None)."""
    probe = cpu_naive_sample()
    if probe is not None and probe["seconds"] <= NAIVE_STEP_LIMIT_S:
        return probe, probe
    return cpu_port_sample(target_seconds), probe


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    probe = cpu_naive_sample()
    use_naive = probe is not None and probe["seconds"] <= NAIVE_STEP_LIMIT_S
    vals, secs, last = [], [], None
    for it in range(args.warmup + args.steps):
        last = cpu_naive_sample() if use_naive else cpu_port_sample(target_seconds=3.0)
        if it >= args.warmup:
            vals.append(last["value"])
            secs.append(last["seconds"])
    value = float(np.mean(vals))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.mean(secs)) * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": base_config(args.gpus, args.shard),
        "note": "the reference's CPU path on the host cores; each step is a bounded sample of the workload",
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": last["cores"], "kind": last["kind"],
                         "sample": last["sample"]},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if probe is not None:
        line["reference_fn_probe"] = {"value": probe["value"], "unit": "TFLOP/s", "seconds": probe["seconds"],
                                      "sample": probe["sample"], "used_for_steps": use_naive}
    print(json.dumps(line), flush=True)
    return 0


# --------------------------------------------------------------------------------------------
# Triton arm: the reference's GPU kernels beside this library (one GPU, fp16 shapes they can run)
# --------------------------------------------------------------------------------------------
def triton_table(steps=10, warmup=3):
    import ref_compare
    if not ref_compare.available():
        return {"unavailable": "baseline/_ref/flash_tt_attn.py (copy of the reference module) is not staged"}
    try:
        import flash_tt_attn as fta
        rows = ref_compare.compare_with_triton(fta.attention, steps=steps, warmup=warmup)
        fta.check_device_status()
        return {"timing": "autograd calls, CUDA events, L2 flushed between calls, same tensors for both", "cases": rows}
    except Exception as e:  # the comparator must never take the bench line down with it
        return {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}


def run_triton_arm(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    import torch
    torch.cuda.set_device(0)
    line = {"impl": "triton", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "triton_ref": triton_table(steps=max(1, min(args.steps, 20)), warmup=max(3, args.warmup))}
    print(json.dumps(line), flush=True)
    return 0


def bind_to_gpu_numa_node(dev_index: int):
    """Run this process on the CPU cores next to the GPU (its PCIe root's NUMA node), so that the
    pinned host buffers it allocates from here on are placed there (first touch). Best effort."""
    try:
        import torch
        p = torch.cuda.get_device_properties(dev_index)
        bus = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        cpus = open(f"/sys/bus/pci/devices/{bus}/local_cpulist").read().strip()
        want = set()
        for part in cpus.split(","):
            a, _, b = part.partition("-")
            want.update(range(int(a), int(b or a) + 1))
        allowed = os.sched_getaffinity(0)
        pick = want & allowed
        if pick and pick != allowed:
            os.sched_setaffinity(0, pick)
            return f"cores {cpus}"
        return "all allowed cores are local" if pick else "no local core allowed"
    except Exception as e:
        return f"not bound ({type(e).__name__})"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "triton"])
    ap.add_argument("--shard", default="heads", choices=["heads", "rows"],
                    help="multi-GPU partition of the headline value (the other one is reported beside it)")
    ap.add_argument("--dbias-sum", default="auto", choices=["auto", "nccl", "peer"],
                    help="ranks that share a head sum dBias with an NCCL all-reduce + cast, or with "
                         "fta_dbias_sum_peers_sync / _sliced over NVLink peer memory (auto: peer memory where symmetric memory works)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--no-triton", action="store_true", help="skip the reference-Triton comparison table")
    ap.add_argument("--rows", type=int, default=0,
                    help="restrict the workload to its first ROWS L1 rows (a small case for ncu captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.impl == "triton":
        return run_triton_arm(args)

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
    numa = bind_to_gpu_numa_node(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(3, args.warmup)

    w = workloads.WORKLOADS[WORKLOAD]
    if args.rows > 0:
        w = w.with_rows(min(args.rows, w.L1))
    dt = torch.bfloat16
    L = _cabi.lib()
    x_full = workloads.make_inputs(w)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2
    stream = torch.cuda.current_stream().cuda_stream
    scale = w.sm_scale
    flops_step = w.flops_fwd() + w.flops_bwd()  # whole problem, all ranks

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # every rank takes part in the creation of every subgroup; one set per group size
    subgroups = {}

    def group_for(peers):
        n = len(peers)
        if world == 1 or n == 1:
            return None
        if n == world:
            return dist.group.WORLD
        if n not in subgroups:
            mine = None
            for g0 in range(0, world, n):
                g_ = dist.new_group(list(range(g0, g0 + n)))
                if g0 <= rank < g0 + n:
                    mine = g_
            subgroups[n] = mine
        return subgroups[n]

    def partition(mode):
        """(heads slice, rows slice, process group or None) of this rank under the partition `mode`."""
        if mode == "rows":
            return slice(0, w.H), fta.shard_rows(w.L1, rank, world), group_for(list(range(world)))
        heads, rows, peers = fta.shard_plan(w.H, w.L1, rank, world)
        return heads, rows, group_for(peers)

    def time_partition(mode, steps, sample_clocks):
        heads, rows, grp = partition(mode)
        nrows = rows.stop - rows.start
        host = {k: torch.from_numpy(np.ascontiguousarray(x_full[k][:, heads, rows] if k != "bias" else
                                                          x_full[k][:, heads])).to(dt).pin_memory()
                for k in ("q", "k", "v", "do", "bias")}
        d = {k: v.to(dev) for k, v in host.items()}
        B, H, L2, D = w.B, heads.stop - heads.start, w.L2, w.D  # H: heads of this rank
        prob = FtaProblem(B, H, nrows, L2, D, _cabi.FTA_BF16)
        o, o_res = torch.empty_like(d["q"]), torch.empty_like(d["q"])
        lse = torch.empty(3, B, H, nrows, L2, dtype=torch.float32, device=dev)
        delta = torch.empty(B, H, nrows, L2, dtype=torch.float32, device=dev)
        dq, dk, dv = (torch.empty_like(d["q"]) for _ in range(3))
        db = torch.empty_like(d["bias"])
        db32 = torch.empty(B, H, L2, L2, dtype=torch.float32, device=dev)
        ws_bytes = int(L.fta_bwd_workspace_bytes(prob))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        sharded = grp is not None
        # how the ranks of a group sum dBias. auto / peer: over NVLink peer memory - a pair with one launch
        # per rank (line-up, the other rank's partial read, sum, rounding), larger groups with the sliced
        # kernel (each rank sums 1/R and stores the result into every rank's buffer; 8 ranks: 0.080 ms
        # against 0.097 for NCCL all-reduce + cast, 4 ranks: equal). nccl: the library collective, also the
        # fallback where symmetric memory is unavailable.
        peer = None
        if sharded and args.dbias_sum in ("peer", "auto"):
            try:
                peer = fta.PeerDbiasSum(db32.shape, grp, dev, dt)
            except Exception as e:  # symmetric memory unavailable: the all-reduce does it
                if args.dbias_sum == "peer":
                    raise
                print(f"[bench] peer-memory dBias sum unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)

        # argument structs built once: at N = 8 a step is 0.45 ms of GPU time and the host has to keep up
        T = {k: t5(d[k]) for k in ("q", "k", "v", "do")}
        T.update(o=t5(o), dq=t5(dq), dk=t5(dk), dv=t5(dv), bias=t4(d["bias"]))
        p_ores, p_lse, p_delta, p_status = o_res.data_ptr(), lse.data_ptr(), delta.data_ptr(), status.data_ptr()
        p_db32, p_db, p_ws = db32.data_ptr(), db.data_ptr(), ws.data_ptr()
        n_db, sm_scale = db32.numel(), float(scale)

        def step(ef=None, marks=None):
            """One pass. `ef`: event recorded after the forward. `marks`: dict that receives an event after
            every call (the per-launch diagnostic loop below; never used in the timed region)."""
            def mark(name):
                if marks is not None:
                    marks[name] = torch.cuda.Event(enable_timing=True)
                    marks[name].record()
            mark("start")
            _cabi.check(L.fta_forward(prob, T["q"], T["k"], T["v"], T["bias"], sm_scale, T["o"], p_ores, p_lse, p_status,
                                      stream), "fta_forward")
            if ef is not None:
                ef.record()
            mark("forward")
            _cabi.check(L.fta_bwd_preprocess(prob, T["o"], p_ores, T["do"], p_delta, stream), "fta_bwd_preprocess")
            mark("preprocess")
            _cabi.check(L.fta_backward(prob, T["q"], T["k"], T["v"], T["bias"], T["do"], p_lse, p_delta, sm_scale,
                                       T["dq"], T["dk"], T["dv"], peer.partial_ptr() if peer else p_db32,
                                       None if sharded else p_db, p_ws, ws_bytes, p_status, stream), "fta_backward")
            mark("backward")
            if peer:
                # barrier between the ranks + one kernel: sum in rank order, round (+ a second barrier
                # where the result is stored into the peers' buffers)
                if peer.sliced:
                    peer.reduce_sliced(stream)
                else:
                    peer.reduce(db, None, stream)
                mark("allreduce")
                mark("cast")
            elif sharded:
                dist.all_reduce(db32, group=grp)
                mark("allreduce")
                _cabi.check(L.fta_dbias_cast(p_db32, p_db, n_db, prob.dtype, stream), "fta_dbias_cast")
                mark("cast")

        # the clock sampler starts before the warm-up: its start-up is over when the timed region begins
        sampler = ClockSampler(local) if (sample_clocks and rank == 0) else None
        if sampler:
            sampler.start()
            sampler.wait_first_sample()
        for _ in range(warmup):
            step()
        barrier()
        # ---- timed region: K steps, each bracketed by CUDA events on the launching stream; L2 is
        # flushed (a 256 MB write) between steps, outside the events. The host only enqueues: events
        # are read after the loop, so the GPU always has the next launches queued.
        if sampler:
            sampler.mark_region_start()
        barrier()
        wall0 = time.perf_counter()
        evs = []
        for _ in range(steps):
            flush.zero_()
            e0, e1, ef, k0, k1 = (torch.cuda.Event(enable_timing=True) for _ in range(5))
            k0.record()  # creates the underlying cudaEvent_t handles (re-recorded inside fta_backward)
            k1.record()
            L.fta_profile_backward_kernel(k0.cuda_event, k1.cuda_event)
            e0.record()
            step(ef)
            e1.record()
            evs.append((e0, e1, ef, k0, k1))
        torch.cuda.synchronize()
        step_ms = [e0.elapsed_time(e1) for e0, e1, ef, k0, k1 in evs]
        fwd_ms = [e0.elapsed_time(ef) for e0, e1, ef, k0, k1 in evs]
        bwdk_ms = [k0.elapsed_time(k1) for e0, e1, ef, k0, k1 in evs]
        barrier()
        wall = time.perf_counter() - wall0
        # ---- per-launch diagnostic loop (outside the timed region): an event after every call, and the
        # two events fta_backward records around its main kernel split that call into bias transposition
        # + zero fill / kernel / dQ + dBias finalise. Events between launches cost a little, so the sum
        # can exceed ms_per_step.
        diag_rows = []
        for _ in range(min(10, steps)):
            flush.zero_()
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k0.record()
            k1.record()
            L.fta_profile_backward_kernel(k0.cuda_event, k1.cuda_event)
            marks = {}
            step(None, marks)
            diag_rows.append((marks, k0, k1))
        torch.cuda.synchronize()
        L.fta_profile_backward_kernel(None, None)
        def _ms(a, b):
            return float(np.mean([m[a].elapsed_time(m[b]) for m, _k0, _k1 in diag_rows]))
        launch_ms = {
            "forward": _ms("start", "forward"),
            "preprocess": _ms("forward", "preprocess"),
            "bwd_prologue": float(np.mean([m["preprocess"].elapsed_time(k0) for m, k0, k1 in diag_rows])),
            "bwd_kernel": float(np.mean([k0.elapsed_time(k1) for m, k0, k1 in diag_rows])),
            "bwd_epilogue": float(np.mean([k1.elapsed_time(m["backward"]) for m, k0, k1 in diag_rows])),
        }
        if sharded:
            launch_ms["dbias_allreduce"] = _ms("backward", "allreduce")
            launch_ms["dbias_cast"] = _ms("allreduce", "cast")
        launch_ms = {k: round(v, 4) for k, v in launch_ms.items()}
        barrier()
        clocks = sampler.stop() if sampler else None
        if int(status.item()) != 0:
            raise SystemExit(f"device status 0x{int(status.item()):x}: a bounded device-side wait ran out")
        t = torch.tensor([float(np.sum(step_ms))], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
        return {"value": flops_step * steps / (total_ms * 1e-3) / 1e12, "ms_per_step": total_ms / steps,
                "fwd_ms": float(np.mean(fwd_ms)), "bwd_kernel_ms": float(np.mean(bwdk_ms)), "clocks": clocks,
                "wall_ms_per_step_incl_flush": wall / steps * 1e3, "heads_per_gpu": H, "rows_per_gpu": nrows,
                "allreduce_ranks": 1 if grp is None else dist.get_world_size(grp),
                "launches_per_step": 5 + (1 if sharded else 0),  # fwd, preprocess, bwd prologue / kernel / epilogue (+ cast or peer sum)
                "dbias_sum": "none" if not sharded else (("peer memory (fta_dbias_sum_peers_sliced_sync)" if peer.sliced else "peer memory (fta_dbias_sum_peers_sync: one launch)") if peer else "nccl all-reduce + cast"),
                "launch_ms": launch_ms,
                "host": host, "grp": grp}

    main_res = time_partition(args.shard, args.steps, True)
    other = None
    if world > 1:
        other_mode = "rows" if args.shard == "heads" else "heads"
        other = time_partition(other_mode, max(5, args.steps // 2), False)
        other = {k: other[k] for k in ("value", "ms_per_step", "fwd_ms", "bwd_kernel_ms", "launch_ms", "allreduce_ranks", "dbias_sum",
                                       "heads_per_gpu", "rows_per_gpu")}
        other["shard"] = other_mode

    # ---- end to end through the public API with HOST buffers: pinned inputs copied to the device,
    # attention + backward, outputs and gradients copied back, every step.
    host, grp = main_res["host"], main_res["grp"]
    e2e = None
    if not args.no_e2e:
        e2e_steps = max(1, min(args.steps, 10))
        out_host = {k: torch.empty_like(host["q"]).pin_memory() for k in ("o", "dq", "dk", "dv")}
        out_host["dbias"] = torch.empty_like(host["bias"]).pin_memory()
        h2d = sum(v.numel() * v.element_size() for v in host.values())
        d2h = sum(v.numel() * v.element_size() for v in out_host.values())

        def e2e_step():
            # the library's host-memory entry point: blocks of L1 rows double-buffered through the GPU,
            # copies in / kernels / copies out on three streams
            fta.attention_fwd_bwd_streamed(host, scale, out_host, block_rows=E2E_BLOCK_ROWS, device=dev, group=grp)

        def measure_e2e():
            for _ in range(3):  # untimed: first touches of the pinned buffers, allocator, streams
                e2e_step()
            barrier()
            ms = []
            for _ in range(e2e_steps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                e2e_step()
                e1.record()
                torch.cuda.synchronize()
                ms.append(e0.elapsed_time(e1))
            barrier()
            te = torch.tensor([float(np.sum(ms))], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(te, op=dist.ReduceOp.MAX)
            return ms, float(te.item()) / e2e_steps

        e2e_ms, e2e_ms_step = measure_e2e()
        # the bound of this leg: the same pinned buffers copied in and out at the same time with
        # nothing else going on (two streams, whole tensors)
        dbuf = {k: torch.empty_like(v, device=dev) for k, v in host.items()}
        sbuf = {k: torch.empty_like(v, device=dev) for k, v in out_host.items()}
        s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

        def copy_ms(do_in, do_out):
            best = 1e30
            for _ in range(3):
                torch.cuda.synchronize()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record()
                s1.wait_event(a0)
                s2.wait_event(a0)
                if do_in:
                    with torch.cuda.stream(s1):
                        for k in host:
                            dbuf[k].copy_(host[k], non_blocking=True)
                if do_out:
                    with torch.cuda.stream(s2):
                        for k in out_host:
                            out_host[k].copy_(sbuf[k], non_blocking=True)
                torch.cuda.current_stream().wait_stream(s1)
                torch.cuda.current_stream().wait_stream(s2)
                a1.record()
                torch.cuda.synchronize()
                best = min(best, a0.elapsed_time(a1))
            return best

        t_in, t_out, t_both = copy_ms(True, False), copy_ms(False, True), copy_ms(True, True)
        # The host side of this leg (a shared machine: PCIe root, driver locks, host cores) now and then
        # runs whole calls at 70-100 ms where 15 ms is normal, with the copy bound measured right after
        # at its usual value. A leg that far off its own bound is taken once more and both are reported.
        e2e_first = None
        flag = torch.tensor([1.0 if e2e_ms_step > 2.5 * t_both else 0.0], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        if float(flag.item()) > 0:
            e2e_first = e2e_ms_step
            e2e_ms, e2e_ms_step = measure_e2e()
        e2e = {"value": flops_step / (e2e_ms_step * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(d2h), "steps": e2e_steps, "ms_per_step": e2e_ms_step,
               # this rank's median beside the mean: the host link is shared, single steps of 25-28 ms occur
               "ms_per_step_median": float(np.median(e2e_ms)),
               "first_attempt_ms_per_step": e2e_first,  # not None: the leg was re-measured once (see bench.py)
               "h2d_only_gbs": h2d / t_in / 1e6, "d2h_only_gbs": d2h / t_out / 1e6,
               "copy_bound_ms": t_both, "frac_of_copy_bound": t_both / e2e_ms_step,
               "note": "per rank: its shard of q,k,v,dO + bias in, o,dq,dk,dv + dbias out; copy_bound_ms = the same "
                       "buffers copied both ways at once with no kernels", "host_numa": numa}
        fta.check_device_status(dev)

    if rank == 0:
        peak_tf, peak_gbs, peak_kind = _peaks()
        r = main_res
        bwd_flops_rank = 2.5 * 4.0 * w.B * r["heads_per_gpu"] * r["rows_per_gpu"] * w.L2 * w.L2 * w.D
        achieved = bwd_flops_rank / (r["bwd_kernel_ms"] * 1e-3) / 1e12
        share = r["heads_per_gpu"] * r["rows_per_gpu"] / float(workloads.WORKLOADS[WORKLOAD].H *
                                                                workloads.WORKLOADS[WORKLOAD].L1)
        cfg = base_config(world, args.shard)
        if args.rows > 0:
            cfg["workload"] = f"{WORKLOAD}[first {w.L1} rows]"
            cfg["L1"] = w.L1
        line = {
            "metric": METRIC, "value": r["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg,
            "detail": {"heads_per_gpu": r["heads_per_gpu"], "rows_per_gpu": r["rows_per_gpu"],
                       "dbias_allreduce_ranks": r["allreduce_ranks"], "dbias_sum": r["dbias_sum"], "fwd_ms": r["fwd_ms"],
                       "bwd_kernel_ms": r["bwd_kernel_ms"], "launch_ms": r["launch_ms"],
                       "frac_of_bf16_peak": r["value"] / (peak_tf * world),
                       "peak": f"{peak_tf} TFLOP/s {peak_kind}",
                       "wall_ms_per_step_incl_flush": r["wall_ms_per_step_incl_flush"]},
            "e2e": e2e if e2e is not None else {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                                                "d2h_bytes_per_step": 0, "note": "skipped (--no-e2e)"},
            "gpu_launches": r["launches_per_step"] * args.steps,
            "clocks": r["clocks"],
            "roofline": {"kernel": "fta_bwd_kernel", "bound": "tensor", "achieved": achieved, "peak": peak_tf,
                         "unit": "TFLOP/s", "frac": achieved / peak_tf, "traffic": int(BWD_KERNEL_DRAM_BYTES * share),
                         "peak_kind": peak_kind},
        }
        if other is not None:
            line["rows_only" if other["shard"] == "rows" else "heads_first"] = other
        if world == 1 and not args.no_cpu_baseline:
            c, probe = cpu_reference_rate()
            line["cpu_baseline"] = {"value": c["value"], "unit": "TFLOP/s", "cores": c["cores"], "kind": c["kind"],
                                    "sample": c["sample"]}
            if probe is not None and probe is not c:
                line["cpu_baseline"]["reference_fn_probe"] = {"value": probe["value"], "seconds": probe["seconds"],
                                                              "sample": probe["sample"]}
        if world == 1 and not args.no_triton and args.rows <= 0:
            line["triton_ref"] = triton_table()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
