#!/usr/bin/env python
"""Sequence-length sweep of fused triangle attention, in the format of the reference's own sweep.

The reference benchmarks B=4, H=8, D=32, L = 2^4 .. 2^12, forward and backward, latency (ms) and
peak memory (GB), and writes one CSV per (mode, metric) named
``fused-attention-batch{B}-head{H}-d{D}-{mode}-{latency|memory}.csv`` with the columns
``L,<fused>,Vanilla PyTorch`` (flash_tt_attn.py:714-843, test_results/*.csv). This script writes
the same files for this library so that B200 curves can be laid over the published ones:

    python flash-triangle-attention_b200/sweep.py --out sweep_out [--dtype bf16|fp16] [--dim 32|64] [--lmax 2048]

Lengths that are not a multiple of 128 run natively (ragged blocks are padded by the tile loads).
The vanilla column is the naive PyTorch statement of the op on the same GPU, skipped (empty cell)
when its (B,H,L,L,L) logits would not fit in ``--vanilla-gb`` of memory. With ``--dtype fp16`` and
a copy of the reference under baseline/_ref a third column, ``Triton [FP16]`` (the reference's own
header), holds the reference's Triton kernels on the same GPU for the lengths they can run
(forward: L a multiple of 128; backward: L a power of two >= 128; empty elsewhere - its published
L < 128 rows read out of bounds or launch an empty grid, flash_tt_attn.py:618, 644). "bwd" times the
backward pass only (forward outside the timed region), as the reference does.
"""
from __future__ import annotations

import argparse
import csv
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

import torch  # noqa: E402

import flash_tt_attn as fta  # noqa: E402
import ref_compare  # noqa: E402


def _time_ms(fn, reps, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        flush.zero_()  # write more than the L2 holds between repetitions
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def _measure(provider, mode, metric, B, H, L, D, dtype, reps, flush):
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(L)
    q, k, v = [torch.randn(B, H, L, L, D, device=dev, dtype=dtype, generator=g).requires_grad_(mode == "bwd")
               for _ in range(3)]
    bias = torch.randn(B, H, L, L, device=dev, dtype=dtype, generator=g).requires_grad_(mode == "bwd")
    scale = D ** -0.5
    op = {"fused": fta.attention, "vanilla": fta.reference_tt_attn}.get(provider)
    if provider == "triton":
        op = ref_compare.load_triton_module().attention
    torch.cuda.reset_peak_memory_stats()
    if mode == "fwd":
        fn = lambda: op(q, k, v, bias, scale)  # noqa: E731
    else:
        o = op(q, k, v, bias, scale)
        do = torch.randn_like(o)
        fn = lambda: o.backward(do, retain_graph=True)  # noqa: E731
    if metric == "memory":
        fn()
        torch.cuda.synchronize()
        return torch.cuda.max_memory_allocated() / 2 ** 30
    return _time_ms(fn, reps, flush)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="sweep_out")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--dim", type=int, default=32)
    ap.add_argument("--lmin", type=int, default=16)
    ap.add_argument("--lmax", type=int, default=2048)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--vanilla-gb", type=float, default=40.0)
    a = ap.parse_args()
    dtype = torch.bfloat16 if a.dtype == "bf16" else torch.float16
    os.makedirs(a.out, exist_ok=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    B, H, D = a.batch, a.heads, a.dim
    Ls = []
    L = a.lmin
    while L <= a.lmax:
        Ls.append(L)
        L *= 2
    fused_name = f"B200 fused [{a.dtype.upper()}]"
    with_triton = dtype == torch.float16 and ref_compare.available()
    for mode in ("fwd", "bwd"):
        for metric in ("latency", "memory"):
            path = os.path.join(a.out, f"fused-attention-batch{B}-head{H}-d{D}-{mode}-{metric}.csv")
            with open(path, "w", newline="") as f:
                wr = csv.writer(f)
                wr.writerow(["L", fused_name, "Vanilla PyTorch"] + (["Triton [FP16]"] if with_triton else []))
                for L in Ls:
                    ours = _measure("fused", mode, metric, B, H, L, D, dtype, a.reps, flush)
                    logits_gb = B * H * L * L * L * 4 * (3 if mode == "bwd" else 2) / 2 ** 30
                    van = ""
                    if logits_gb <= a.vanilla_gb:
                        van = f"{_measure('vanilla', mode, metric, B, H, L, D, dtype, a.reps, flush):.6f}"
                    row = [f"{float(L):.6f}", f"{ours:.6f}", van]
                    if with_triton:
                        tri = ""
                        if ref_compare.triton_supports(L, L, D, dtype, mode == "bwd", B * H) is None:
                            tri = f"{_measure('triton', mode, metric, B, H, L, D, dtype, a.reps, flush):.6f}"
                        row.append(tri)
                    wr.writerow(row)
                    f.flush()
            print("wrote", path)
    fta.check_device_status()


if __name__ == "__main__":
    main()
