"""Seeded synthetic workloads for triangle attention.

The reference measures on ``torch.randn`` tensors (flash_tt_attn.py:779-783) and tests on
``normal_(0, 0.5)`` tensors (flash_tt_attn.py:677-682); no dataset is involved. The
workloads below are synthetic stand-ins with the shapes, value distributions and seeds of
the benchmark configurations (pair-stack crops of a structure-prediction model).

Values are drawn on the host with numpy's PCG64 in the fixed order q, k, v, dO, bias
(, mask) in float32; callers round them ONCE to the dtype under test and hand the same
rounded values to the kernels and to the checker.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class Workload:
    name: str
    B: int
    H: int
    L1: int
    L2: int
    D: int
    dtype: str  # "fp32" | "fp16" | "bf16"
    seed: int
    qkv_std: float = 1.0
    bias_std: float = 1.0
    mask_frac: float = 0.0  # Bernoulli fraction of key columns masked with -1e9
    backward: bool = True

    @property
    def sm_scale(self) -> float:
        return 1.0 / math.sqrt(self.D)

    def flops_fwd(self) -> float:
        return 4.0 * self.B * self.H * self.L1 * self.L2 * self.L2 * self.D

    def flops_bwd(self) -> float:
        return 2.5 * self.flops_fwd()

    def with_rows(self, L1: int) -> "Workload":
        """Same workload restricted to ``L1`` rows (a shard of the L1 axis)."""
        return Workload(self.name, self.B, self.H, L1, self.L2, self.D, self.dtype, self.seed,
                        self.qkv_std, self.bias_std, self.mask_frac, self.backward)


# The benchmark configurations, by the names used in the documentation.
WORKLOADS = {
    # CPU-runnable case of the naive path
    "c1_cpu_l64": Workload("c1_cpu_l64", 1, 4, 64, 64, 32, "fp32", 0),
    # README benchmark shape of the reference
    "c2_readme_l256": Workload("c2_readme_l256", 4, 8, 256, 256, 32, "fp16", 1),
    # pair-stack crop with 10 % masked key columns
    "c3_crop_l384": Workload("c3_crop_l384", 1, 4, 384, 384, 32, "bf16", 2, mask_frac=0.1),
    # large-complex inference, forward only; std 1/sqrt(D) for q,k,v, std 2 for the bias
    "c4_infer_l1024": Workload("c4_infer_l1024", 1, 4, 1024, 1024, 32, "bf16", 3,
                               qkv_std=1.0 / math.sqrt(32.0), bias_std=2.0, backward=False),
    # long-sequence training
    "c5_train_l2048": Workload("c5_train_l2048", 1, 8, 2048, 2048, 64, "bf16", 4),
    # the headline metric's shape
    "ns_l768": Workload("ns_l768", 1, 4, 768, 768, 32, "bf16", 0),
}


def make_inputs(w: Workload, rows: slice | None = None) -> dict:
    """Draw q, k, v, dO (B,H,L1,L2,D) and bias (B,H,L2,L2) as float32 numpy arrays.

    ``rows`` restricts the returned q, k, v, dO to a slice of the L1 axis (the values are
    those of the full tensor; the generator always draws the full tensors so that a shard
    sees the same numbers as the unsharded run). The mask, if any, is shared by all query
    rows and all heads of a batch element and is already folded into ``bias``.
    """
    rng = np.random.Generator(np.random.PCG64(w.seed))
    shape = (w.B, w.H, w.L1, w.L2, w.D)
    out = {}
    for name in ("q", "k", "v"):
        out[name] = (rng.standard_normal(shape, dtype=np.float32) * np.float32(w.qkv_std))
    out["do"] = rng.standard_normal(shape, dtype=np.float32)
    bias = rng.standard_normal((w.B, w.H, w.L2, w.L2), dtype=np.float32) * np.float32(w.bias_std)
    if w.mask_frac > 0.0:
        masked = rng.random((w.B, 1, 1, w.L2)) < w.mask_frac
        masked[..., 0] = False  # never mask every key of a row
        bias = bias + np.where(masked, np.float32(-1e9), np.float32(0.0)).astype(np.float32)
        out["mask"] = masked
    out["bias"] = bias.astype(np.float32)
    if rows is not None:
        for name in ("q", "k", "v", "do"):
            out[name] = np.ascontiguousarray(out[name][:, :, rows])
    return out
