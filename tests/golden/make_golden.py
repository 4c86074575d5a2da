"""Generate the golden vectors that pin the CPU oracle to the reference.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

The reference module cannot be imported on a machine without a GPU (its module body asks
Triton for the active driver), so its pure-PyTorch definition of the op,
``reference_tt_attn`` (flash_tt_attn.py:845-864), is taken out of the source file by its
AST node and executed unmodified on CPU tensors; gradients come from torch autograd, as in
the reference's own ``test_op`` (flash_tt_attn.py:685-692). Inputs are the seeded numpy
draws of the cases below; only outputs are stored (``golden_*.npz``), the tests regenerate
the inputs from the seed.
"""
from __future__ import annotations

import ast
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name -> (B, H, L, D, seed, std, sm_scale, masked key columns (> 0) or masked query rows (< 0), full_outputs)
CASES = {
    "tiny_l16": (1, 2, 16, 16, 11, 1.0, 0.25, 0, True),
    "c1_cpu_l64": (1, 4, 64, 32, 0, 1.0, 1.0 / np.sqrt(32.0), 0, False),
    "testop_l32": (2, 2, 32, 32, 20, 0.5, 0.5, 0, False),  # distribution/scale of the reference's test_op
    "masked_l32": (1, 2, 32, 16, 7, 1.0, 0.25, 5, False),
    # -1e9 on whole QUERY rows (what an ending-node call makes of masked key columns): every key of
    # such a row is masked, the float32 logits lose the q.k term and the reference's answer is the
    # uniform distribution over the keys
    "maskedrows_l32": (1, 2, 32, 16, 9, 1.0, 0.25, -4, False),
}
SAMPLE_STRIDE = 37


def case_inputs(name):
    B, H, L, D, seed, std, scale, mask_cols, _ = CASES[name]
    rng = np.random.Generator(np.random.PCG64(seed))
    shape = (B, H, L, L, D)
    q = rng.standard_normal(shape, dtype=np.float32) * np.float32(std)
    k = rng.standard_normal(shape, dtype=np.float32) * np.float32(std)
    v = rng.standard_normal(shape, dtype=np.float32) * np.float32(std)
    do = rng.standard_normal(shape, dtype=np.float32)
    bias = rng.standard_normal((B, H, L, L), dtype=np.float32) * np.float32(std)
    if mask_cols > 0:
        cols = rng.choice(np.arange(1, L), size=mask_cols, replace=False)
        bias[..., cols] += np.float32(-1e9)
    elif mask_cols < 0:  # that many fully masked query rows
        rows = rng.choice(np.arange(1, L), size=-mask_cols, replace=False)
        bias[:, :, rows, :] += np.float32(-1e9)
    return q, k, v, do, bias, float(scale)


def load_reference_fn(ref_root):
    src = open(os.path.join(ref_root, "flash_tt_attn.py")).read()
    tree = ast.parse(src)
    node = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "reference_tt_attn")
    ns = {"torch": torch}
    exec(compile(ast.Module(body=[node], type_ignores=[]), "flash_tt_attn.py", "exec"), ns)
    return ns["reference_tt_attn"]


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference-checkout")
    ref_root = sys.argv[1]
    fn = load_reference_fn(ref_root)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    for name, cfg in CASES.items():
        q, k, v, do, bias, scale = case_inputs(name)
        tq, tk, tv, tb = (torch.from_numpy(a.copy()).requires_grad_() for a in (q, k, v, bias))
        out = fn(tq, tk, tv, tb, scale)
        out.backward(torch.from_numpy(do))
        res = {"o": out.detach().numpy(), "dq": tq.grad.numpy(), "dk": tk.grad.numpy(),
               "dv": tv.grad.numpy(), "dbias": tb.grad.numpy()}
        store = {}
        for key, arr in res.items():
            flat = arr.reshape(-1).astype(np.float32)
            if cfg[-1]:
                store[key] = arr.astype(np.float32)
            else:
                store[key + "_sample"] = flat[::SAMPLE_STRIDE].copy()
            store[key + "_sum"] = np.float64(flat.astype(np.float64).sum())
            store[key + "_sumsq"] = np.float64((flat.astype(np.float64) ** 2).sum())
        path = os.path.join(HERE, f"golden_{name}.npz")
        np.savez_compressed(path, **store)
        print(name, {k2: (v2.shape if hasattr(v2, "shape") else v2) for k2, v2 in store.items()},
              os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
