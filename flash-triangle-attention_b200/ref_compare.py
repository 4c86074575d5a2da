"""The reference project's own code as a comparator (benchmarks and tests only; never on the
product path).

``baseline/_ref/`` holds an unmodified copy of the reference's two Python files
(``flash_tt_attn.py``, ``example_usage.py``); it is made by ``__graft_entry__.build()`` where a
reference checkout is present, is not part of the source history, and travels with the tree.
Two things are taken from it:

* ``reference_tt_attn`` (flash_tt_attn.py:845-864), the naive PyTorch definition of the op. It is
  pure torch, so it is lifted out of the file by its AST node and runs anywhere, CPU included
  (importing the whole module needs an active Triton GPU driver, flash_tt_attn.py:115);
* the Triton path, ``attention`` (flash_tt_attn.py:554-663), by importing the module on a GPU
  machine. With Triton >= 3.0 the file only compiles with
  ``TRITON_ALLOW_NON_CONSTEXPR_GLOBALS=1`` (its ``INV_LN2`` / ``LN2`` globals, lines 38-39, are
  annotated, not constexpr instances).

What the Triton path can run, from reading its source: fp16 only (lines 99, 350, 356, 425);
``L1 == L2 == L`` (584, 616); forward for any ``L % 128 == 0`` (block pointers without boundary
checks: other L read out of bounds); backward only for L a power of two (618) and >= 128 (grid
``L // 128``, 644). ``triton_supports`` encodes exactly that, and nothing else is ever launched.
"""
from __future__ import annotations

import ast
import importlib.util
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(os.path.dirname(_HERE), "baseline", "_ref")
REF_MODULE = os.path.join(REF_DIR, "flash_tt_attn.py")
REF_EXAMPLE = os.path.join(REF_DIR, "example_usage.py")

_triton_module = None


def available() -> bool:
    return os.path.exists(REF_MODULE)


def load_naive_fn(path: str = REF_MODULE):
    """The reference's ``reference_tt_attn``, compiled from its own source text, unmodified."""
    import torch
    tree = ast.parse(open(path).read())
    node = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "reference_tt_attn")
    ns = {"torch": torch}
    exec(compile(ast.Module(body=[node], type_ignores=[]), "flash_tt_attn.py", "exec"), ns)
    return ns["reference_tt_attn"]


def triton_supports(L1: int, L2: int, D: int, dtype, backward: bool, batch_heads: int = 1) -> str | None:
    """None when the reference's Triton path can run the case, else the reason it cannot."""
    import torch
    if dtype != torch.float16:
        return "reference cannot run this case: its Triton kernels are fp16 only"
    if L1 != L2:
        return "reference cannot run this case: it needs L1 == L2"
    if D not in (32, 64, 128, 256):
        return "reference cannot run this case: no forward config for this head dimension"
    if L2 % 128 != 0:
        return "reference cannot run this case: L must be a multiple of 128 (no boundary checks)"
    if backward and (L2 & (L2 - 1)) != 0:
        return "reference cannot run this case: its backward needs L a power of two"
    if backward and batch_heads * L1 > 65535:
        # its backward launches put B*H*L1 on the y / z axis of the grid (flash_tt_attn.py:630, 644)
        return "reference cannot run this case: B*H*L1 exceeds the 65535 limit of the grid axis its backward uses"
    return None


def load_triton_module():
    """Import the reference module (GPU machine only). Its ``attention`` is the Triton path."""
    global _triton_module
    if _triton_module is not None:
        return _triton_module
    if not available():
        raise FileNotFoundError(f"{REF_MODULE} is missing (made by __graft_entry__.build() from a reference checkout)")
    os.environ.setdefault("TRITON_ALLOW_NON_CONSTEXPR_GLOBALS", "1")
    name = "reference_flash_tt_attn"
    spec = importlib.util.spec_from_file_location(name, REF_MODULE)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    _triton_module = mod
    return mod


def time_fwd_bwd(attention_fn, q, k, v, bias, do, scale, backward: bool, steps: int, warmup: int, flush):
    """Mean milliseconds per call of ``attention_fn(q, k, v, bias, scale)`` (+ ``.backward(do)``),
    through autograd, CUDA events on the current stream, ``flush`` (a buffer larger than L2) written
    between calls outside the events."""
    import torch

    def once():
        for t in (q, k, v, bias):
            t.grad = None
        if backward:
            o = attention_fn(q, k, v, bias, scale)
            o.backward(do)
        else:
            with torch.no_grad():
                attention_fn(q, k, v, bias, scale)

    for _ in range(max(1, warmup)):
        once()
    torch.cuda.synchronize()
    evs = []
    for _ in range(steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        once()
        e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    ms = [a.elapsed_time(b) for a, b in evs]
    return sum(ms) / len(ms)


# the shapes the Triton comparator is timed on (all fp16): (label, B, H, L, D, backward)
TRITON_CASES = (
    ("ns shape, forward (the reference's backward cannot run L=768)", 1, 4, 768, 32, False),
    ("B1 H4 L512, forward + backward", 1, 4, 512, 32, True),
    ("B1 H4 L1024, forward + backward", 1, 4, 1024, 32, True),
    ("c2_readme_l256, forward", 4, 8, 256, 32, False),
    ("c2_readme_l256, forward + backward", 4, 8, 256, 32, True),
)


def compare_with_triton(ours_attention, steps: int = 10, warmup: int = 3, cases=TRITON_CASES, device="cuda"):
    """Times the reference's Triton ``attention`` and ``ours_attention`` on the same fp16 tensors,
    same process, same events and L2 flush. Returns a list of dicts (one per case)."""
    import torch
    ref = load_triton_module()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    out = []
    for label, B, H, L, D, backward in cases:
        why = triton_supports(L, L, D, torch.float16, backward, B * H)
        row = {"case": label, "B": B, "H": H, "L": L, "D": D, "dtype": "fp16", "mode": "fwd+bwd" if backward else "fwd"}
        if why:
            row["unavailable"] = why
            out.append(row)
            continue
        g = torch.Generator(device=device).manual_seed(1234 + L)
        mk = lambda *s: torch.randn(*s, device=device, dtype=torch.float32, generator=g).to(torch.float16)
        q, k, v, do = (mk(B, H, L, L, D) for _ in range(4))
        bias = mk(B, H, L, L)
        for t in (q, k, v, bias):
            t.requires_grad_(backward)
        scale = D ** -0.5
        flops = 4.0 * B * H * L * L * L * D * (3.5 if backward else 1.0)
        t_ref = time_fwd_bwd(ref.attention, q, k, v, bias, do, scale, backward, steps, warmup + 1, flush)
        t_our = time_fwd_bwd(ours_attention, q, k, v, bias, do, scale, backward, steps, warmup, flush)
        row.update(triton_ms=t_ref, ours_ms=t_our, triton_tflops=flops / t_ref / 1e9, ours_tflops=flops / t_our / 1e9,
                   speedup=t_ref / t_our)
        out.append(row)
        del q, k, v, do, bias
    return out
