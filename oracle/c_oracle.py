"""Build and call the plain-C oracle (tt_attn_oracle.c). TEST INFRASTRUCTURE only.

``build()`` compiles the C restatement next to its source with gcc + OpenMP; ``load()``
binds it with ctypes. The arrays handed over are float32, C-contiguous.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "tt_attn_oracle.c")
_LIB = os.path.join(_HERE, "libtt_attn_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    if (not force) and os.path.exists(_LIB) and os.path.getmtime(_LIB) >= os.path.getmtime(_SRC):
        return _LIB
    cmd = ["gcc", "-O3", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", "-o", _LIB, _SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return _LIB


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB):
            build()
        lib = ctypes.CDLL(_LIB)
        fp = ctypes.POINTER(ctypes.c_float)
        lib.tt_oracle_forward.argtypes = [fp, fp, fp, fp] + [ctypes.c_int] * 5 + [ctypes.c_float, fp, fp]
        lib.tt_oracle_forward.restype = ctypes.c_int
        lib.tt_oracle_forward_backward.argtypes = (
            [fp] * 5 + [ctypes.c_int] * 5 + [ctypes.c_float] + [fp] * 5
        )
        lib.tt_oracle_forward_backward.restype = ctypes.c_int
        lib.tt_oracle_num_threads.restype = ctypes.c_int
        _lib = lib
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def num_threads() -> int:
    return int(load().tt_oracle_num_threads())


def forward(q, k, v, bias, sm_scale, return_lse=False):
    lib = load()
    q, k, v, bias = _f32(q), _f32(k), _f32(v), _f32(bias)
    B, H, L1, L2, D = q.shape
    assert bias.shape == (B, H, L2, L2)
    o = np.empty_like(q)
    lse = np.empty((B, H, L1, L2), dtype=np.float32)
    rc = lib.tt_oracle_forward(_p(q), _p(k), _p(v), _p(bias), B, H, L1, L2, D, float(sm_scale), _p(o), _p(lse))
    if rc != 0:
        raise RuntimeError(f"tt_oracle_forward failed: {rc}")
    return (o, lse) if return_lse else o


def forward_backward(q, k, v, bias, do, sm_scale):
    lib = load()
    q, k, v, bias, do = _f32(q), _f32(k), _f32(v), _f32(bias), _f32(do)
    B, H, L1, L2, D = q.shape
    o, dq, dk, dv = (np.empty_like(q) for _ in range(4))
    dbias = np.empty((B, H, L2, L2), dtype=np.float32)
    rc = lib.tt_oracle_forward_backward(
        _p(q), _p(k), _p(v), _p(bias), _p(do), B, H, L1, L2, D, float(sm_scale),
        _p(o), _p(dq), _p(dk), _p(dv), _p(dbias))
    if rc != 0:
        raise RuntimeError(f"tt_oracle_forward_backward failed: {rc}")
    return {"o": o, "dq": dq, "dk": dk, "dv": dv, "dbias": dbias}


if __name__ == "__main__":
    print(build(force=True))
