"""ctypes binding of libfta.so (the C ABI declared in include/fta.h).

The library is required: importing this module on a machine where libfta.so has not been
built raises immediately, and there is no CPU or framework fallback behind it.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfta.so")

FTA_FP16, FTA_BF16 = 0, 1


class FtaProblem(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("H", ctypes.c_int32), ("L1", ctypes.c_int32),
                ("L2", ctypes.c_int32), ("D", ctypes.c_int32), ("dtype", ctypes.c_int32)]


class FtaTensor5(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("stride", ctypes.c_int64 * 5)]


class FtaTensor4(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("stride", ctypes.c_int64 * 4)]


class FtaError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        super().__init__(f"{where}: {strerror(code)} (code {code})")


_lib = None

# every symbol include/fta.h declares
EXPORTS = (
    "fta_version", "fta_strerror", "fta_last_cuda_error", "fta_forward", "fta_bwd_preprocess",
    "fta_bwd_workspace_bytes", "fta_bwd_num_planes", "fta_backward", "fta_dbias_cast", "fta_dbias_sum_peers", "fta_dbias_sum_peers_sync", "fta_dbias_sum_peers_sliced", "fta_dbias_sum_peers_sliced_sync",
    "fta_read_status", "fta_profile_backward_kernel", "fta_backward_noalloc", "fta_noalloc_max_bytes",
    "fta_memcpy_2d", "fta_mask_bias",
)


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python flash-triangle-attention_b200/build.py` "
            "(nvcc, sm_100a). There is no fallback path.")
    L = ctypes.CDLL(LIB_PATH)
    P5, P4, PP = ctypes.POINTER(FtaTensor5), ctypes.POINTER(FtaTensor4), ctypes.POINTER(FtaProblem)
    vp, f32 = ctypes.c_void_p, ctypes.c_float
    L.fta_version.restype = ctypes.c_int
    L.fta_strerror.restype = ctypes.c_char_p
    L.fta_strerror.argtypes = [ctypes.c_int]
    L.fta_last_cuda_error.restype = ctypes.c_int
    L.fta_forward.restype = ctypes.c_int
    L.fta_forward.argtypes = [PP, P5, P5, P5, P4, f32, P5, vp, vp, vp, vp]
    L.fta_bwd_preprocess.restype = ctypes.c_int
    L.fta_bwd_preprocess.argtypes = [PP, P5, vp, P5, vp, vp]
    L.fta_bwd_workspace_bytes.restype = ctypes.c_size_t
    L.fta_bwd_workspace_bytes.argtypes = [PP]
    L.fta_bwd_num_planes.restype = ctypes.c_int
    L.fta_bwd_num_planes.argtypes = [PP]
    L.fta_backward.restype = ctypes.c_int
    L.fta_backward.argtypes = [PP, P5, P5, P5, P4, P5, vp, vp, f32, P5, P5, P5, vp, vp, vp,
                               ctypes.c_size_t, vp, vp]
    L.fta_dbias_cast.restype = ctypes.c_int
    L.fta_dbias_cast.argtypes = [vp, vp, ctypes.c_int64, ctypes.c_int32, vp]
    L.fta_dbias_sum_peers.restype = ctypes.c_int
    L.fta_dbias_sum_peers.argtypes = [vp, ctypes.c_int32, ctypes.c_int64, vp, vp, ctypes.c_int32, vp]
    L.fta_dbias_sum_peers_sync.restype = ctypes.c_int
    L.fta_dbias_sum_peers_sync.argtypes = [vp, vp, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, vp, vp,
                                           ctypes.c_int32, ctypes.c_uint64, vp, vp]
    L.fta_dbias_sum_peers_sliced_sync.restype = ctypes.c_int
    L.fta_dbias_sum_peers_sliced_sync.argtypes = [vp, vp, vp, vp, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64,
                                                  ctypes.c_int32, ctypes.c_uint64, vp, vp]
    L.fta_dbias_sum_peers_sliced.restype = ctypes.c_int
    L.fta_dbias_sum_peers_sliced.argtypes = [vp, vp, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32, vp]
    L.fta_read_status.restype = ctypes.c_int
    L.fta_read_status.argtypes = [vp, ctypes.POINTER(ctypes.c_int32), vp]
    L.fta_backward_noalloc.restype = ctypes.c_int
    L.fta_backward_noalloc.argtypes = [PP, P5, P5, P5, P4, P5, vp, vp, f32, P5, P5, P5, vp, vp, vp, vp]
    L.fta_noalloc_max_bytes.restype = ctypes.c_size_t
    L.fta_noalloc_max_bytes.argtypes = []
    L.fta_mask_bias.restype = ctypes.c_int
    L.fta_mask_bias.argtypes = [PP, P4, vp, vp, vp]
    L.fta_memcpy_2d.restype = ctypes.c_int
    L.fta_memcpy_2d.argtypes = [vp, ctypes.c_size_t, vp, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, vp]
    L.fta_profile_backward_kernel.restype = ctypes.c_int
    L.fta_profile_backward_kernel.argtypes = [vp, vp]
    _lib = L
    return L


def strerror(code: int) -> str:
    return lib().fta_strerror(int(code)).decode()


def check(code: int, where: str):
    if code != 0:
        raise FtaError(code, where)


def t5(t) -> FtaTensor5:
    """Descriptor of a (B,H,L1,L2,D) torch tensor (pointer + element strides)."""
    s = FtaTensor5()
    s.ptr = t.data_ptr()
    for i, st in enumerate(t.stride()):
        s.stride[i] = st
    return s


def t4(t) -> FtaTensor4:
    s = FtaTensor4()
    s.ptr = t.data_ptr()
    for i, st in enumerate(t.stride()):
        s.stride[i] = st
    return s
