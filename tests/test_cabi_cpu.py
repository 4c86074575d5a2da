"""CPU-side checks of the C ABI: the library loads, exports every symbol include/fta.h
declares, and rejects bad arguments on the host before anything touches a device."""
import ctypes
import os
import re

import pytest

import _cabi
from _cabi import FtaProblem, FtaTensor4, FtaTensor5

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "fta.h")).read()
    return sorted(set(re.findall(r"FTA_API\s+[\w\s\*]+?\b(fta_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _cabi.lib()
    names = _declared()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/fta.h but not exported"
    assert sorted(_cabi.EXPORTS) == names
    assert lib.fta_version() >= 100


def test_strerror_is_total():
    for code in range(-15, 1):
        s = _cabi.strerror(code)
        assert isinstance(s, str) and s
    assert "128" in _cabi.strerror(-2)


def _t5(ptr=0x1000, strides=(1 << 20, 1 << 18, 4096, 32, 1)):
    t = FtaTensor5()
    t.ptr = ptr
    for i, s in enumerate(strides):
        t.stride[i] = s
    return t


def _t4(ptr=0x1000, strides=(1 << 20, 1 << 14, 128, 1)):
    t = FtaTensor4()
    t.ptr = ptr
    for i, s in enumerate(strides):
        t.stride[i] = s
    return t


@pytest.mark.parametrize("prob,code", [
    (FtaProblem(1, 1, 4, 100, 32, 1), -2),   # L2 not a multiple of 128
    (FtaProblem(0, 1, 4, 128, 32, 1), -2),   # empty batch
    (FtaProblem(1, 1, 0, 128, 32, 1), -2),   # no rows
    (FtaProblem(1, 1, 4, 128, 16, 1), -3),   # head dim the forward kernel has no tile for
    (FtaProblem(1, 1, 4, 128, 128, 1), -3),
    (FtaProblem(1, 1, 4, 128, 32, 7), -4),   # dtype
])
def test_forward_rejects_bad_problem_on_host(prob, code):
    lib = _cabi.lib()
    rc = lib.fta_forward(prob, _t5(), _t5(), _t5(), _t4(), 1.0, _t5(), None, 0x2000, 0x3000, None)
    assert rc == code


def test_forward_rejects_bad_tensors_on_host():
    lib = _cabi.lib()
    prob = FtaProblem(1, 1, 4, 128, 32, 1)
    ok5, ok4 = _t5(), _t4()
    assert lib.fta_forward(prob, _t5(ptr=0), ok5, ok5, ok4, 1.0, ok5, None, 0x2000, 0x3000, None) == -1
    assert lib.fta_forward(prob, _t5(ptr=0x1004), ok5, ok5, ok4, 1.0, ok5, None, 0x2000, 0x3000, None) == -6
    assert lib.fta_forward(prob, _t5(strides=(1 << 20, 1 << 18, 4096, 32, 2)), ok5, ok5, ok4, 1.0, ok5,
                           None, 0x2000, 0x3000, None) == -5
    assert lib.fta_forward(prob, ok5, ok5, _t5(strides=(1 << 20, 1 << 18, 4100, 32, 1)), ok4, 1.0, ok5,
                           None, 0x2000, 0x3000, None) == -5
    assert lib.fta_forward(prob, ok5, ok5, ok5, _t4(strides=(1 << 20, 1 << 14, 128, 2)), 1.0, ok5,
                           None, 0x2000, 0x3000, None) == -5
    assert lib.fta_forward(prob, ok5, ok5, ok5, ok4, 1.0, ok5, None, None, 0x3000, None) == -1
    # statistics and residual pointers must be 16-byte aligned too
    assert lib.fta_forward(prob, ok5, ok5, ok5, ok4, 1.0, ok5, None, 0x2004, 0x3000, None) == -6
    assert lib.fta_forward(prob, ok5, ok5, ok5, ok4, 1.0, ok5, 0x5008, 0x2000, 0x3000, None) == -6


def test_backward_rejects_small_workspace_and_null():
    lib = _cabi.lib()
    prob = FtaProblem(1, 2, 5, 256, 32, 1)
    need = lib.fta_bwd_workspace_bytes(prob)
    planes = lib.fta_bwd_num_planes(prob)
    assert planes >= 1
    # float32 dQ accumulator + planes + key-major bias copy
    assert need >= 1 * 2 * 5 * 256 * 32 * 4 + planes * 2 * 256 * 256 * 4 + 2 * 256 * 256 * 2
    a5, a4 = _t5(), _t4()
    args = lambda ws, nbytes: lib.fta_backward(prob, a5, a5, a5, a4, a5, 0x2000, 0x2100, 1.0, a5, a5, a5,
                                               0x2200, None, ws, nbytes, 0x3000, None)
    assert args(0x10000, need - 1) == -7
    assert args(0x10010, need) == -7      # not 256-byte aligned
    assert args(None, need) == -1
    # lse, delta and the dBias buffers are read / written with 16-byte vectors and bulk copies
    bad = lambda lse, delta, db32, dbc: lib.fta_backward(prob, a5, a5, a5, a4, a5, lse, delta, 1.0, a5, a5, a5,
                                                         db32, dbc, 0x10000, need, 0x3000, None)
    assert bad(0x2004, 0x2100, 0x2200, None) == -6
    assert bad(0x2000, 0x2108, 0x2200, None) == -6
    assert bad(0x2000, 0x2100, 0x2204, None) == -6
    assert bad(0x2000, 0x2100, 0x2200, 0x2302) == -6
    assert lib.fta_bwd_preprocess(prob, a5, 0x4004, a5, 0x2100, None) == -6
    assert lib.fta_bwd_workspace_bytes(FtaProblem(1, 1, 4, 100, 32, 1)) == 0


def test_plane_count_follows_the_schedule():
    """The number of private dBias planes = row blocks per (head, key block). Without a GPU the
    library assumes 148 SMs. While the planes fit half the L2 the best single-wave schedule wins
    (one head: 24 planes of 32 rows, not 23 of 34); when they do not, the fewest planes within 7 %."""
    lib = _cabi.lib()
    planes = lambda B, H, L1, L2, D: lib.fta_bwd_num_planes(FtaProblem(B, H, L1, L2, D, 1))
    assert planes(1, 4, 768, 768, 32) == 6      # the headline shape: 144 CTAs of 128 rows
    assert planes(1, 1, 768, 768, 32) == 24     # one head per GPU (4 GPUs): 144 CTAs of 32 rows
    assert planes(1, 1, 384, 768, 32) == 24     # one head x half the rows (8 GPUs)
    assert planes(1, 2, 768, 768, 32) == 12
    assert planes(1, 8, 2048, 2048, 64) == 8    # 134 MB per plane set: the tolerant rule
    for shape in ((1, 4, 1, 128, 32), (2, 3, 7, 136, 64), (4, 8, 256, 256, 32)):
        n = planes(*shape)
        assert 1 <= n <= 64 and n <= shape[2]


def test_dbias_cast_argument_checks():
    lib = _cabi.lib()
    assert lib.fta_dbias_cast(None, 0x1000, 16, 1, None) == -1
    assert lib.fta_dbias_cast(0x1000, 0x2000, 6, 1, None) == -2
    assert lib.fta_dbias_cast(0x1000, 0x2000, 16, 5, None) == -4
    assert lib.fta_dbias_cast(0x1004, 0x2000, 16, 1, None) == -6
    assert lib.fta_dbias_cast(0x1000, 0x2008, 16, 1, None) == -6
    assert lib.fta_read_status(None, None, None) == -1
