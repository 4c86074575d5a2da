"""Device-side failures are bounded, visible and leave the GPU usable.

Nothing here faults, traps or hangs a GPU: the failure is a wait on a barrier that nobody arrives
at, and the wait gives up by itself after a few milliseconds (tests/cuda/wait_timeout_probe.cu uses
the product's own ``mbar_wait`` from csrc/tc05.cuh with a small limit).
"""
import ctypes
import os
import shutil
import subprocess

import numpy as np
import pytest
import torch

import _cabi
import flash_tt_attn as fta
import workloads

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "flash-triangle-attention_b200", "csrc")
SRC = os.path.join(ROOT, "tests", "cuda", "wait_timeout_probe.cu")


def _nvcc():
    cand = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    return cand if os.path.exists(cand) else shutil.which("nvcc")


@pytest.fixture(scope="module")
def probe(tmp_path_factory):
    nvcc = _nvcc()
    if not nvcc:
        pytest.skip("nvcc is needed to build the test-only probe kernel")
    out = str(tmp_path_factory.mktemp("probe") / "libwaitprobe.so")
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O2", "-shared", "-Xcompiler",
                    "-fPIC", "-I", CSRC, SRC, "-o", out], check=True)
    lib = ctypes.CDLL(out)
    lib.wait_probe_launch.restype = ctypes.c_int
    lib.wait_probe_launch.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]
    return lib


def test_bounded_wait_runs_out_records_status_and_returns(probe):
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # healthy launch: the barrier is arrived at, nothing is recorded
    assert probe.wait_probe_launch(status.data_ptr(), 1, 5_000_000, waited.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(waited.item()) == 0
    # nobody arrives: the wait gives up after its limit (5 ms), the kernel returns by itself
    assert probe.wait_probe_launch(status.data_ptr(), 0, 5_000_000, waited.data_ptr(), stream) == 0
    torch.cuda.synchronize()   # returns: the kernel did not hang
    assert int(status.item()) == 0x1000 | 0x7
    assert 4_000_000 <= int(waited.item()) <= 500_000_000
    # the library reports the word the same way
    code = ctypes.c_int32(0)
    assert _cabi.lib().fta_read_status(status.data_ptr(), ctypes.byref(code), stream) == -10
    assert code.value == 0x1007
    # the context is intact: a healthy launch and a real forward + backward follow
    status.zero_()
    assert probe.wait_probe_launch(status.data_ptr(), 1, 5_000_000, waited.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    q = torch.randn(1, 1, 2, 128, 32, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(1, 1, 128, 128, device="cuda", dtype=torch.bfloat16)
    o = fta.attention(q, q.detach(), q.detach(), b, 0.2)
    o.sum().backward()
    fta.check_device_status()
    assert torch.isfinite(q.grad).all()


def test_status_word_of_an_earlier_call_surfaces_without_a_sync():
    """The module mirrors its status word to pinned host memory after every call and looks at the
    mirror before the next launch: a recorded failure raises at the next call (here the word is
    set by hand, as a kernel whose wait ran out would)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    q = torch.randn(1, 1, 2, 128, 32, device="cuda", dtype=torch.float16)
    b = torch.randn(1, 1, 128, 128, device="cuda", dtype=torch.float16)
    fta.attention(q, q, q, b, 0.2)
    st = fta._status_of(dev)
    st.word.fill_(0x1042)          # what a timed-out wait at site 0x42 leaves behind
    fta.attention(q, q, q, b, 0.2)  # publishes the word to the mirror (no exception yet, no sync)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="0x1042"):
        fta.attention(q, q, q, b, 0.2)
    fta.attention(q, q, q, b, 0.2)  # the word was cleared when it was reported
    fta.check_device_status()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_one_process_two_devices():
    """The kernels' shared-memory attribute is a per-device setting: one process that calls the
    library on cuda:0 and then on cuda:1 must work on both."""
    w = workloads.Workload("t", 1, 1, 3, 128, 32, "bf16", seed=2)
    x = workloads.make_inputs(w)
    outs = []
    for dev in ("cuda:0", "cuda:1"):
        t = {k: torch.from_numpy(x[k]).to(dev).to(torch.bfloat16) for k in ("q", "k", "v", "do", "bias")}
        for k in ("q", "k", "v", "bias"):
            t[k].requires_grad_()
        o = fta.attention(t["q"], t["k"], t["v"], t["bias"], w.sm_scale)
        o.backward(t["do"])
        torch.cuda.synchronize(dev)
        fta.check_device_status(dev)
        outs.append([o.detach().cpu(), t["q"].grad.cpu(), t["k"].grad.cpu(), t["v"].grad.cpu(), t["bias"].grad.cpu()])
    for a, b_ in zip(*outs[:2]):
        assert torch.equal(a, b_) or np.allclose(a.float().numpy(), b_.float().numpy(), atol=2e-2)


def test_peer_sum_wait_runs_out_without_a_peer():
    """fta_dbias_sum_peers_sync waits for every rank's epoch word; here "rank 1" is a second buffer on the
    same GPU whose word nobody ever writes, so the 5 ms wait runs out: the kernel must leave
    0x1000 | 0x61 in the status word, write no output, return, and the device must stay usable."""
    import _cabi
    L = _cabi.lib()
    dev = torch.device("cuda", 0)
    n = 4096
    parts = [torch.ones(n, device=dev), torch.ones(n, device=dev)]
    flags = [torch.zeros(2, dtype=torch.int32, device=dev), torch.zeros(2, dtype=torch.int32, device=dev)]
    pp = torch.tensor([p.data_ptr() for p in parts], dtype=torch.int64, device=dev)
    fp = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.full((n,), -7.0, dtype=torch.bfloat16, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    rc = L.fta_dbias_sum_peers_sync(pp.data_ptr(), fp.data_ptr(), 2, 0, 1, n, None, out.data_ptr(), _cabi.FTA_BF16,
                                    5_000_000, status.data_ptr(), st)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == (0x1000 | 0x61)
    assert bool((out == -7.0).all())           # no output after a failed line-up
    assert int(flags[0][0]) == 1 and int(flags[1][0]) == 1   # this rank did publish its epoch everywhere
    # the word of "rank 1" set by hand: the same call now goes through
    status.zero_()
    flags[0][1] = 1
    rc = L.fta_dbias_sum_peers_sync(pp.data_ptr(), fp.data_ptr(), 2, 0, 1, n, None, out.data_ptr(), _cabi.FTA_BF16,
                                    5_000_000, status.data_ptr(), st)
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == 0 and bool((out == 2.0).all())
