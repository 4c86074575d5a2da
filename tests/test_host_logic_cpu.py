"""Host-side logic that needs no GPU: the autograd boundary's argument checks, the workload
generator, and the L1 sharding scheme (with a 2-rank gloo group standing in for NCCL)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import flash_tt_attn as fta
import workloads
from oracle import tt_attn_oracle as npo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_attention_asserts_like_the_reference():
    q = torch.zeros(1, 1, 2, 128, 32, dtype=torch.float16)
    b = torch.zeros(1, 1, 128, 128, dtype=torch.float16)
    with pytest.raises(AssertionError):          # dtype mismatch (flash_tt_attn.py:561)
        fta.attention(q, q, q, b.float(), 1.0)
    with pytest.raises(AssertionError):          # head-dim mismatch (flash_tt_attn.py:559)
        fta.attention(q, q[..., :16], q, b, 1.0)
    with pytest.raises(AssertionError):          # no CPU path
        fta.attention(q, q, q, b, 1.0)
    with pytest.raises(AssertionError):
        fta.attention(q.float(), q.float(), q.float(), b.float(), 1.0)


def test_shard_rows_partition():
    for L1, world in [(768, 8), (384, 4), (10, 4), (3, 8), (1024, 2)]:
        seen = []
        for r in range(world):
            s = fta.shard_rows(L1, r, world)
            seen.extend(range(s.start, s.stop))
        assert seen == list(range(L1))


def test_workloads_are_seeded_and_masked():
    w = workloads.WORKLOADS["c3_crop_l384"].with_rows(4)
    a, b = workloads.make_inputs(w), workloads.make_inputs(w)
    for k in ("q", "k", "v", "do", "bias"):
        assert np.array_equal(a[k], b[k])
    masked = a["mask"][0, 0, 0]
    assert 10 < masked.sum() < 80 and not masked[0]
    assert np.all(a["bias"][0, :, :, masked] < -1e8)
    ns = workloads.WORKLOADS["ns_l768"]
    assert ns.flops_fwd() == 4.0 * 4 * 768 ** 3 * 32
    assert abs(ns.flops_fwd() + ns.flops_bwd() - 811.75e9) < 0.01e9


def test_reference_tt_attn_matches_oracle():
    w = workloads.Workload("t", 1, 2, 3, 128, 32, "fp32", 5)
    x = workloads.make_inputs(w)
    o = fta.reference_tt_attn(*(torch.from_numpy(x[k]) for k in ("q", "k", "v", "bias")), w.sm_scale)
    ref = npo.forward(x["q"], x["k"], x["v"], x["bias"], w.sm_scale)
    np.testing.assert_allclose(o.numpy(), ref, atol=2e-5, rtol=1e-4)


_WORKER = r"""
import os, sys
sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "flash-triangle-attention_b200"))
import numpy as np, torch, torch.distributed as dist
import flash_tt_attn as fta, workloads
from oracle import tt_attn_oracle as npo
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size=2)
rank = dist.get_rank()
w = workloads.Workload("t", 1, 2, 6, 128, 32, "fp32", 9)
rows = fta.shard_rows(w.L1, rank, 2)
x = workloads.make_inputs(w, rows)          # this rank's shard of the L1 rows; bias replicated
part = npo.forward_backward(x["q"], x["k"], x["v"], x["bias"], x["do"], w.sm_scale)
db = torch.from_numpy(part["dbias"].copy())
dist.all_reduce(db)                          # the path's only collective: sum of partial dBias
full = workloads.make_inputs(w)
ref = npo.forward_backward(full["q"], full["k"], full["v"], full["bias"], full["do"], w.sm_scale)
assert np.allclose(db.numpy(), ref["dbias"], atol=1e-4), "dbias"
for k in ("o", "dq", "dk", "dv"):
    assert np.allclose(part[k], ref[k][:, :, rows], atol=1e-5), k
dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_sharded_rows_with_gloo_allreduce(tmp_path):
    """Two CPU ranks: rows sharded, bias replicated, float32 dBias all-reduced (the scheme the
    GPU path runs over NCCL), checked against the unsharded oracle."""
    script = tmp_path / "worker.py"
    script.write_text(_WORKER.format(root=ROOT, port=29000 + os.getpid() % 2000))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=120)[0] for p in procs]
    for p, out in zip(procs, outs):
        assert p.returncode == 0, out


def test_shard_plan_covers_every_head_and_row_once():
    """Heads first, rows second: every (head, row) belongs to exactly one rank; ranks that share a
    head are consecutive and form one all-reduce group; different heads never share a group."""
    import numpy as np
    for H, L1, world in [(4, 768, 1), (4, 768, 2), (4, 768, 4), (4, 768, 8), (8, 2048, 8), (3, 10, 4), (2, 5, 8)]:
        cover = np.zeros((H, L1), dtype=np.int32)
        groups = {}
        for rank in range(world):
            heads, rows, peers = fta.shard_plan(H, L1, rank, world)
            cover[heads, rows] += 1
            assert rank in peers and peers == list(range(peers[0], peers[0] + len(peers)))
            groups.setdefault((heads.start, heads.stop), set()).add(tuple(peers))
        assert (cover == 1).all(), (H, L1, world)
        assert all(len(g) == 1 for g in groups.values())
