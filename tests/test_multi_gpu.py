"""Row-sharded run on 2 GPUs (NCCL): each rank owns half of the L1 rows, the bias is replicated,
the backward all-reduces the float32 dBias. Runs as child processes; skipped with < 2 GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_WORKER = r"""
import os, sys
sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "flash-triangle-attention_b200"))
import numpy as np, torch, torch.distributed as dist
import flash_tt_attn as fta, workloads
from oracle import tt_attn_oracle as npo
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
w = workloads.Workload("t", 1, 2, 10, 256, 32, "bf16", 13)
rows = fta.shard_rows(w.L1, rank, world)
x = workloads.make_inputs(w, rows)
t = {{k: torch.from_numpy(x[k]).cuda().to(torch.bfloat16) for k in ("q", "k", "v", "do", "bias")}}
for k in ("q", "k", "v", "bias"):
    t[k].requires_grad_()
o = fta.attention(t["q"], t["k"], t["v"], t["bias"], w.sm_scale, group=dist.group.WORLD)
o.backward(t["do"])
torch.cuda.synchronize(); fta.check_device_status()
full = workloads.make_inputs(w)
r = {{k: torch.from_numpy(full[k]).to(torch.bfloat16).float().numpy() for k in ("q", "k", "v", "do", "bias")}}
ref = npo.forward_backward(r["q"], r["k"], r["v"], r["bias"], r["do"], w.sm_scale)
got = {{"o": o, "dq": t["q"].grad, "dk": t["k"].grad, "dv": t["v"].grad}}
for k, v in got.items():
    g = v.detach().float().cpu().numpy()
    assert npo.max_abs(g, ref[k][:, :, rows]) <= 2e-2 and npo.rel_l2(g, ref[k][:, :, rows]) <= 1e-2, k
db = fta.last_dbias_f32().cpu().numpy()          # all-reduced: the full dBias on every rank
assert npo.max_abs(db, ref["dbias"]) <= 2e-2 and npo.rel_l2(db, ref["dbias"]) <= 1e-2
assert npo.rel_l2(t["bias"].grad.float().cpu().numpy(), ref["dbias"]) <= 1e-2
dist.destroy_process_group()
print("rank", rank, "ok")
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_row_sharding_matches_oracle(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER.format(root=ROOT))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 400), str(script)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]


_PEER_WORKER = r"""
import os, sys
sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "flash-triangle-attention_b200"))
import torch, torch.distributed as dist
import flash_tt_attn as fta
import _cabi
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
dev = torch.device("cuda", rank)
B, H, L2 = 1, 2, 256
peer = fta.PeerDbiasSum((B, H, L2, L2), dist.group.WORLD, dev, torch.bfloat16)
L = _cabi.lib()
stream = torch.cuda.current_stream().cuda_stream
for step in range(5):   # both partial buffers, several times over
    g = torch.Generator(device=dev).manual_seed(100 * step + rank)
    part = torch.randn(B, H, L2, L2, device=dev, generator=g) * 3.0
    peer.partial().copy_(part)
    out16 = torch.empty(B, H, L2, L2, dtype=torch.bfloat16, device=dev)
    out32 = torch.empty(B, H, L2, L2, dtype=torch.float32, device=dev)
    peer.reduce(out16, out32)
    ref = part.clone()
    dist.all_reduce(ref)          # NCCL, same two addends: a + b either way
    torch.cuda.synchronize()
    assert torch.equal(out32, ref), (step, float((out32 - ref).abs().max()))
    assert torch.equal(out16, ref.to(torch.bfloat16))
    # every rank holds the same bits
    both = [torch.empty_like(out32) for _ in range(world)]
    dist.all_gather(both, out32)
    assert torch.equal(both[0], both[1])
# the sliced variant (what groups of more than two use), forced on for this pair
import torch.distributed._symmetric_memory as symm_mem
out_sym = symm_mem.empty((peer.n,), dtype=torch.bfloat16, device=dev)
oh = symm_mem.rendezvous(out_sym, dist.group.WORLD)
outs = torch.tensor([int(p) for p in oh.buffer_ptrs], dtype=torch.int64, device=dev)
for step in range(3):
    g = torch.Generator(device=dev).manual_seed(777 * step + rank)
    part = torch.randn(B, H, L2, L2, device=dev, generator=g) * 3.0
    peer.partial().copy_(part)
    peer.hdl.barrier(channel=0)
    assert L.fta_dbias_sum_peers_sliced(peer.parts[peer.step & 1].data_ptr(), outs.data_ptr(), world, rank, peer.n, 1, stream) == 0
    peer.hdl.barrier(channel=0)
    peer.step += 1
    ref = part.clone(); dist.all_reduce(ref); torch.cuda.synchronize()
    assert torch.equal(out_sym.view(B, H, L2, L2), ref.to(torch.bfloat16)), step
# ... and with both line-ups inside the kernels (epoch words continue where reduce() left them)
for step in range(3):
    g = torch.Generator(device=dev).manual_seed(555 * step + rank)
    part = torch.randn(B, H, L2, L2, device=dev, generator=g) * 3.0
    peer.partial().copy_(part)
    out_sym.zero_()
    rc = L.fta_dbias_sum_peers_sliced_sync(peer.parts[peer.step & 1].data_ptr(), outs.data_ptr(), peer._flag_ptrs.data_ptr(),
                                           peer.flags.data_ptr(), world, rank, peer.step + 1, peer.n, 1, 0,
                                           peer.status.word.data_ptr(), stream)
    assert rc == 0
    peer.step += 1
    got = out_sym.view(B, H, L2, L2).clone()      # enqueued behind the wait kernel: complete
    ref = part.clone(); dist.all_reduce(ref); torch.cuda.synchronize()
    fta.check_device_status()
    assert torch.equal(got, ref.to(torch.bfloat16)), step
    dist.barrier()   # nobody zeroes its buffer while the other rank still writes into it
# argument checks of the entry point, no launch
assert L.fta_dbias_sum_peers(None, 2, 64, None, out16.data_ptr(), 1, stream) == -1
assert L.fta_dbias_sum_peers(peer.parts[0].data_ptr(), 2, 60, None, out16.data_ptr(), 1, stream) == -2
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_dbias_sum_over_peer_memory_equals_the_allreduce(tmp_path):
    """fta_dbias_sum_peers through PeerDbiasSum (symmetric memory, plain peer loads, no multicast)
    gives the bits of the NCCL all-reduce + cast on both ranks, step after step."""
    script = tmp_path / "peer_worker.py"
    script.write_text(_PEER_WORKER.format(root=ROOT))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29900 + os.getpid() % 90), str(script)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
