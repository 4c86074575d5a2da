"""Parity of the CUDA path (flash_tt_attn.attention -> ctypes -> libfta.so) with the CPU oracle.

Tolerance (stated by the port's specification): fp16/bf16 outputs and gradients within max-abs
2e-2 AND relative-L2 1e-2 of a float32 reference evaluated on the same rounded inputs. dBias is
judged on the float32 buffer the kernels produce (its rounding to the bias dtype alone costs up
to half an ulp of values of magnitude ~16, i.e. more than 2e-2); the rounded copy must meet the
relative-L2 bound.
"""
import os

import numpy as np
import pytest
import torch

import flash_tt_attn as fta
import workloads
from golden import make_golden as mg
from oracle import c_oracle, tt_attn_oracle as npo

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-2
REL_L2 = 1e-2
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _dt(name):
    return {"fp16": torch.float16, "bf16": torch.bfloat16}[name]


def _run(x, scale, dtype, bwd=True):
    """x: dict of float32 numpy arrays. Returns (got, rounded inputs as float32 numpy)."""
    t = {k: torch.from_numpy(np.ascontiguousarray(x[k])).cuda().to(dtype) for k in ("q", "k", "v", "do", "bias")}
    r = {k: v.float().cpu().numpy() for k, v in t.items()}
    for k in ("q", "k", "v", "bias"):
        t[k].requires_grad_()
    o = fta.attention(t["q"], t["k"], t["v"], t["bias"], scale)
    got = {"o": o}
    if bwd:
        o.backward(t["do"])
        got.update(dq=t["q"].grad, dk=t["k"].grad, dv=t["v"].grad, dbias=t["bias"].grad,
                   dbias32=fta.last_dbias_f32())
    torch.cuda.synchronize()
    fta.check_device_status()
    return {k: v.detach().float().cpu().numpy() for k, v in got.items()}, r


def _check(got, ref, keys=("o", "dq", "dk", "dv", "dbias32")):
    for k in keys:
        want = ref["dbias" if k == "dbias32" else k]
        assert not np.isnan(got[k]).any(), k
        assert npo.max_abs(got[k], want) <= MAX_ABS, (k, npo.max_abs(got[k], want))
        assert npo.rel_l2(got[k], want) <= REL_L2, (k, npo.rel_l2(got[k], want))
    if "dbias" in got:
        assert npo.rel_l2(got["dbias"], ref["dbias"]) <= REL_L2


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("shape", [
    (1, 1, 1, 128, 32), (1, 2, 3, 128, 32), (2, 1, 8, 128, 32), (1, 1, 7, 256, 32), (1, 2, 5, 384, 32),
    (1, 1, 4, 128, 64), (1, 2, 3, 256, 64), (2, 2, 20, 256, 32),
])
def test_forward_backward_parity(shape, dtype):
    B, H, L1, L2, D = shape
    w = workloads.Workload("t", B, H, L1, L2, D, dtype, seed=100 + L1 + L2 + D)
    x = workloads.make_inputs(w)
    got, r = _run(x, w.sm_scale, _dt(dtype))
    ref = npo.forward_backward(r["q"], r["k"], r["v"], r["bias"], r["do"], w.sm_scale)
    _check(got, ref)


def test_golden_c1_through_cuda_path():
    """The reference's CPU-runnable case (B1 H4 L64 D32, seed 0), embedded in an L2 = 128 problem:
    64 padding keys are masked with -1e9 (they get probability 0) and 64 padding queries are
    ignored. Compared with the golden vectors produced by the reference's own function."""
    q, k, v, do, bias, scale = mg.case_inputs("c1_cpu_l64")
    gold = np.load(os.path.join(GOLD, "golden_c1_cpu_l64.npz"))
    B, H, L, _, D = q.shape
    pad5 = lambda a: np.concatenate([a, np.zeros((B, H, L, 128 - L, D), np.float32)], axis=3)
    pb = np.full((B, H, 128, 128), -1e9, np.float32)
    pb[:, :, :L, :L] = bias
    pb[:, :, L:, :L] = 0.0
    x = {"q": pad5(q), "k": pad5(k), "v": pad5(v), "do": pad5(do), "bias": pb}
    got, _ = _run(x, scale, torch.float16)
    crop = {"o": got["o"][:, :, :, :L], "dq": got["dq"][:, :, :, :L], "dk": got["dk"][:, :, :, :L],
            "dv": got["dv"][:, :, :, :L], "dbias": got["dbias32"][:, :, :L, :L]}
    for key, arr in crop.items():
        flat = np.ascontiguousarray(arr).reshape(-1)[:: mg.SAMPLE_STRIDE]
        want = gold[key + "_sample"]
        assert np.max(np.abs(flat - want)) <= MAX_ABS, (key, float(np.max(np.abs(flat - want))))
        assert npo.rel_l2(flat, want) <= REL_L2, key
    assert np.all(got["dbias32"][:, :, :L, L:] == 0.0)  # masked keys receive no gradient


@pytest.mark.parametrize("ending_node", [False, True])
def test_masked_crop_starting_and_ending_node(ending_node):
    """Pair-stack crop with 10 % of the key columns masked by -1e9 (bf16), on a shard of rows;
    the ending-node variant is the same kernel on inputs with L1/L2 transposed."""
    w = workloads.WORKLOADS["c3_crop_l384"]
    x = workloads.make_inputs(w)
    if ending_node:
        for k in ("q", "k", "v", "do"):
            x[k] = x[k].transpose(0, 1, 3, 2, 4)
        x["bias"] = x["bias"].transpose(0, 1, 3, 2)
        masked = None
    else:
        masked = x["mask"][0, 0, 0]
    rows = slice(100, 124)
    for k in ("q", "k", "v", "do"):
        x[k] = x[k][:, :, rows]
    got, r = _run(x, w.sm_scale, torch.bfloat16)
    ref = npo.forward_backward(r["q"], r["k"], r["v"], r["bias"], r["do"], w.sm_scale)
    _check(got, ref)
    if masked is not None:
        assert np.all(got["dbias32"][..., masked] == 0.0)
        assert np.all(got["dk"][:, :, :, masked] == 0.0) and np.all(got["dv"][:, :, :, masked] == 0.0)


def test_reference_test_op_regime():
    """The reference's own test (flash_tt_attn.py:666-712): fp16, N(0, 0.5) inputs, sm_scale 0.5,
    B2 H4 L256 D32, against the naive PyTorch path in fp16 with its tolerances (atol 1e-2 for
    o, dq, dk, dv and 2e-2 for dBias)."""
    torch.manual_seed(20)
    B, H, L, D = 2, 4, 256, 32
    mk = lambda *s: torch.empty(*s, dtype=torch.float16, device="cuda").normal_(0.0, 0.5).requires_grad_()
    q, k, v, b = mk(B, H, L, L, D), mk(B, H, L, L, D), mk(B, H, L, L, D), mk(B, H, L, L)
    dout = torch.randn_like(q)
    ref = fta.reference_tt_attn(q, k, v, b, 0.5)
    ref.backward(dout)
    rg = [t.grad.clone() for t in (q, k, v, b)]
    for t in (q, k, v, b):
        t.grad = None
    out = fta.attention(q, k, v, b, 0.5)
    out.backward(dout)
    fta.check_device_status()
    assert torch.allclose(ref, out, atol=1e-2, rtol=0)
    for name, g, t, atol in (("dq", rg[0], q, 1e-2), ("dk", rg[1], k, 1e-2), ("dv", rg[2], v, 1e-2),
                             ("db", rg[3], b, 2e-2)):
        assert torch.allclose(g, t.grad, atol=atol), (name, float((g - t.grad).abs().max()))


def test_example_usage_flow():
    """example_usage.py of the reference: k and v do not require grad (randn_like drops it)."""
    q = torch.randn(4, 8, 128, 128, 32, dtype=torch.float16, device="cuda", requires_grad=True)
    k, v = torch.randn_like(q), torch.randn_like(q)
    bias = torch.randn(4, 8, 128, 128, dtype=torch.float16, device="cuda", requires_grad=True)
    out = fta.attention(q, k, v, bias, 1.0 / 32 ** 0.5)
    loss = torch.nn.functional.mse_loss(out, torch.randn_like(out))
    loss.backward()
    fta.check_device_status()
    assert q.grad is not None and bias.grad is not None and k.grad is None and v.grad is None
    assert torch.isfinite(q.grad).all() and torch.isfinite(bias.grad).all()
    assert out.shape == q.shape and out.dtype == q.dtype


def test_dbias_is_bit_reproducible_and_sharding_is_consistent():
    w = workloads.Workload("t", 1, 2, 12, 256, 32, "bf16", seed=77)
    x = workloads.make_inputs(w)
    a, _ = _run(x, w.sm_scale, torch.bfloat16)
    b, _ = _run(x, w.sm_scale, torch.bfloat16)
    for k in ("o", "dk", "dv", "dbias32", "dbias"):
        assert np.array_equal(a[k], b[k]), k          # fixed-order sums: bitwise equal
    assert np.allclose(a["dq"], b["dq"], atol=2e-2)   # dQ: float32 reductions over key blocks
    # two shards of 6 rows: per-row results identical, partial dBias sums to the full one
    parts = []
    for rows in (slice(0, 6), slice(6, 12)):
        xs = dict(x)
        for k in ("q", "k", "v", "do"):
            xs[k] = x[k][:, :, rows]
        parts.append(_run(xs, w.sm_scale, torch.bfloat16)[0])
    for k in ("o", "dk", "dv"):
        assert np.array_equal(np.concatenate([p[k] for p in parts], axis=2), a[k]), k
    assert np.allclose(parts[0]["dbias32"] + parts[1]["dbias32"], a["dbias32"], atol=1e-4, rtol=1e-5)


def test_non_contiguous_inputs_are_accepted():
    w = workloads.Workload("t", 1, 1, 128, 128, 32, "bf16", seed=5)
    x = workloads.make_inputs(w)
    t = {k: torch.from_numpy(x[k]).cuda().to(torch.bfloat16) for k in x if k != "mask"}
    ref = fta.attention(t["q"].transpose(2, 3).contiguous(), t["k"].transpose(2, 3).contiguous(),
                        t["v"].transpose(2, 3).contiguous(), t["bias"], w.sm_scale)
    out = fta.attention(t["q"].transpose(2, 3), t["k"].transpose(2, 3), t["v"].transpose(2, 3), t["bias"],
                        w.sm_scale)
    fta.check_device_status()
    assert torch.equal(ref, out)


def _report(tag, got, ref, keys=("o", "dq", "dk", "dv", "dbias32")):
    """One line per output with the measured distance from the oracle (shown with ``pytest -s``)."""
    for k in keys:
        want = ref["dbias" if k == "dbias32" else k]
        print(f"PARITY {tag:28s} {k:8s} max-abs {npo.max_abs(got[k], want):.5f} rel-L2 {npo.rel_l2(got[k], want):.6f} "
              f"max|ref| {float(np.max(np.abs(want))):.2f}")


def test_full_size_metric_shape_all_rows_against_oracle():
    """B1 H4 L768 D32 bf16 (the headline shape): EVERY output, all 768 L1 rows, against the float32
    oracle on the same rounded inputs - dBias is the float32 sum over all 768 rows, the tightest
    quantity of the path - plus the V = 1 => O = 1 property."""
    w = workloads.WORKLOADS["ns_l768"]
    x = workloads.make_inputs(w)
    got, r = _run(x, w.sm_scale, torch.bfloat16)
    ref = c_oracle.forward_backward(r["q"], r["k"], r["v"], r["bias"], r["do"], w.sm_scale)
    _report("ns_l768 bf16", got, ref)
    _check(got, ref)
    t = {k: torch.from_numpy(x[k]).cuda().to(torch.bfloat16) for k in ("q", "k", "bias")}
    ones = torch.ones_like(t["q"])
    o = fta.attention(t["q"], t["k"], ones, t["bias"], w.sm_scale)
    fta.check_device_status()
    assert float((o.float() - 1.0).abs().max()) <= 1e-2


def test_c2_readme_shape_full_against_oracle():
    """The reference's README benchmark shape, B4 H8 L256 D32 fp16, N(0,1), seed 1: all outputs of
    the whole problem against the float32 oracle."""
    w = workloads.WORKLOADS["c2_readme_l256"]
    x = workloads.make_inputs(w)
    got, r = _run(x, w.sm_scale, torch.float16)
    ref = c_oracle.forward_backward(r["q"], r["k"], r["v"], r["bias"], r["do"], w.sm_scale)
    _report("c2_readme_l256 fp16", got, ref)
    _check(got, ref)


@pytest.mark.parametrize("ending_node", [False, True])
def test_c3_crop_full_against_oracle(ending_node):
    """Pair-stack crop B1 H4 L384 D32 bf16 with 10 % of the key columns masked by -1e9, all 384 rows,
    as starting node and as ending node (L1/L2 transposed inputs, bias transposed): all outputs
    against the oracle; masked key columns receive exactly zero dBias, dK and dV."""
    w = workloads.WORKLOADS["c3_crop_l384"]
    x = workloads.make_inputs(w)
    masked = x["mask"][0, 0, 0]
    if ending_node:
        for k in ("q", "k", "v", "do"):
            x[k] = np.ascontiguousarray(x[k].transpose(0, 1, 3, 2, 4))
        # the mask term moves with the bias: after the transposition it sits on QUERY rows, so whole
        # rows of the attended plane are masked (softmax over -1e9 + N(0,1) stays finite)
        x["bias"] = np.ascontiguousarray(x["bias"].transpose(0, 1, 3, 2))
    got, r = _run(x, w.sm_scale, torch.bfloat16)
    ref = c_oracle.forward_backward(r["q"], r["k"], r["v"], r["bias"], r["do"], w.sm_scale)
    _report("c3_crop_l384 bf16 " + ("ending" if ending_node else "starting"), got, ref)
    _check(got, ref)
    if not ending_node:
        assert np.all(got["dbias32"][..., masked] == 0.0)
        assert np.all(got["dk"][:, :, :, masked] == 0.0) and np.all(got["dv"][:, :, :, masked] == 0.0)


def test_c5_long_sequence_row_subset_dbias_against_oracle():
    """B1 H8 L2=2048 D64 bf16 on a 64-row subset of L1: kernel and oracle see the same rows, so the
    float32 dBias (a 64-term sum per element at the largest tile count of any config) is comparable
    along with O, dQ, dK, dV."""
    w5 = workloads.WORKLOADS["c5_train_l2048"]
    w = workloads.Workload("c5_rows64", w5.B, w5.H, 64, w5.L2, w5.D, "bf16", w5.seed)
    x = workloads.make_inputs(w)
    got, r = _run(x, w.sm_scale, torch.bfloat16)
    ref = c_oracle.forward_backward(r["q"], r["k"], r["v"], r["bias"], r["do"], w.sm_scale)
    _report("c5 64 rows of L2048 D64 bf16", got, ref)
    _check(got, ref)



def test_ending_node_views_need_no_copy_in_forward_and_backward():
    """Ending-node orientation passed as transposed VIEWS (D stays contiguous): the tensor maps and
    the output stores take the strides as they are; values and gradients equal the copied form."""
    w = workloads.Workload("t", 1, 2, 128, 256, 32, "bf16", seed=11)
    x = workloads.make_inputs(w)
    t = {k: torch.from_numpy(x[k]).cuda().to(torch.bfloat16) for k in x if k != "mask"}
    # stored (B,H,L2,L1,D); the op sees (B,H,L1,L2,D) through transpose(2,3)
    res = []
    for copy in (True, False):
        leaf = {k: t[k].transpose(2, 3).contiguous().clone().requires_grad_(True) for k in ("q", "k", "v")}
        bias = t["bias"].clone().requires_grad_(True)
        args = [leaf[k].transpose(2, 3) for k in ("q", "k", "v")]
        if copy:
            args = [a.contiguous() for a in args]
        else:
            assert not args[0].is_contiguous()
        o = fta.attention(*args, bias, w.sm_scale)
        o.backward(t["do"])
        fta.check_device_status()
        res.append((o.detach(), leaf["q"].grad, leaf["k"].grad, leaf["v"].grad, bias.grad))
    for a, b in zip(*res):
        assert torch.equal(a, b)



@pytest.mark.parametrize("L2,masked,dtype", [(200, True, "bf16"), (300, True, "bf16"), (392, False, "bf16"),
                                             (136, True, "fp16"), (256, True, "bf16"), (200, False, "fp16")])
def test_ragged_l2_and_key_mask_in_the_kernels(L2, masked, dtype, monkeypatch):
    """L2 not a multiple of 128 and / or a boolean key mask, handled inside the kernels: q, k, v are
    read in place (no padded copy: ``F.pad`` is forbidden here for L2 % 8 == 0), the results equal
    the oracle on the same problem written with a -1e9 bias, masked keys receive exactly zero dBias,
    dK and dV."""
    B, H, L1, D = 2, 2, 5, 32
    tdt = _dt(dtype)
    g = torch.Generator().manual_seed(7 + L2)
    q, k, v, do = [torch.randn(B, H, L1, L2, D, generator=g).to(tdt) for _ in range(4)]
    bias = torch.randn(B, H, L2, L2, generator=g).to(tdt)
    mask = None
    if masked:
        mask = torch.rand(B, L2, generator=g) > 0.2
        mask[:, 0] = True
    if L2 % 8 == 0:
        def no_pad(*a, **kw):
            raise AssertionError("attention() copied its inputs for an L2 the kernels handle natively")
        monkeypatch.setattr(torch.nn.functional, "pad", no_pad)
    scale = D ** -0.5
    leaves = [a.cuda().requires_grad_(True) for a in (q, k, v, bias)]
    o = fta.attention(*leaves, scale, key_mask=None if mask is None else mask.cuda())
    o.backward(do.cuda())
    fta.check_device_status()
    assert o.shape == (B, H, L1, L2, D)
    bm = bias.float()
    if mask is not None:
        bm = torch.where(mask[:, None, None, :], bm, torch.tensor(-1.0e9))
    ref = npo.forward_backward(q.float().numpy(), k.float().numpy(), v.float().numpy(), bm.numpy(),
                               do.float().numpy(), scale)
    got = {"o": o, "dq": leaves[0].grad, "dk": leaves[1].grad, "dv": leaves[2].grad, "dbias": leaves[3].grad,
           "dbias32": fta.last_dbias_f32()}
    got = {n: t.detach().float().cpu().numpy() for n, t in got.items()}
    got["dbias32"] = got["dbias32"][:, :, :L2, :L2]  # an L2 that is not a multiple of 8 ran padded to one
    for name in ("o", "dq", "dk", "dv", "dbias32"):
        want = ref["dbias" if name == "dbias32" else name]
        assert not np.isnan(got[name]).any(), name
        assert npo.max_abs(got[name], want) <= MAX_ABS, (name, npo.max_abs(got[name], want))
        assert npo.rel_l2(got[name], want) <= REL_L2, name
    assert npo.rel_l2(got["dbias"], ref["dbias"]) <= REL_L2
    if mask is not None:
        for b_ in range(B):
            dead = ~mask[b_].numpy()
            assert np.all(got["dbias32"][b_][:, :, dead] == 0.0)
            assert np.all(got["dk"][b_][:, :, dead] == 0.0) and np.all(got["dv"][b_][:, :, dead] == 0.0)


def test_fully_masked_batch_element_gives_zero_rows():
    """Every key of a batch element masked: its output rows and all its gradients are exactly 0,
    nothing is NaN, and the other batch element is untouched."""
    B, H, L1, L2, D = 2, 1, 3, 128, 32
    g = torch.Generator().manual_seed(3)
    q, k, v, do = [torch.randn(B, H, L1, L2, D, generator=g).to(torch.bfloat16).cuda() for _ in range(4)]
    bias = torch.randn(B, H, L2, L2, generator=g).to(torch.bfloat16).cuda()
    mask = torch.ones(B, L2, dtype=torch.bool)
    mask[1] = False
    leaves = [a.requires_grad_(True) for a in (q, k, v, bias)]
    o = fta.attention(*leaves, D ** -0.5, key_mask=mask.cuda())
    o.backward(do)
    fta.check_device_status()
    for t in (o, *[l.grad for l in leaves]):
        assert torch.isfinite(t).all()
    assert float(o[1].detach().abs().max()) == 0.0
    for l in leaves:
        assert float(l.grad[1].abs().max()) == 0.0
    ref = fta.attention(q[:1].detach(), k[:1].detach(), v[:1].detach(), bias[:1].detach(), D ** -0.5)
    assert torch.equal(ref, o[:1].detach())


def test_streamed_host_entry_point_matches_the_device_path():
    """Pinned host tensors streamed through the GPU in blocks of rows: O, dQ, dK, dV are bit-equal to
    one call on device-resident tensors (rows are independent problems); dBias agrees in float32."""
    w = workloads.Workload("t", 1, 2, 20, 256, 32, "bf16", seed=17)
    x = workloads.make_inputs(w)
    host = {k: torch.from_numpy(x[k]).to(torch.bfloat16).pin_memory() for k in ("q", "k", "v", "do", "bias")}
    out = {k: torch.empty_like(host["q"]).pin_memory() for k in ("o", "dq", "dk", "dv")}
    out["dbias"] = torch.empty_like(host["bias"]).pin_memory()
    fta.attention_fwd_bwd_streamed(host, w.sm_scale, out, block_rows=4)
    db_streamed = fta.last_dbias_f32().clone()
    t = {k: host[k].cuda() for k in host}
    for k in ("q", "k", "v", "bias"):
        t[k].requires_grad_()
    o = fta.attention(t["q"], t["k"], t["v"], t["bias"], w.sm_scale)
    o.backward(t["do"])
    fta.check_device_status()
    assert torch.equal(out["o"], o.detach().cpu())
    for name, leaf in (("dq", "q"), ("dk", "k"), ("dv", "v")):
        assert torch.equal(out[name], t[leaf].grad.cpu()), name
    ref = fta.last_dbias_f32()
    assert float((db_streamed - ref).abs().max()) <= 1e-4 * float(ref.abs().max()) + 1e-5
    assert npo.rel_l2(out["dbias"].float().numpy(), ref.cpu().numpy()) <= 5e-3


def _device_inputs(w, dtype, with_do=True):
    """Full-size tensors drawn on the device (host generation of GiB-sized tensors is too slow for
    a test); the checks below copy the sampled rows back and hand the same values to the oracle."""
    g = torch.Generator(device="cuda").manual_seed(w.seed)
    shape = (w.B, w.H, w.L1, w.L2, w.D)
    t = {k: (torch.randn(shape, device="cuda", dtype=torch.float32, generator=g) * w.qkv_std).to(dtype)
         for k in ("q", "k", "v")}
    if with_do:
        t["do"] = torch.randn(shape, device="cuda", dtype=torch.float32, generator=g).to(dtype)
    t["bias"] = (torch.randn((w.B, w.H, w.L2, w.L2), device="cuda", dtype=torch.float32, generator=g)
                 * w.bias_std).to(dtype)
    return t


def _rows_to_numpy(t, sl):
    return {k: (v if k == "bias" else v[:, :, sl]).float().cpu().numpy() for k, v in t.items()}


def test_c4_inference_shape_forward_only():
    """B1 H4 L1024 D32 bf16, forward only (q,k,v std 1/sqrt(D), bias std 2): sampled L1 rows against
    the oracle and the V = 1 property over the whole tensor."""
    w = workloads.WORKLOADS["c4_infer_l1024"]
    t = _device_inputs(w, torch.bfloat16, with_do=False)
    with torch.no_grad():
        o = fta.attention(t["q"], t["k"], t["v"], t["bias"], w.sm_scale)
        ones = fta.attention(t["q"], t["k"], torch.ones_like(t["v"]), t["bias"], w.sm_scale)
    fta.check_device_status()
    assert float((ones.float() - 1.0).abs().max()) <= 1e-2
    for i in (0, 511, 1023):
        sl = slice(i, i + 1)
        r = _rows_to_numpy(t, sl)
        ref = c_oracle.forward(r["q"], r["k"], r["v"], r["bias"], w.sm_scale)
        got = o[:, :, sl].float().cpu().numpy()
        assert npo.max_abs(got, ref) <= MAX_ABS and npo.rel_l2(got, ref) <= REL_L2, i


def test_c5_long_sequence_training_shape_sampled_rows():
    """B1 H8 L2048 D64 bf16 (4 GiB per tensor), forward + backward: sampled L1 rows of O, dQ, dK,
    dV against the oracle (they are per-row quantities) and the row sums of dBias (each dS row
    sums to zero, so every row of dBias must too, relative to its absolute sum)."""
    free, _ = torch.cuda.mem_get_info()
    if free < 80 * 2 ** 30:
        pytest.skip("needs about 70 GiB of device memory")
    w = workloads.WORKLOADS["c5_train_l2048"]
    t = _device_inputs(w, torch.bfloat16)
    for k in ("q", "k", "v", "bias"):
        t[k].requires_grad_()
    o = fta.attention(t["q"], t["k"], t["v"], t["bias"], w.sm_scale)
    o.backward(t["do"])
    fta.check_device_status()
    db32 = fta.last_dbias_f32()
    rowsum = db32.double().sum(-1)
    scale_ = db32.double().abs().sum(-1)
    assert float((rowsum.abs() / scale_).max()) < 2e-3
    got = {"o": o.detach(), "dq": t["q"].grad, "dk": t["k"].grad, "dv": t["v"].grad}
    vals = {k: v.detach() for k, v in t.items()}
    for i in (0, 1000, 2047):
        sl = slice(i, i + 1)
        r = _rows_to_numpy(vals, sl)
        ref = c_oracle.forward_backward(r["q"], r["k"], r["v"], r["bias"], r["do"], w.sm_scale)
        for k in ("o", "dq", "dk", "dv"):
            a = got[k][:, :, sl].float().cpu().numpy()
            assert npo.max_abs(a, ref[k]) <= MAX_ABS, (k, i, npo.max_abs(a, ref[k]))
            assert npo.rel_l2(a, ref[k]) <= REL_L2, (k, i, npo.rel_l2(a, ref[k]))
