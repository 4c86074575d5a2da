"""The CPU oracles (numpy and C restatements) against the golden vectors generated from the
reference's own ``reference_tt_attn`` + autograd (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

from golden import make_golden as mg
from oracle import c_oracle, tt_attn_oracle as npo

GOLD = os.path.join(os.path.dirname(__file__), "golden")
KEYS = ("o", "dq", "dk", "dv", "dbias")


def _check(res, gold, full, atol, rtol):
    for key in KEYS:
        flat = np.asarray(res[key], dtype=np.float32).reshape(-1)
        if full:
            np.testing.assert_allclose(res[key], gold[key], atol=atol, rtol=rtol, err_msg=key)
        else:
            np.testing.assert_allclose(flat[:: mg.SAMPLE_STRIDE], gold[key + "_sample"], atol=atol, rtol=rtol, err_msg=key)
        s = float(flat.astype(np.float64).sum())
        ss = float((flat.astype(np.float64) ** 2).sum())
        assert abs(s - float(gold[key + "_sum"])) <= 1e-3 * max(1.0, np.sqrt(float(gold[key + "_sumsq"]))), key
        assert abs(ss - float(gold[key + "_sumsq"])) <= 1e-4 * max(1.0, float(gold[key + "_sumsq"])), key


@pytest.mark.parametrize("name", list(mg.CASES))
@pytest.mark.parametrize("impl", ["numpy32", "numpy64", "c"])
def test_oracle_matches_reference_golden(name, impl):
    q, k, v, do, bias, scale = mg.case_inputs(name)
    gold = np.load(os.path.join(GOLD, f"golden_{name}.npz"))
    if impl == "c":
        res = c_oracle.forward_backward(q, k, v, bias, do, scale)
    else:
        res = npo.forward_backward(q, k, v, bias, do, scale, dtype=np.float32 if impl == "numpy32" else np.float64)
    # the golden values are fp32 torch results: agreement to fp32 round-off of the sums
    _check(res, gold, mg.CASES[name][-1], atol=2e-4, rtol=2e-4)


def test_masked_columns_get_zero_dbias():
    q, k, v, do, bias, scale = mg.case_inputs("masked_l32")
    res = c_oracle.forward_backward(q, k, v, bias, do, scale)
    masked = bias[0, 0, 0] < -1e8
    assert masked.sum() == 5
    assert np.all(res["dbias"][..., masked] == 0.0)


def test_forward_only_and_lse_agree():
    q, k, v, do, bias, scale = mg.case_inputs("tiny_l16")
    o_c, lse_c = c_oracle.forward(q, k, v, bias, scale, return_lse=True)
    o_n, lse_n = npo.forward(q, k, v, bias, scale, return_lse=True)
    np.testing.assert_allclose(o_c, o_n, atol=1e-5, rtol=1e-5)
    np.testing.assert_allclose(lse_c, lse_n, atol=1e-4, rtol=1e-5)
    # base-2 log-sum-exp definition (flash_tt_attn.py:258)
    x = np.einsum("bhijd,bhikd->bhijk", q, k).astype(np.float64) * scale + bias[:, :, None]
    ref = np.log2(np.exp(x - x.max(-1, keepdims=True)).sum(-1)) + x.max(-1) * npo.LOG2E
    np.testing.assert_allclose(lse_c, ref, atol=1e-4, rtol=1e-5)


def test_non_square_rows():
    """L1 != L2 (a shard of rows): each row is an independent problem, dBias sums over the shard."""
    q, k, v, do, bias, scale = mg.case_inputs("tiny_l16")
    full = c_oracle.forward_backward(q, k, v, bias, do, scale)
    a = c_oracle.forward_backward(q[:, :, :5], k[:, :, :5], v[:, :, :5], bias, do[:, :, :5], scale)
    b = c_oracle.forward_backward(q[:, :, 5:], k[:, :, 5:], v[:, :, 5:], bias, do[:, :, 5:], scale)
    for key in ("o", "dq", "dk", "dv"):
        np.testing.assert_allclose(np.concatenate([a[key], b[key]], axis=2), full[key], atol=1e-6, rtol=1e-6)
    np.testing.assert_allclose(a["dbias"] + b["dbias"], full["dbias"], atol=1e-5, rtol=1e-5)
