"""CPU oracle for triangle attention (TEST INFRASTRUCTURE, never on the product path).

A numpy restatement of the reference's definition of the op,
``reference_tt_attn`` (flash_tt_attn.py:845-864):

    qk   = q @ k^T                         (853)
    x    = qk * sm_scale + bias[:, :, None] (856-857; the reference's ``b.view(B,H,1,L,L)``
                                            is written here as a broadcast over L1 so that
                                            L1 != L2 works)
    p    = softmax(x.float(), -1).to(v.dtype)   (860)
    out  = p @ v                           (863)

and of the gradients autograd derives from it (the same quantities the reference's
backward kernels produce, flash_tt_attn.py:338-359 and 414-430):

    dV = P^T dO ; dP = dO V^T ; delta = rowsum(dO * O) ; dS = P * (dP - delta)
    dQ = sm_scale * dS K ; dK = sm_scale * dS^T Q ; dBias[b,h,j,k] = sum_i dS[b,h,i,j,k]

Everything is evaluated in ``dtype`` (float32 by default, float64 for tolerance studies)
on inputs that were already rounded to the precision under test, chunked over L1 rows so
that the (B,H,L1,L2,L2) logits never exist at once.

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference``
legs of ``bench.py`` may import this module; it is the checker, not the product.
Pinned against the reference's own function by ``tests/golden/`` (see make_golden.py there).
"""
from __future__ import annotations

import math

import numpy as np

LOG2E = 1.4426950408889634  # the reference's INV_LN2 (flash_tt_attn.py:38)


def _chunk_rows(L1: int, L2: int, budget_elems: int = 1 << 24) -> int:
    return max(1, min(L1, budget_elems // max(1, L2 * L2)))


def _logits(qk, bias_bh, sm_scale, dtype):
    """qk * sm_scale + bias as the reference forms it: three float32 tensors in a row (qk, the
    scaled qk, the sum with the bias; flash_tt_attn.py:853-857 on float32 inputs). The roundings
    only matter where a huge negative bias (-1e9) absorbs the q.k term - a fully masked row gets the
    uniform distribution - and there they are the reference's answer, so the float64 mode keeps
    them too; everything after the logits is evaluated in ``dtype``."""
    x = qk.astype(np.float32, copy=False)
    x = x * np.float32(sm_scale)
    x = x + bias_bh.astype(np.float32, copy=False)[None]
    return x.astype(dtype, copy=False)


def forward(q, k, v, bias, sm_scale, dtype=np.float32, return_lse=False):
    """O (and optionally the base-2 log-sum-exp the reference stores, flash_tt_attn.py:258).

    q, k, v: (B, H, L1, L2, D); bias: (B, H, L2, L2). Returns arrays of ``dtype``.
    """
    q = np.asarray(q, dtype=dtype)
    k = np.asarray(k, dtype=dtype)
    v = np.asarray(v, dtype=dtype)
    bias = np.asarray(bias, dtype=dtype)
    B, H, L1, L2, D = q.shape
    assert k.shape == q.shape and v.shape == q.shape
    assert bias.shape == (B, H, L2, L2)
    o = np.empty_like(q)
    lse2 = np.empty((B, H, L1, L2), dtype=dtype) if return_lse else None
    step = _chunk_rows(L1, L2)
    for b in range(B):
        for h in range(H):
            bb = bias[b, h]
            for i0 in range(0, L1, step):
                i1 = min(L1, i0 + step)
                x = np.matmul(q[b, h, i0:i1], k[b, h, i0:i1].transpose(0, 2, 1))  # (r, L2, L2)
                x = _logits(x, bb, sm_scale, dtype)
                m = x.max(axis=-1, keepdims=True)
                np.subtract(x, m, out=x)
                np.exp(x, out=x)
                s = x.sum(axis=-1, keepdims=True)
                x /= s
                o[b, h, i0:i1] = np.matmul(x, v[b, h, i0:i1])
                if return_lse:
                    lse2[b, h, i0:i1] = ((m + np.log(s)) * dtype(LOG2E))[..., 0]
    return (o, lse2) if return_lse else o


def forward_backward(q, k, v, bias, do, sm_scale, dtype=np.float32):
    """Returns dict(o, dq, dk, dv, dbias); dbias is summed over the L1 rows."""
    q = np.asarray(q, dtype=dtype)
    k = np.asarray(k, dtype=dtype)
    v = np.asarray(v, dtype=dtype)
    bias = np.asarray(bias, dtype=dtype)
    do = np.asarray(do, dtype=dtype)
    B, H, L1, L2, D = q.shape
    o = np.empty_like(q)
    dq = np.empty_like(q)
    dk = np.empty_like(q)
    dv = np.empty_like(q)
    dbias = np.zeros((B, H, L2, L2), dtype=np.float64)
    step = _chunk_rows(L1, L2)
    sc = dtype(sm_scale)
    for b in range(B):
        for h in range(H):
            bb = bias[b, h]
            for i0 in range(0, L1, step):
                i1 = min(L1, i0 + step)
                qq, kk, vv, dd = q[b, h, i0:i1], k[b, h, i0:i1], v[b, h, i0:i1], do[b, h, i0:i1]
                x = np.matmul(qq, kk.transpose(0, 2, 1))
                x = _logits(x, bb, sm_scale, dtype)
                x -= x.max(axis=-1, keepdims=True)
                np.exp(x, out=x)
                x /= x.sum(axis=-1, keepdims=True)  # x = P
                oo = np.matmul(x, vv)
                o[b, h, i0:i1] = oo
                dv[b, h, i0:i1] = np.matmul(x.transpose(0, 2, 1), dd)
                dp = np.matmul(dd, vv.transpose(0, 2, 1))
                delta = (dd * oo).sum(axis=-1, keepdims=True)
                dp -= delta
                dp *= x  # dp = dS
                dq[b, h, i0:i1] = np.matmul(dp, kk) * sc
                dk[b, h, i0:i1] = np.matmul(dp.transpose(0, 2, 1), qq) * sc
                dbias[b, h] += dp.sum(axis=0, dtype=np.float64)
    return {"o": o, "dq": dq, "dk": dk, "dv": dv, "dbias": dbias.astype(dtype)}


def flops_fwd(B, H, L1, L2, D):
    """FLOP model of the headline metric: 4*B*H*L1*L2^2*D forward, 2.5x that backward."""
    return 4.0 * B * H * L1 * L2 * L2 * D


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = math.sqrt(float((b * b).sum()))
    return math.sqrt(float(((a - b) ** 2).sum())) / max(den, 1e-30)


def max_abs(a, b):
    return float(np.max(np.abs(np.asarray(a, dtype=np.float64) - np.asarray(b, dtype=np.float64))))
