"""Drop-in for the reference module ``flash_tt_attn``: ``attention(q, k, v, b_pw, sm_scale)``.

Same entry point, argument meaning and autograd behaviour as the reference's
``_attention`` / ``attention = _attention.apply`` (flash_tt_attn.py:554-663), with the three
Triton launches replaced by hand-written sm_100a kernels reached through the C ABI of
``libfta.so`` (include/fta.h):

  forward   : ``_attn_fwd[grid](...)``              (577-586)  -> ``fta_forward``
  backward  : ``_attn_bwd_preprocess[pre_grid]``    (636-641)  -> ``fta_bwd_preprocess``
              ``_attn_bwd[grid]`` + ``zeros_like``  (613, 647-658) -> ``fta_backward``

Differences from the reference, all relaxations:
  * fp16 and bf16 (the reference is fp16 only, line 99); L1 may differ from L2 (the reference
    needs a square pair representation, lines 584 and 616); L2 need not be a power of two
    (line 618) nor a multiple of 128 (ragged last blocks are padded by the tile loads and clipped
    by the stores; only a bias-sized tensor is staged, ``fta_mask_bias``); a boolean ``key_mask``
    removes keys;
  * ``dO`` and non-dense inputs are made contiguous instead of asserted on (604-606);
  * dBias is accumulated in float32 in a fixed order (bit-reproducible) and rounded once,
    instead of fp16 atomics (425-426); with bf16 inputs the forward also saves the 16 bits of O
    that its rounding drops, so that delta = rowsum(dO * O) - and with it dBias, a sum over all
    L1 rows - keeps the accuracy the fp16 path has (costs one more saved tensor of q's size;
    ``FTA_SAVE_O_RESIDUAL=0`` switches it off);
  * an optional ``group`` (a ``torch.distributed`` process group): q, k, v hold this rank's
    shard of the L1 rows, the bias is replicated, and the backward all-reduces the float32
    dBias over the group before rounding.

There is no fallback: without a CUDA device and a built ``libfta.so`` every call raises.
"""
from __future__ import annotations

import os

import torch

import _cabi
from _cabi import FtaProblem, check, t4, t5

__all__ = ["attention", "attention_fwd_bwd_streamed", "reference_tt_attn", "check_device_status",
           "last_dbias_f32", "shard_plan", "shard_rows", "PeerDbiasSum"]

_DEBUG = os.environ.get("FTA_DEBUG", "0") == "1"
_SAVE_O_RESIDUAL = os.environ.get("FTA_SAVE_O_RESIDUAL", "1") != "0"
_status_words = {}
_copy_streams = {}
_last = {"dbias_f32": None}


class _Status:
    """Per-device status word of the kernels plus a pinned host mirror of it.

    The kernels never trap: a bounded device-side wait that runs out writes a code to ``word`` and
    the launch returns with unfinished outputs. After every call of this module the word is copied
    to ``mirror`` on the stream (4 bytes, no synchronisation); the next call looks at the mirror
    on the host before it launches anything, so a failure surfaces as an exception at most one
    call late without the hot path ever waiting for the device."""

    def __init__(self, device):
        self.word = torch.zeros(1, dtype=torch.int32, device=device)
        self.mirror = torch.zeros(1, dtype=torch.int32).pin_memory()

    def publish(self):
        self.mirror.copy_(self.word, non_blocking=True)

    def raise_if_set(self, code=None):
        code = int(self.mirror[0]) if code is None else code
        if code != 0:
            self.word.zero_()
            self.mirror.zero_()
            raise RuntimeError(f"flash_tt_attn: device status 0x{code:x} (a bounded device-side wait ran out "
                               "in an earlier call; its outputs are incomplete)")


def _status_of(device) -> _Status:
    key = (device.type, device.index)
    st = _status_words.get(key)
    if st is None:
        st = _status_words[key] = _Status(device)
    return st


def _status(device) -> torch.Tensor:
    return _status_of(device).word


def check_device_status(device=None) -> None:
    """Raise if a kernel of this module reported a device-side error (a bounded wait that ran
    out). Synchronises the device's current stream."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    st = _status_of(device)
    st.raise_if_set(int(st.word.item()))


def last_dbias_f32():
    """The float32 dBias of the most recent backward call (before rounding to the bias dtype)."""
    return _last["dbias_f32"]


def _dense(t: torch.Tensor) -> torch.Tensor:
    """Inputs the kernels can address directly: unit stride in D, other strides multiples of 8
    elements, 16-byte aligned base. Anything else is copied."""
    ok = t.stride(-1) == 1 and all(s % 8 == 0 and s > 0 for s in t.stride()[:-1]) and t.data_ptr() % 16 == 0
    return t if ok else t.contiguous()


def _problem(q: torch.Tensor) -> FtaProblem:
    B, H, L1, L2, D = q.shape
    return FtaProblem(B, H, L1, L2, D, _cabi.FTA_BF16 if q.dtype == torch.bfloat16 else _cabi.FTA_FP16)


def _l2p(L2: int) -> int:
    return (L2 + 127) // 128 * 128


class _attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, b_pw, sm_scale, group=None, key_mask=None):
        HEAD_DIM_Q, HEAD_DIM_K, HEAD_DIM_V = q.shape[-1], k.shape[-1], v.shape[-1]
        assert HEAD_DIM_Q == HEAD_DIM_K and HEAD_DIM_K == HEAD_DIM_V
        assert HEAD_DIM_K in {32, 64}, "head dimension must be 32 or 64"
        assert q.dtype == k.dtype == v.dtype == b_pw.dtype
        assert q.dtype in (torch.float16, torch.bfloat16), "fp16 or bf16 only"
        assert q.is_cuda, "flash_tt_attn.attention needs CUDA tensors (there is no CPU path)"
        assert q.dim() == 5 and q.shape == k.shape == v.shape
        B, H, L1, L2, D = q.shape
        assert b_pw.shape == (B, H, L2, L2), "bias must be (B, H, L2, L2)"
        assert L2 % 8 == 0, "the kernels address rows of L2 elements with 16-byte steps (attention() pads other L2)"

        st = _status_of(q.device)
        st.raise_if_set()  # an earlier call's device-side failure, seen through the host mirror
        q, k, v, b_pw = _dense(q), _dense(k), _dense(v), _dense(b_pw)
        L2p = _l2p(L2)
        L = _cabi.lib()
        prob = _problem(q)
        o = torch.empty((B, H, L1, L2, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((3, B, H, L1, L2p), dtype=torch.float32, device=q.device)  # softmax statistics
        # the bits of O that rounding to bf16 drops, for the backward's delta (fp16 keeps enough)
        need_bwd = any(ctx.needs_input_grad[:4])
        o_res = torch.empty_like(o) if (need_bwd and _SAVE_O_RESIDUAL and q.dtype == torch.bfloat16) else None
        with torch.cuda.device(q.device):
            stream = torch.cuda.current_stream().cuda_stream
            bias_k = b_pw  # what the kernels read
            if key_mask is not None or L2p != L2:
                # Ragged L2 and / or a boolean key mask: only this bias-sized tensor is staged (whole
                # 128-blocks, -inf on padding and masked keys); q, k, v are read in place.
                km = None
                if key_mask is not None:
                    assert key_mask.dtype == torch.bool and key_mask.shape == (B, L2), "key_mask: bool (B, L2)"
                    km = key_mask.to(device=q.device, dtype=torch.uint8).contiguous()
                bias_k = torch.empty((B, H, L2p, L2p), dtype=q.dtype, device=q.device)
                check(L.fta_mask_bias(prob, t4(b_pw), None if km is None else km.data_ptr(), bias_k.data_ptr(), stream),
                      "fta_mask_bias")
            check(L.fta_forward(prob, t5(q), t5(k), t5(v), t4(bias_k), float(sm_scale), t5(o),
                                None if o_res is None else o_res.data_ptr(),
                                lse.data_ptr(), st.word.data_ptr(), stream), "fta_forward")
            st.publish()
        if _DEBUG:
            check_device_status(q.device)
        ctx.save_for_backward(q, k, v, o, bias_k, lse, o_res)
        ctx.sm_scale = float(sm_scale)
        ctx.group = group
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, bias_k, lse, o_res = ctx.saved_tensors
        assert do.dtype == q.dtype
        do = _dense(do)
        B, H, L1, L2, D = q.shape
        L2p = _l2p(L2)
        dev = q.device
        dq = torch.empty((B, H, L1, L2, D), dtype=q.dtype, device=dev)
        dk = torch.empty_like(dq)
        dv = torch.empty_like(dq)
        db = torch.empty((B, H, L2, L2), dtype=q.dtype, device=dev)
        db32 = torch.empty((B, H, L2, L2), dtype=torch.float32, device=dev)
        delta = torch.empty((B, H, L1, L2p), dtype=torch.float32, device=dev)
        prob = _problem(q)
        L = _cabi.lib()
        ws_bytes = int(L.fta_bwd_workspace_bytes(prob))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        st = _status_of(dev)
        st.raise_if_set()
        status = st.word
        sharded = ctx.group is not None
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream().cuda_stream
            check(L.fta_bwd_preprocess(prob, t5(o), None if o_res is None else o_res.data_ptr(), t5(do),
                                       delta.data_ptr(), stream), "fta_bwd_preprocess")
            check(L.fta_backward(prob, t5(q), t5(k), t5(v), t4(bias_k), t5(do), lse.data_ptr(), delta.data_ptr(),
                                 ctx.sm_scale, t5(dq), t5(dk), t5(dv), db32.data_ptr(),
                                 None if sharded else db.data_ptr(), ws.data_ptr(), ws_bytes,
                                 status.data_ptr(), stream), "fta_backward")
            if sharded:
                # the only collective of the path: sum the per-rank partial dBias over NVLink
                torch.distributed.all_reduce(db32, op=torch.distributed.ReduceOp.SUM, group=ctx.group)
                check(L.fta_dbias_cast(db32.data_ptr(), db.data_ptr(), db32.numel(), prob.dtype, stream),
                      "fta_dbias_cast")
            st.publish()
        if _DEBUG:
            check_device_status(dev)
        _last["dbias_f32"] = db32
        return dq, dk, dv, db, None, None, None


def attention(q, k, v, b_pw, sm_scale, group=None, key_mask=None):
    """Fused triangle attention: ``softmax(q k^T * sm_scale + b_pw) v`` for q, k, v of shape
    (B, H, L1, L2, D) and a pair bias (B, H, L2, L2) shared by the L1 rows; differentiable in
    q, k, v and b_pw (dBias is summed over L1). See the module docstring.

    Two extensions of the reference's call (flash_tt_attn.py:663; its README lists both as to-do,
    README.md:17-18): ``key_mask`` (bool (B, L2), or anything that broadcasts to (B, 1, 1, L2);
    True = attend) removes keys, and ``L2`` need not be a multiple of 128. Both are handled inside
    the kernels - ragged last blocks are padded by the tile loads and clipped by the stores, masked
    keys get exactly zero probability and exactly zero dBias, dK, dV - and only a bias-sized tensor
    is staged; q, k, v are never copied. (An ``L2`` that is not a multiple of 8 is first padded to
    one: the kernels step through rows of ``L2`` elements 16 bytes at a time.) A query whose every
    key is masked gets a zero output row and zero gradients."""
    B, H, L1, L2, D = q.shape
    if key_mask is not None:
        if key_mask.dim() == 4:
            key_mask = key_mask.reshape(key_mask.shape[0], L2)
        key_mask = key_mask.expand(B, L2)
    if L2 % 8 == 0:
        return _attention.apply(q, k, v, b_pw, sm_scale, group, key_mask)
    pad = (L2 + 7) // 8 * 8 - L2
    F = torch.nn.functional  # F.pad is differentiable: gradients of the padding are dropped on the way back
    if key_mask is None:
        key_mask = torch.ones((B, L2), dtype=torch.bool, device=q.device)
    out = _attention.apply(F.pad(q, (0, 0, 0, pad)), F.pad(k, (0, 0, 0, pad)), F.pad(v, (0, 0, 0, pad)),
                           F.pad(b_pw, (0, pad, 0, pad)), sm_scale, group, F.pad(key_mask, (0, pad), value=False))
    return out[:, :, :, :L2]


def reference_tt_attn(q, k, v, b, sm_scale):
    """Naive PyTorch statement of the op (what the reference's function of the same name
    computes, flash_tt_attn.py:845-864): logits in the input dtype, softmax in float32, the
    probabilities cast back to ``v.dtype``. Materialises (B,H,L1,L2,L2); for checks only."""
    logits = torch.einsum("bhijd,bhikd->bhijk", q, k) * sm_scale + b.unsqueeze(2)
    p = torch.softmax(logits.float(), dim=-1).to(v.dtype)
    return torch.einsum("bhijk,bhikd->bhijd", p, v)


def shard_plan(H: int, L1: int, rank: int, world: int):
    """How ``world`` ranks split one triangle-attention problem: heads first, L1 rows second.

    Heads are independent problems INCLUDING their dBias, so ranks that own different heads never
    exchange anything; only ranks that share a head (they own different blocks of its L1 rows)
    sum their float32 dBias. ``gcd(world, H)`` head shards, ``world / gcd`` row shards per head
    shard; ranks of one head shard are consecutive.

    Returns ``(heads, rows, peers)``: this rank's slice of H, its slice of L1, and the ranks it
    all-reduces dBias with (a list; of length 1 when no collective is needed)."""
    import math
    hs = math.gcd(world, H)
    rs = world // hs
    hi, ri = rank // rs, rank % rs
    per_h = H // hs
    heads = slice(hi * per_h, (hi + 1) * per_h)
    return heads, shard_rows(L1, ri, rs), list(range(hi * rs, (hi + 1) * rs))


def shard_rows(L1: int, rank: int, world: int) -> slice:
    """Contiguous block of L1 rows owned by ``rank`` (rows are independent problems)."""
    per = (L1 + world - 1) // world
    return slice(min(L1, rank * per), min(L1, (rank + 1) * per))


class PeerDbiasSum:
    """The cross-GPU sum of dBias over NVLink peer memory instead of an NCCL all-reduce.

    Every rank of ``group`` keeps its float32 partial dBias in a buffer that the other ranks can
    address (``torch.distributed._symmetric_memory``: one allocation per rank, exchanged once at
    construction - a collective call). ``partial()`` is the tensor to hand to ``fta_backward`` as
    ``dbias_f32``; ``reduce()`` is one launch of ``fta_dbias_sum_peers_sync``: the kernel lines the ranks
    up itself (epoch words the ranks write into each other's memory, a bounded wait), then each rank
    reads all partials, adds them in rank order and rounds once - one short kernel where the
    all-reduce is a ~30-50 us collective plus a cast. Two partial buffers are used in turn, so that a rank may write its next partial
    while a slower peer still reads the previous one. Every rank reading (world - 1) partials pays
    for pairs (an 8-GPU heads-first split); larger groups use ``reduce_sliced``: each rank sums a
    1/world slice and stores the rounded result into every rank's (symmetric) output buffer. Construction raises where symmetric memory is unavailable: callers fall back
    to ``torch.distributed.all_reduce`` + ``fta_dbias_cast``."""

    def __init__(self, shape, group, device, dtype):
        # no NVLink multicast binding: plain peer mappings only
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.shape = tuple(shape)
        self.n = 1
        for d in self.shape:
            self.n *= int(d)
        assert self.n % 8 == 0
        self.dtype_code = _cabi.FTA_BF16 if dtype == torch.bfloat16 else _cabi.FTA_FP16
        self.buf = symm_mem.empty((2, self.n), dtype=torch.float32, device=device)
        self.hdl = symm_mem.rendezvous(self.buf, group)
        self.world = int(self.hdl.world_size)
        base = [int(p) for p in self.hdl.buffer_ptrs]
        self.parts = [torch.tensor([p + slot * self.n * 4 for p in base], dtype=torch.int64, device=device)
                      for slot in (0, 1)]
        # epoch words for the line-up inside the kernel (fta_dbias_sum_peers_sync): one array of `world`
        # words per rank, written by the peers; zero on every rank before anybody's first launch
        self.flags = symm_mem.empty((64,), dtype=torch.int32, device=device)
        self.flags.zero_()
        self.flags_hdl = symm_mem.rendezvous(self.flags, group)
        self._flag_ptrs = torch.tensor([int(p) for p in self.flags_hdl.buffer_ptrs], dtype=torch.int64, device=device)
        self.rank = int(self.hdl.rank)
        self.status = _status_of(torch.device(device))
        self.flags_hdl.barrier(channel=0)
        # groups of more than two: each rank sums a slice and stores the rounded result into every
        # rank's output buffer (fta_dbias_sum_peers_sliced), also symmetric memory
        self.sliced = self.world > 2
        if self.sliced:
            self.out = symm_mem.empty((self.n,), dtype=dtype, device=device)
            self.out_hdl = symm_mem.rendezvous(self.out, group)
            self._outs = torch.tensor([int(p) for p in self.out_hdl.buffer_ptrs], dtype=torch.int64, device=device)
        self._views = [self.buf[slot].view(self.shape) for slot in (0, 1)]
        self._ptrs = [v.data_ptr() for v in self._views]
        self._parts_ptrs = [t.data_ptr() for t in self.parts]
        self._lib = _cabi.lib()
        self.step = 0

    def partial(self):
        """This rank's float32 partial for the current step (pass it as ``dbias_f32``)."""
        return self._views[self.step & 1]

    def partial_ptr(self):
        return self._ptrs[self.step & 1]

    def reduce(self, out_cast, out_f32=None, stream=None, wait_limit_ns=0):
        """After this rank's ``fta_backward`` has been enqueued: ONE launch that lines the ranks up (epoch
        words in peer memory, bounded wait: a peer that never arrives leaves a code in the status word
        instead of a hang), sums the partials in rank order and rounds."""
        stream = torch.cuda.current_stream(self.buf.device).cuda_stream if stream is None else stream
        check(self._lib.fta_dbias_sum_peers_sync(self._parts_ptrs[self.step & 1], self._flag_ptrs.data_ptr(), self.world,
                                                 self.rank, self.step + 1, self.n,
                                                 None if out_f32 is None else out_f32.data_ptr(),
                                                 None if out_cast is None else out_cast.data_ptr(), self.dtype_code,
                                                 int(wait_limit_ns), self.status.word.data_ptr(), stream),
              "fta_dbias_sum_peers_sync")
        self.step += 1

    def reduce_sliced(self, stream=None, wait_limit_ns=0):
        """Groups of more than two ranks: every rank sums its 1/world slice and stores the rounded result
        into every rank's output buffer; the line-ups before (partials complete) and after (all slices
        arrived) happen inside the two kernels ``fta_dbias_sum_peers_sliced_sync`` enqueues, with bounded
        waits. Returns this rank's output buffer (shape of the partial, bias dtype): complete for work
        enqueued on the same stream after this call, valid until the next ``reduce_sliced``."""
        assert self.sliced
        stream = torch.cuda.current_stream(self.buf.device).cuda_stream if stream is None else stream
        check(self._lib.fta_dbias_sum_peers_sliced_sync(self._parts_ptrs[self.step & 1], self._outs.data_ptr(),
                                                        self._flag_ptrs.data_ptr(), self.flags.data_ptr(), self.world,
                                                        self.rank, self.step + 1, self.n, self.dtype_code,
                                                        int(wait_limit_ns), self.status.word.data_ptr(), stream),
              "fta_dbias_sum_peers_sliced_sync")
        self.step += 1
        return self.out.view(self.shape)


def _block_sizes(L1: int, block_rows: int):
    """Blocks of L1 rows for the streamed entry point: full blocks in the middle, a third and two
    thirds of a block at either end, so that the first copy in and the last copy out (which nothing
    overlaps) are short."""
    ramp = [max(1, block_rows // 3), max(1, 2 * block_rows // 3)]
    if L1 <= 3 * block_rows:
        return [block_rows] * (L1 // block_rows) + ([L1 % block_rows] if L1 % block_rows else [])
    left = L1 - 2 * sum(ramp)
    sizes = ramp + [block_rows] * (left // block_rows)
    if left % block_rows:
        sizes.append(left % block_rows)
    return sizes + ramp[::-1]


def _copy_rows(lib, dst, dst_row0, src, src_row0, nrows, stream):
    """Rows [row0, row0 + nrows) of the L1 axis of every (b, h): one strided transfer. Both tensors
    are (B, H, *, L2, D) and dense in their last two axes and across (b, h)."""
    B, H = dst.shape[0], dst.shape[1]
    es = dst.element_size()
    row = dst.shape[3] * dst.shape[4] * es
    # one pitch for every (b, h) slab (the stride of a size-1 batch axis carries no meaning)
    assert B == 1 or (dst.stride(0) == H * dst.stride(1) and src.stride(0) == H * src.stride(1))
    assert dst.stride(2) * es == row and src.stride(2) * es == row
    check(lib.fta_memcpy_2d(dst.data_ptr() + dst_row0 * row, dst.stride(1) * es, src.data_ptr() + src_row0 * row,
                            src.stride(1) * es, nrows * row, B * H, stream), "fta_memcpy_2d")


def attention_fwd_bwd_streamed(host, sm_scale, out, block_rows=96, device=None, group=None):
    """Forward + backward for tensors that live in (pinned) HOST memory, streamed through the GPU
    in blocks of L1 rows: the copies of block i+1 (host to device) and of the results of block
    i-1 (device to host) run on their own streams while the kernels of block i run, so a call
    costs about max(copy in, copy out, compute) instead of their sum. Rows of L1 are independent
    problems; only dBias couples them, and it is summed over the blocks in float32, in block
    order, and rounded once. Each block moves with one strided transfer per tensor
    (``fta_memcpy_2d``) through three device slots, and its kernels are enqueued straight through
    the C ABI on buffers allocated once per call (no autograd graph: a block costs the host a
    fraction of a millisecond, which matters because a block's kernels run for about as long).

    host : dict with ``q, k, v, do`` of shape (B, H, L1, L2, D) and ``bias`` (B, H, L2, L2), CPU
           tensors (pinned for asynchronous copies), contiguous, 16-bit dtype; L2 a multiple of 8
    out  : dict with ``o, dq, dk, dv`` like ``q`` and ``dbias`` like ``bias``, CPU tensors (pinned)
    group: with a process group, ``host`` holds this rank's rows and dBias is all-reduced once.
    Returns after everything has arrived in ``out``.
    """
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    q_h, b_h = host["q"], host["bias"]
    B, H, L1, L2, D = q_h.shape
    assert L2 % 8 == 0 and D in (32, 64) and q_h.dtype in (torch.float16, torch.bfloat16)
    L = _cabi.lib()
    NSLOT = 3
    names_in, names_out = ("q", "k", "v", "do"), ("o", "dq", "dk", "dv")
    for t in [host[n] for n in names_in] + [out[n] for n in names_out]:
        assert t.is_contiguous() and t.shape == q_h.shape and t.dtype == q_h.dtype
    dtype_code = _cabi.FTA_BF16 if q_h.dtype == torch.bfloat16 else _cabi.FTA_FP16
    L2p = _l2p(L2)
    with torch.cuda.device(dev):
        cur = torch.cuda.current_stream(dev)
        st = _status_of(dev)
        st.raise_if_set()
        # the two copy streams are kept per device: every new side stream has its own allocator pool,
        # and a tensor allocated under it costs a cudaMalloc per call until the pools have filled up
        key = (dev.type, dev.index)
        if key not in _copy_streams:
            _copy_streams[key] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
        s_in, s_out = _copy_streams[key]
        sizes = _block_sizes(L1, block_rows)
        cap = max(sizes)
        mk = lambda *shape, dtype=q_h.dtype: torch.empty(shape, dtype=dtype, device=dev)
        slots = [{**{k: mk(B, H, cap, L2, D) for k in names_in + names_out}, "ores": mk(B, H, cap, L2, D),
                  "lse": mk(3, B, H, cap, L2p, dtype=torch.float32), "delta": mk(B, H, cap, L2p, dtype=torch.float32)}
                 for _ in range(NSLOT)]
        ws_bytes = int(L.fta_bwd_workspace_bytes(FtaProblem(B, H, cap, L2, D, dtype_code)))
        ws = mk(ws_bytes, dtype=torch.uint8)
        ev_in = [torch.cuda.Event() for _ in range(NSLOT)]
        ev_comp = [torch.cuda.Event() for _ in range(NSLOT)]
        ev_out = [torch.cuda.Event() for _ in range(NSLOT)]
        bias = torch.empty(b_h.shape, dtype=b_h.dtype, device=dev)  # from the current stream's pool
        s_in.wait_stream(cur)
        with torch.cuda.stream(s_in):
            bias.copy_(b_h, non_blocking=True)
        cur.wait_stream(s_in)
        bias_k = bias
        if L2p != L2:
            bias_k = mk(B, H, L2p, L2p)
            check(L.fta_mask_bias(FtaProblem(B, H, 1, L2, D, dtype_code), t4(bias), None, bias_k.data_ptr(), cur.cuda_stream),
                  "fta_mask_bias")
        bias4 = t4(bias_k)
        db32 = torch.zeros((B, H, L2, L2), dtype=torch.float32, device=dev)
        db_blk = torch.empty_like(db32)
        resid = q_h.dtype == torch.bfloat16 and _SAVE_O_RESIDUAL
        r0 = 0
        for blk, n in enumerate(sizes):
            slot = blk % NSLOT
            sl = slots[slot]
            if blk >= NSLOT:
                s_in.wait_event(ev_comp[slot])  # the kernels of block blk - NSLOT have read this slot's inputs
                cur.wait_event(ev_out[slot])    # ... and its results are on their way out of the output buffers
            for name in names_in:
                _copy_rows(L, sl[name], 0, host[name], r0, n, s_in.cuda_stream)
            ev_in[slot].record(s_in)
            cur.wait_event(ev_in[slot])
            prob = FtaProblem(B, H, n, L2, D, dtype_code)
            v5 = {k: t5(sl[k][:, :, :n]) for k in names_in + names_out}
            ores_ptr = sl["ores"].data_ptr() if resid else None
            # the residual buffer is addressed with the strides of `o` (the slot's full block)
            check(L.fta_forward(prob, v5["q"], v5["k"], v5["v"], bias4, float(sm_scale), v5["o"], ores_ptr,
                                sl["lse"].data_ptr(), st.word.data_ptr(), cur.cuda_stream), "fta_forward")
            check(L.fta_bwd_preprocess(prob, v5["o"], ores_ptr, v5["do"], sl["delta"].data_ptr(), cur.cuda_stream),
                  "fta_bwd_preprocess")
            check(L.fta_backward(prob, v5["q"], v5["k"], v5["v"], bias4, v5["do"], sl["lse"].data_ptr(),
                                 sl["delta"].data_ptr(), float(sm_scale), v5["dq"], v5["dk"], v5["dv"],
                                 db_blk.data_ptr(), None, ws.data_ptr(), ws_bytes, st.word.data_ptr(), cur.cuda_stream),
                  "fta_backward")
            db32 += db_blk
            ev_comp[slot].record(cur)
            s_out.wait_event(ev_comp[slot])
            for name in names_out:
                _copy_rows(L, out[name], r0, sl[name], 0, n, s_out.cuda_stream)
            ev_out[slot].record(s_out)
            r0 += n
        if group is not None:
            torch.distributed.all_reduce(db32, op=torch.distributed.ReduceOp.SUM, group=group)
        out["dbias"].copy_(db32.to(b_h.dtype), non_blocking=True)
        _last["dbias_f32"] = db32
        st.publish()
        cur.wait_stream(s_out)
        torch.cuda.synchronize(dev)
    check_device_status(dev)
