/* libfta: B200 (sm_100a) triangle attention, C ABI.
 *
 * Drop-in kernels for the hot path of BryanZWu/flash-triangle-attention: the three Triton
 * launches behind `flash_tt_attn.attention` (forward; backward preprocess + backward).
 * For q, k, v of shape (B,H,L1,L2,D) and a pair bias of shape (B,H,L2,L2) shared by the L1
 * rows:
 *     S = sm_scale * q k^T + bias ;  P = softmax_k(S) ;  O = P v
 *     dV = P^T dO ; dP = dO v^T ; dS = P (dP - rowsum(dO O))
 *     dQ = sm_scale dS k ; dK = sm_scale dS^T q ; dBias = sum over L1 of dS
 *
 * Conventions
 *  - plain pointers, sizes and element strides; no framework types;
 *  - every pointer is a DEVICE pointer on the current CUDA device unless stated otherwise;
 *  - the library never allocates or frees device memory: outputs, the log-sum-exp, the
 *    workspace and the status word belong to the caller;
 *  - all work is enqueued on `stream` (a cudaStream_t passed as void*); calls return
 *    without synchronising;
 *  - return value 0 on success, a negative FTA_ERR_* otherwise; bad arguments are rejected
 *    on the host before anything is launched; nothing traps or asserts on the device;
 *  - device-side waits are bounded; a wait that runs out writes a non-zero code to the
 *    caller's status word (see fta_read_status) and the kernel returns;
 *  - supported: dtype fp16 / bf16 (q, k, v, bias, o, dO and the gradients share it),
 *    D in {32, 64}, any L1 >= 1 (L1 != L2 is fine: a shard of rows), innermost (D) stride 1 and
 *    16-byte aligned rows; L2 a multiple of 128, or any multiple of 8 with the bias passed
 *    through fta_mask_bias first (ragged last blocks are padded on the fly by the loads and
 *    clipped by the stores: q, k, v, dO and the outputs are never copied);
 *  - L2p below is L2 rounded up to a multiple of 128; the softmax statistics and delta have rows
 *    of L2p floats (the kernels move them in whole 128-query blocks);
 *  - every device pointer handed to the library (tensors, lse, delta, dBias buffers, the optional
 *    residual) must be 16-byte aligned, the workspace 256-byte aligned: FTA_ERR_ALIGN /
 *    FTA_ERR_WORKSPACE otherwise (the kernels move data with 16-byte vectors and bulk copies).
 */
#ifndef FTA_H_
#define FTA_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define FTA_API __attribute__((visibility("default")))
#else
#define FTA_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum { FTA_FP16 = 0, FTA_BF16 = 1 };

enum {
  FTA_OK = 0,
  FTA_ERR_NULL = -1,       /* a required pointer is NULL */
  FTA_ERR_SHAPE = -2,      /* non-positive size, or L2 not a multiple of 8 */
  FTA_ERR_HEAD_DIM = -3,   /* D not in {32, 64} */
  FTA_ERR_DTYPE = -4,      /* dtype not FTA_FP16 / FTA_BF16 */
  FTA_ERR_STRIDE = -5,     /* D stride != 1, or a stride that is not a multiple of 8 elements */
  FTA_ERR_ALIGN = -6,      /* a device pointer that is not 16-byte aligned */
  FTA_ERR_WORKSPACE = -7,  /* workspace too small */
  FTA_ERR_TENSOR_MAP = -8, /* the driver refused a TMA tensor map */
  FTA_ERR_CUDA = -9,       /* a CUDA runtime call failed (see fta_last_cuda_error) */
  FTA_ERR_DEVICE = -10,    /* status word non-zero: a bounded device wait ran out */
  FTA_ERR_TOO_LARGE = -11  /* size beyond a documented maximum */
};

typedef struct FtaProblem {
  int32_t B, H, L1, L2, D;
  int32_t dtype; /* FTA_FP16 or FTA_BF16 */
} FtaProblem;

/* (B,H,L1,L2,D) tensor: base pointer + element strides of the five dimensions. */
typedef struct FtaTensor5 {
  void* ptr;
  int64_t stride[5];
} FtaTensor5;

/* (B,H,L2,L2) pair bias: base pointer + element strides (query index, then key index). */
typedef struct FtaTensor4 {
  void* ptr;
  int64_t stride[4];
} FtaTensor4;

/* Library version (major*10000 + minor*100 + patch). */
FTA_API int fta_version(void);

/* Text for an FTA_ERR_* code. Never NULL. */
FTA_API const char* fta_strerror(int code);

/* cudaError_t of the last failing CUDA call made by this library on this thread. */
FTA_API int fta_last_cuda_error(void);

/* Forward pass. Replaces the `_attn_fwd` launch of `_attention.forward`
 * (flash_tt_attn.py:556-593, kernel 128-264): writes O (same dtype as q) and the softmax
 * statistics of every query row for the backward pass, `lse`, float32 contiguous of shape
 * (3,B,H,L1,L2p): plane 0 holds -max_k(S) in natural-log units, plane 1 holds
 * -log2(sum_k exp(S - max)). The reference saves their combination, the base-2
 * log-sum-exp max*log2(e) + log2(sum) (flash_tt_attn.py:258-263) = -(plane0*log2(e) + plane1);
 * the two parts are kept apart here because their float32 sum loses log2(sum) when a row is
 * fully masked with a large negative bias (|max| ~ 1e9). Plane 2 holds that combination,
 * plane0*log2(e) + plane1, for rows with |max| <= 1e4 (the backward pass then needs one
 * statistic per row) and NaN for the others (the backward pass uses planes 0 and 1).
 * `o_resid` is optional (NULL: not written): a buffer with the dtype and the strides of `o` that
 * receives the part of O lost when it is rounded to 16 bits, dtype(O_f32 - dtype(O_f32)). Handed
 * to fta_bwd_preprocess it makes delta = rowsum(dO * O) as if O had 16 mantissa bits; with bf16
 * and O rounded to 8 bits the error of delta alone costs about 0.01 max-abs in a dBias summed
 * over several hundred rows. The reference has no such output (it is fp16 only).
 * `bias` spans whole 128-blocks: the caller's (B,H,L2,L2) tensor when L2 is a multiple of 128,
 * else the (B,H,L2p,L2p) copy made by fta_mask_bias (also the way to drop keys with a mask).
 * `status` points to one int32 the caller zeroed. */
FTA_API int fta_forward(const FtaProblem* prob, const FtaTensor5* q, const FtaTensor5* k,
                const FtaTensor5* v, const FtaTensor4* bias, float sm_scale,
                const FtaTensor5* o, void* o_resid, float* lse, int32_t* status, void* stream);

/* Backward preprocess. Replaces `_attn_bwd_preprocess` (flash_tt_attn.py:266-288, launched
 * at 636-641): delta[b,h,i,j] = sum_d O[b,h,i,j,d] * dO[b,h,i,j,d], float32, shape (B,H,L1,L2p)
 * contiguous (entries j >= L2 are set to 0).
 * `o_resid` (may be NULL) is the residual fta_forward wrote, laid out like `o`: when given,
 * O + residual takes the place of O. */
FTA_API int fta_bwd_preprocess(const FtaProblem* prob, const FtaTensor5* o, const void* o_resid,
                       const FtaTensor5* dout, float* delta, void* stream);

/* Padded, masked copy of the pair bias, for problems whose L2 is not a multiple of 128 and / or
 * that remove keys with a boolean mask (the reference's roadmap items, README.md:17-18; its
 * kernels have neither). `out` is (B,H,L2p,L2p) contiguous in the bias dtype:
 *     out[b,h,q,k] = bias[b,h,q,k]   for q, k < L2 and key_mask[b,k] != 0
 *                  = -inf            for every other key k (masked, or padding k >= L2)
 *                  = 0               for kept keys of the padding queries q >= L2
 * `key_mask` is (B,L2) bytes on the device, 8-byte aligned, non-zero = attend; NULL keeps every
 * key. Pass `out` as the bias (strides L2p*L2p*H, L2p*L2p, L2p, 1) to fta_forward and
 * fta_backward: masked keys then get exactly zero probability and exactly zero dBias / dK / dV;
 * a query whose every key is masked gets O = 0 and zero gradients. dBias is still returned
 * as (B,H,L2,L2). Only this bias-sized tensor is staged; q, k, v, dO are read in place. */
FTA_API int fta_mask_bias(const FtaProblem* prob, const FtaTensor4* bias, const uint8_t* key_mask, void* out,
                          void* stream);

/* Bytes of workspace fta_backward needs for `prob` (a float32 dQ accumulator and the
 * partial dBias planes). 256-byte aligned workspace required. */
FTA_API size_t fta_bwd_workspace_bytes(const FtaProblem* prob);

/* Number of partial dBias planes the backward kernel produces for `prob` (each plane is
 * the sum of dS over a fixed subset of the L1 rows; they are summed in plane order). */
FTA_API int fta_bwd_num_planes(const FtaProblem* prob);

/* Backward pass. Replaces the `_attn_bwd` launch and the `zeros_like` dBias buffer of
 * `_attention.backward` (flash_tt_attn.py:596-660, kernel 442-550). Needs `lse` (all three planes) from
 * fta_forward and `delta` from fta_bwd_preprocess. Writes dq, dk, dv (dtype of q), the
 * float32 dBias `dbias_f32` (B,H,L2,L2 contiguous; the sum over this call's L1 rows, in a
 * fixed order, so bit-reproducible) and, when `dbias_cast` is not NULL, the same rounded to
 * the bias dtype (what the reference returns, flash_tt_attn.py:613). A caller that shards L1
 * over several GPUs passes dbias_cast = NULL, sums dbias_f32 over ranks and then calls
 * fta_dbias_cast. */
FTA_API int fta_backward(const FtaProblem* prob, const FtaTensor5* q, const FtaTensor5* k,
                 const FtaTensor5* v, const FtaTensor4* bias, const FtaTensor5* dout,
                 const float* lse, const float* delta, float sm_scale, const FtaTensor5* dq,
                 const FtaTensor5* dk, const FtaTensor5* dv, float* dbias_f32, void* dbias_cast,
                 void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* dst[i] = (dtype) src[i] for n elements (n a multiple of 4): the final rounding of dBias to
 * the bias dtype after a cross-GPU sum (the reference accumulates directly in that dtype,
 * flash_tt_attn.py:425-426, 613). */
FTA_API int fta_dbias_cast(const float* src, void* dst, int64_t n, int32_t dtype, void* stream);

/* The cross-GPU sum of dBias and its rounding in one kernel, over peer memory instead of a
 * library collective: out[i] = sum over r = 0 .. nranks-1 (in that order, so every rank gets the same
 * bits) of parts[r][i], written as float32 (`out_f32`, may be NULL) and / or rounded to the bias
 * dtype (`out_cast`, may be NULL). `parts` is a DEVICE array of `nranks` device pointers: entry r
 * addresses rank r's float32 partial (the `dbias_f32` of its fta_backward) as this GPU sees it - its
 * own buffer, or a peer mapping (CUDA IPC / virtual-memory export, NVLink). n a multiple of 8, buffers
 * 16-byte aligned. The kernel only reads and adds: the caller makes sure that every rank's partial is
 * complete before this launch (a barrier between the ranks on the streams involved) and is not
 * rewritten until every rank's launch has finished (e.g. two partial buffers used in turn). Stands
 * where the reference has its fp16 atomics into one buffer (flash_tt_attn.py:425-426): the
 * reference itself is single-GPU. */
FTA_API int fta_dbias_sum_peers(const float* const* parts, int32_t nranks, int64_t n, float* out_f32,
                        void* out_cast, int32_t dtype, void* stream);

/* fta_dbias_sum_peers with the line-up of the ranks inside the kernel, so that the sum is ONE launch
 * per rank and step with no barrier launch and no library collective. `flags`: device array of
 * `nranks` device pointers, entry r = rank r's array of `nranks` int32 epoch words as this GPU sees it
 * (zero before the first call, in memory every rank can write: the same kind of peer mapping as the
 * partials). `epoch` = 1, 2, 3, ... the same on every rank for the same step. The kernel publishes
 * "rank `rank`'s partial of this epoch is complete" (it was written by earlier work on `stream`) into
 * every rank's words, waits until all `nranks` words of this rank have reached `epoch`, then sums.
 * The wait is bounded: after `wait_limit_ns` (0 = one second) of the GPU's global timer the kernel
 * writes 0x1000 | 0x61 to `status` and returns without output - nothing traps, the context stays
 * usable. Partials must alternate between two buffers from step to step (a rank may be one step ahead
 * of a peer that is still reading). One process per GPU: never two ranks as kernels on one GPU.
 * No counterpart in the reference. */
FTA_API int fta_dbias_sum_peers_sync(const float* const* parts, int32_t* const* flags, int32_t nranks,
                             int32_t rank, int32_t epoch, int64_t n, float* out_f32, void* out_cast,
                             int32_t dtype, uint64_t wait_limit_ns, int32_t* status, void* stream);

/* The same sum with the work split over the ranks (reduce-scatter and all-gather in one kernel), for
 * groups where every rank reading every partial would be too much traffic: rank `rank` adds the
 * partials of its 1/nranks slice of the elements (rank order), rounds, and stores the 16-bit result
 * into EVERY rank's output buffer. `outs`: device array of `nranks` device pointers to the ranks'
 * (n-element, 16-bit, 16-byte aligned) output buffers as this GPU sees them. The caller lines the ranks
 * up before the launch (partials complete, previous outputs consumed) and once more after it: a rank's
 * output buffer is complete when every rank's launch has finished. No counterpart in the reference. */
FTA_API int fta_dbias_sum_peers_sliced(const float* const* parts, void* const* outs, int32_t nranks,
                               int32_t rank, int64_t n, int32_t dtype, void* stream);

/* fta_dbias_sum_peers_sliced with both line-ups inside: the ranks wait for each other's partials in the
 * kernel (as in fta_dbias_sum_peers_sync; words [0, nranks) of a rank's flag array), each rank
 * publishes "my slice is in your buffer" when its last block is done (words [nranks, 2 nranks); word
 * 2 nranks of a rank's OWN array is the block counter), and a one-block kernel enqueued behind the sum
 * holds `stream` until all slices have arrived: work enqueued after this call sees the complete result
 * in this rank's output buffer. `flags`: device array of the ranks' flag arrays (2 nranks + 1 int32
 * each, zero before the first call) as this GPU sees them; `my_flags`: this rank's own array (local
 * address). Same epoch rule, same bounded waits (status 0x1000 | 0x62 / 0x63), nranks <= 31.
 * No counterpart in the reference. */
FTA_API int fta_dbias_sum_peers_sliced_sync(const float* const* parts, void* const* outs, int32_t* const* flags,
                                    const int32_t* my_flags, int32_t nranks, int32_t rank, int32_t epoch,
                                    int64_t n, int32_t dtype, uint64_t wait_limit_ns, int32_t* status,
                                    void* stream);

/* Backward pass without a caller-provided workspace. It has no counterpart in the reference.
 * For callers that cannot allocate device memory where they call this library (a framework's
 * memory-planning phase, a plugin interface that only passes inputs and outputs, a loop that
 * forbids cudaMalloc): same arguments and results as fta_backward, but the scratch memory is a
 * fixed array inside the library, fta_noalloc_max_bytes() long (64 MiB), present once on every
 * GPU that loads the library until the process exits. Nothing is allocated or freed.
 *  - Problems whose fta_bwd_workspace_bytes() exceeds that size are rejected with
 *    FTA_ERR_TOO_LARGE before anything is launched.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current); make that first call before any stream capture.
 *  - All calls on a device share the one array: two calls whose work overlaps on the GPU
 *    (different streams, different threads) race on it. Keep them on one stream, or order them.
 *    The array keeps what the last call wrote; each call clears or overwrites what it reads.
 *  - The looked-up address is cached per device for the life of the process; it does not survive
 *    a cudaDeviceReset of that device. */
FTA_API int fta_backward_noalloc(const FtaProblem* prob, const FtaTensor5* q, const FtaTensor5* k,
                                 const FtaTensor5* v, const FtaTensor4* bias, const FtaTensor5* dout,
                                 const float* lse, const float* delta, float sm_scale,
                                 const FtaTensor5* dq, const FtaTensor5* dk, const FtaTensor5* dv,
                                 float* dbias_f32, void* dbias_cast, int32_t* status, void* stream);

/* Size in bytes of the fixed scratch array used by fta_backward_noalloc. */
FTA_API size_t fta_noalloc_max_bytes(void);

/* Strided block copy on `stream`: `rows` pieces of `width_bytes`, `src_pitch_bytes` apart in the
 * source and `dst_pitch_bytes` apart in the destination (one cudaMemcpy2DAsync; either side may be
 * pinned host or device memory, the direction is inferred from the pointers). What the host-memory
 * entry point of the Python module uses to move a block of L1 rows of every (b,h) of a
 * (B,H,L1,L2,D) tensor with ONE transfer per tensor instead of one per (b,h). It has no
 * counterpart in the reference (whose tensors always live on the device). */
FTA_API int fta_memcpy_2d(void* dst, size_t dst_pitch_bytes, const void* src, size_t src_pitch_bytes,
                          size_t width_bytes, size_t rows, void* stream);

/* Profiling hook, off by default. After this call, every fta_backward on the calling thread
 * records `start_event` right before and `stop_event` right after its main kernel (the
 * tcgen05 backward kernel, excluding the memset, transpose and finalise kernels around it) on
 * the stream it is given. Both are cudaEvent_t passed as void*; NULL, NULL switches it off.
 * No counterpart in the reference (it times whole calls with do_bench, flash_tt_attn.py:804). */
FTA_API int fta_profile_backward_kernel(void* start_event, void* stop_event);

/* Copies the status word to the host and synchronises `stream`. Returns FTA_OK when it is
 * zero, FTA_ERR_DEVICE otherwise; `*code_out` (host pointer, may be NULL) receives the raw
 * word: 0x1000 | site for a wait that ran out. */
FTA_API int fta_read_status(const int32_t* status, int32_t* code_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FTA_H_ */
