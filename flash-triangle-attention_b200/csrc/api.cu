// C ABI of libfta (declared in include/fta.h): argument validation, TMA tensor maps, launches.
// Nothing here allocates device memory; every buffer belongs to the caller.
#include "../../include/fta.h"

#include "fta_kernels.h"
#include "tmap.h"

namespace {

thread_local int g_last_cuda_error = 0;
thread_local cudaEvent_t g_prof_start = nullptr, g_prof_stop = nullptr;

int cuda_fail(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return FTA_ERR_CUDA;
}
int cuda_fail(int e) { return cuda_fail(static_cast<cudaError_t>(e)); }

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

int check_problem(const FtaProblem* p) {
  if (!p) return FTA_ERR_NULL;
  if (p->B <= 0 || p->H <= 0 || p->L1 <= 0 || p->L2 <= 0) return FTA_ERR_SHAPE;
  if (p->L2 % 8 != 0) return FTA_ERR_SHAPE;
  if (p->D != 32 && p->D != 64) return FTA_ERR_HEAD_DIM;
  if (p->dtype != FTA_FP16 && p->dtype != FTA_BF16) return FTA_ERR_DTYPE;
  if (static_cast<long long>(p->B) * p->H > 65535) return FTA_ERR_TOO_LARGE;
  return FTA_OK;
}

int check_t5(const FtaTensor5* t) {
  if (!t || !t->ptr) return FTA_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(t->ptr) % 16 != 0) return FTA_ERR_ALIGN;
  if (t->stride[4] != 1) return FTA_ERR_STRIDE;
  for (int i = 0; i < 4; ++i)
    if (t->stride[i] <= 0 || t->stride[i] % 8 != 0) return FTA_ERR_STRIDE;
  return FTA_OK;
}

int check_t4(const FtaTensor4* t) {
  if (!t || !t->ptr) return FTA_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(t->ptr) % 16 != 0) return FTA_ERR_ALIGN;
  if (t->stride[3] != 1) return FTA_ERR_STRIDE;
  for (int i = 0; i < 3; ++i)
    if (t->stride[i] <= 0 || t->stride[i] % 8 != 0) return FTA_ERR_STRIDE;
  return FTA_OK;
}

// 5-D map over (D, L2, L1, H, B), tile = 128 rows of L2 x D, swizzle = row bytes (64 or 128).
int map5(CUtensorMap* m, const FtaProblem* p, const FtaTensor5* t) {
  const uint64_t dims[5] = {static_cast<uint64_t>(p->D), static_cast<uint64_t>(p->L2),
                            static_cast<uint64_t>(p->L1), static_cast<uint64_t>(p->H),
                            static_cast<uint64_t>(p->B)};
  const uint64_t str[5] = {0, static_cast<uint64_t>(t->stride[3]) * 2, static_cast<uint64_t>(t->stride[2]) * 2,
                           static_cast<uint64_t>(t->stride[1]) * 2, static_cast<uint64_t>(t->stride[0]) * 2};
  const uint32_t box[5] = {static_cast<uint32_t>(p->D), 128, 1, 1, 1};
  return fta::make_tmap_16bit(m, t->ptr, 5, dims, str, box, p->D * 2) == 0 ? FTA_OK : FTA_ERR_TENSOR_MAP;
}

int padded_l2(const FtaProblem* p) { return (p->L2 + 127) / 128 * 128; }

// 4-D map over the bias (key, query, H, B); `box_k` keys x 128 queries per tile. The bias the kernels
// read always spans whole 128-blocks: the caller's tensor when L2 is a multiple of 128, else the
// padded copy made by fta_mask_bias.
int map_bias(CUtensorMap* m, const FtaProblem* p, const FtaTensor4* t, int box_k, int swizzle) {
  const uint64_t l2p = static_cast<uint64_t>(padded_l2(p));
  // a ragged problem must come with the padded copy: rows at least L2p apart, planes L2p rows apart
  if (l2p != static_cast<uint64_t>(p->L2) &&
      (static_cast<uint64_t>(t->stride[2]) < l2p || static_cast<uint64_t>(t->stride[1]) < l2p * l2p))
    return FTA_ERR_STRIDE;
  const uint64_t dims[4] = {l2p, l2p, static_cast<uint64_t>(p->H), static_cast<uint64_t>(p->B)};
  const uint64_t str[4] = {0, static_cast<uint64_t>(t->stride[2]) * 2, static_cast<uint64_t>(t->stride[1]) * 2,
                           static_cast<uint64_t>(t->stride[0]) * 2};
  const uint32_t box[4] = {static_cast<uint32_t>(box_k), 128, 1, 1};
  return fta::make_tmap_16bit(m, t->ptr, 4, dims, str, box, swizzle) == 0 ? FTA_OK : FTA_ERR_TENSOR_MAP;
}

size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

int num_sms() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

}  // namespace

namespace fta {
int record_cuda_error(int cuda_error) { return cuda_fail(cuda_error); }
}  // namespace fta

extern "C" {

int fta_version(void) { return 200; }

const char* fta_strerror(int code) {
  switch (code) {
    case FTA_OK: return "ok";
    case FTA_ERR_NULL: return "a required pointer is NULL";
    case FTA_ERR_SHAPE: return "bad shape: sizes must be positive and L2 a multiple of 8 (of 128 without fta_mask_bias)";
    case FTA_ERR_HEAD_DIM: return "unsupported head dimension: D must be 32 or 64";
    case FTA_ERR_DTYPE: return "unsupported dtype: fp16 or bf16 only";
    case FTA_ERR_STRIDE: return "bad stride: D stride must be 1, other strides positive multiples of 8 elements";
    case FTA_ERR_ALIGN: return "every device pointer must be 16-byte aligned";
    case FTA_ERR_WORKSPACE: return "workspace too small or misaligned";
    case FTA_ERR_TENSOR_MAP: return "the driver refused a TMA tensor map";
    case FTA_ERR_CUDA: return "a CUDA runtime call failed";
    case FTA_ERR_DEVICE: return "a bounded device-side wait ran out (status word non-zero)";
    case FTA_ERR_TOO_LARGE: return "size beyond a documented maximum";
    default: return "unknown error";
  }
}

int fta_last_cuda_error(void) { return g_last_cuda_error; }

int fta_forward(const FtaProblem* prob, const FtaTensor5* q, const FtaTensor5* k, const FtaTensor5* v,
                const FtaTensor4* bias, float sm_scale, const FtaTensor5* o, void* o_resid, float* lse,
                int32_t* status, void* stream) {
  int rc = check_problem(prob);
  if (rc) return rc;
  if ((rc = check_t5(q)) || (rc = check_t5(k)) || (rc = check_t5(v)) || (rc = check_t5(o)) ||
      (rc = check_t4(bias)))
    return rc;
  if (!lse || !status) return FTA_ERR_NULL;
  if (!aligned16(lse) || !aligned16(o_resid)) return FTA_ERR_ALIGN;
  fta::FwdArgs a;
  if ((rc = map5(&a.tmQ, prob, q)) || (rc = map5(&a.tmK, prob, k)) || (rc = map5(&a.tmV, prob, v)) ||
      (rc = map_bias(&a.tmBias, prob, bias, 64, 128)))
    return rc;
  a.o = o->ptr;
  a.o_resid = o_resid;
  a.lse = lse;
  a.status = status;
  a.B = prob->B;
  a.H = prob->H;
  a.L1 = prob->L1;
  a.L2 = prob->L2;
  a.D = prob->D;
  a.bf16 = prob->dtype == FTA_BF16;
  for (int i = 0; i < 4; ++i) a.so[i] = o->stride[i];
  a.sm_scale = sm_scale;
  if (const int e = fta::launch_fwd(a, static_cast<cudaStream_t>(stream))) return cuda_fail(e);
  return FTA_OK;
}

int fta_bwd_preprocess(const FtaProblem* prob, const FtaTensor5* o, const void* o_resid, const FtaTensor5* dout,
                       float* delta, void* stream) {
  int rc = check_problem(prob);
  if (rc) return rc;
  if ((rc = check_t5(o)) || (rc = check_t5(dout))) return rc;
  if (!delta) return FTA_ERR_NULL;
  if (!aligned16(o_resid)) return FTA_ERR_ALIGN;
  long long so[4], sd[4];
  for (int i = 0; i < 4; ++i) {
    so[i] = o->stride[i];
    sd[i] = dout->stride[i];
  }
  const int l2p = padded_l2(prob);
  if (l2p != prob->L2) {
    // the entries of queries past L2 (whole 128-blocks are read by the backward kernel) must be finite
    const cudaError_t e = cudaMemsetAsync(delta, 0, sizeof(float) * static_cast<size_t>(prob->B) * prob->H * prob->L1 * l2p,
                                          static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e);
  }
  if (const int e = fta::launch_preprocess(o->ptr, o_resid, so, dout->ptr, sd, delta, l2p, prob->B, prob->H, prob->L1,
                                           prob->L2, prob->D, prob->dtype == FTA_BF16,
                                           static_cast<cudaStream_t>(stream)))
    return cuda_fail(e);
  return FTA_OK;
}

int fta_mask_bias(const FtaProblem* prob, const FtaTensor4* bias, const uint8_t* key_mask, void* out, void* stream) {
  int rc = check_problem(prob);
  if (rc) return rc;
  if ((rc = check_t4(bias))) return rc;
  if (!out) return FTA_ERR_NULL;
  if (!aligned16(out) || reinterpret_cast<uintptr_t>(key_mask) % 8 != 0) return FTA_ERR_ALIGN;
  long long sb[4];
  for (int i = 0; i < 4; ++i) sb[i] = bias->stride[i];
  if (const int e = fta::launch_mask_bias(bias->ptr, sb, key_mask, out, prob->B, prob->H, prob->L2, padded_l2(prob),
                                          prob->dtype == FTA_BF16, static_cast<cudaStream_t>(stream)))
    return cuda_fail(e);
  return FTA_OK;
}

int fta_bwd_num_planes(const FtaProblem* prob) {
  if (check_problem(prob)) return 0;
  return fta::bwd_num_planes(prob->B, prob->H, prob->L1, prob->L2, prob->D, num_sms());
}

size_t fta_bwd_workspace_bytes(const FtaProblem* prob) {
  if (check_problem(prob)) return 0;
  const size_t rows = static_cast<size_t>(prob->B) * prob->H * prob->L1 * prob->L2;
  const size_t plane = static_cast<size_t>(prob->B) * prob->H * prob->L2 * prob->L2 * sizeof(float);
  const size_t l2p = static_cast<size_t>(padded_l2(prob));
  return align256(rows * prob->D * sizeof(float)) + align256(plane * fta_bwd_num_planes(prob)) +
         align256(static_cast<size_t>(prob->B) * prob->H * l2p * l2p * 2);  // + key-major copy of the bias (16-bit, whole blocks)
}

int fta_backward(const FtaProblem* prob, const FtaTensor5* q, const FtaTensor5* k, const FtaTensor5* v,
                 const FtaTensor4* bias, const FtaTensor5* dout, const float* lse, const float* delta,
                 float sm_scale, const FtaTensor5* dq, const FtaTensor5* dk, const FtaTensor5* dv,
                 float* dbias_f32, void* dbias_cast, void* workspace, size_t workspace_bytes, int32_t* status,
                 void* stream) {
  int rc = check_problem(prob);
  if (rc) return rc;
  if ((rc = check_t5(q)) || (rc = check_t5(k)) || (rc = check_t5(v)) || (rc = check_t5(dout)) ||
      (rc = check_t5(dq)) || (rc = check_t5(dk)) || (rc = check_t5(dv)) || (rc = check_t4(bias)))
    return rc;
  if (!lse || !delta || !dbias_f32 || !status || !workspace) return FTA_ERR_NULL;
  // the kernel fetches the statistics with 512-byte bulk copies and the epilogue writes dBias with
  // 16-byte stores
  if (!aligned16(lse) || !aligned16(delta) || !aligned16(dbias_f32) || !aligned16(dbias_cast)) return FTA_ERR_ALIGN;
  if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0 || workspace_bytes < fta_bwd_workspace_bytes(prob))
    return FTA_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t rows = static_cast<size_t>(prob->B) * prob->H * prob->L1 * prob->L2;
  const size_t dq_bytes = rows * prob->D * sizeof(float);
  const long long plane_elems = static_cast<long long>(prob->B) * prob->H * prob->L2 * prob->L2;
  float* dq32 = static_cast<float*>(workspace);
  float* planes = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + align256(dq_bytes));
  const int nplanes = fta_bwd_num_planes(prob);
  void* bias_t = reinterpret_cast<uint8_t*>(planes) + align256(static_cast<size_t>(plane_elems) * 4 * nplanes);
  const bool bf16 = prob->dtype == FTA_BF16;

  fta::BwdArgs a;
  FtaTensor4 bt;  // key-major copy: (B, H, key, query) contiguous
  bt.ptr = bias_t;
  const int l2p = padded_l2(prob);
  bt.stride[0] = static_cast<int64_t>(prob->H) * l2p * l2p;
  bt.stride[1] = static_cast<int64_t>(l2p) * l2p;
  bt.stride[2] = l2p;
  bt.stride[3] = 1;
  if ((rc = map5(&a.tmQ, prob, q)) || (rc = map5(&a.tmK, prob, k)) || (rc = map5(&a.tmV, prob, v)) ||
      (rc = map5(&a.tmDO, prob, dout)) || (rc = map_bias(&a.tmBiasT, prob, &bt, 64, 128)))
    return rc;
  {
    // dq32 seen as (B*H*L1, L2, D) float32; the kernel adds 128-query x 32-column tiles into it with
    // TMA reductions (the part of a ragged last query block beyond L2 is clipped)
    const uint64_t bhi = static_cast<uint64_t>(prob->B) * prob->H * prob->L1;
    if (bhi >= (1ull << 31)) return FTA_ERR_SHAPE;  // tile coordinates are signed 32-bit
    const uint64_t dims[3] = {static_cast<uint64_t>(prob->D), static_cast<uint64_t>(prob->L2), bhi};
    const uint64_t str[3] = {0, static_cast<uint64_t>(prob->D) * 4, static_cast<uint64_t>(prob->L2) * prob->D * 4};
    const uint32_t box[3] = {32, 128, 1};
    if (fta::make_tmap(&a.tmDQ, 4, dq32, 3, dims, str, box, 128) != 0) return FTA_ERR_TENSOR_MAP;
    // the partial dBias planes, key-major: (nplanes * B*H, L2 keys, L2 queries) float32, clipped alike
    const uint64_t pdims[3] = {static_cast<uint64_t>(prob->L2), static_cast<uint64_t>(prob->L2),
                               static_cast<uint64_t>(nplanes) * prob->B * prob->H};
    const uint64_t pstr[3] = {0, static_cast<uint64_t>(prob->L2) * 4, static_cast<uint64_t>(prob->L2) * prob->L2 * 4};
    if (fta::make_tmap(&a.tmPlane, 4, planes, 3, pdims, pstr, box, 128) != 0) return FTA_ERR_TENSOR_MAP;
  }
  a.lse = lse;
  a.delta = delta;
  a.dq32 = dq32;
  a.dk = dk->ptr;
  a.dv = dv->ptr;
  a.status = status;
  a.B = prob->B;
  a.H = prob->H;
  a.L1 = prob->L1;
  a.L2 = prob->L2;
  a.D = prob->D;
  a.bf16 = bf16;
  long long sdq[4];
  for (int i = 0; i < 4; ++i) {
    a.sdk[i] = dk->stride[i];
    a.sdv[i] = dv->stride[i];
    sdq[i] = dq->stride[i];
  }
  a.sm_scale = sm_scale;

  long long sb[4];
  for (int i = 0; i < 4; ++i) sb[i] = bias->stride[i];
  if (const int e = fta::launch_bwd_prologue(bias->ptr, sb, bias_t, prob->B, prob->H, l2p, dq32,
                                             static_cast<long long>(rows) * prob->D, st))
    return cuda_fail(e);
  if (g_prof_start) cudaEventRecord(g_prof_start, st);
  if (const int e = fta::launch_bwd(a, st)) return cuda_fail(e);
  if (g_prof_stop) cudaEventRecord(g_prof_stop, st);
  if (const int e = fta::launch_bwd_epilogue(dq32, dq->ptr, sdq, prob->B, prob->H, prob->L1, prob->L2, prob->D,
                                             sm_scale, planes, nplanes, dbias_f32, dbias_cast, bf16, st))
    return cuda_fail(e);
  return FTA_OK;
}

int fta_dbias_cast(const float* src, void* dst, int64_t n, int32_t dtype, void* stream) {
  if (!src || !dst) return FTA_ERR_NULL;
  if (n <= 0 || n % 4 != 0) return FTA_ERR_SHAPE;
  if (dtype != FTA_FP16 && dtype != FTA_BF16) return FTA_ERR_DTYPE;
  if (!aligned16(src) || !aligned16(dst)) return FTA_ERR_ALIGN;
  if (const int e = fta::launch_dbias_cast(src, n, dst, dtype == FTA_BF16, static_cast<cudaStream_t>(stream)))
    return cuda_fail(e);
  return FTA_OK;
}

int fta_dbias_sum_peers(const float* const* parts, int32_t nranks, int64_t n, float* out_f32, void* out_cast,
                        int32_t dtype, void* stream) {
  if (!parts || (!out_f32 && !out_cast)) return FTA_ERR_NULL;
  if (nranks < 1 || nranks > 64 || n <= 0 || n % 8 != 0) return FTA_ERR_SHAPE;
  if (dtype != FTA_FP16 && dtype != FTA_BF16) return FTA_ERR_DTYPE;
  if ((reinterpret_cast<uintptr_t>(parts) & 7u) || (out_f32 && !aligned16(out_f32)) || (out_cast && !aligned16(out_cast)))
    return FTA_ERR_ALIGN;
  if (const int e = fta::launch_dbias_sum_peers(parts, nranks, n, out_f32, out_cast, dtype == FTA_BF16, nullptr, 0, 0, 0,
                                                nullptr, static_cast<cudaStream_t>(stream)))
    return cuda_fail(e);
  return FTA_OK;
}

int fta_dbias_sum_peers_sync(const float* const* parts, int32_t* const* flags, int32_t nranks, int32_t rank,
                             int32_t epoch, int64_t n, float* out_f32, void* out_cast, int32_t dtype,
                             uint64_t wait_limit_ns, int32_t* status, void* stream) {
  if (!parts || !flags || !status || (!out_f32 && !out_cast)) return FTA_ERR_NULL;
  if (nranks < 1 || nranks > 64 || rank < 0 || rank >= nranks || epoch <= 0 || n <= 0 || n % 8 != 0) return FTA_ERR_SHAPE;
  if (dtype != FTA_FP16 && dtype != FTA_BF16) return FTA_ERR_DTYPE;
  if ((reinterpret_cast<uintptr_t>(parts) & 7u) || (reinterpret_cast<uintptr_t>(flags) & 7u) ||
      (out_f32 && !aligned16(out_f32)) || (out_cast && !aligned16(out_cast)))
    return FTA_ERR_ALIGN;
  if (wait_limit_ns == 0) wait_limit_ns = 1000000000ull;
  if (const int e = fta::launch_dbias_sum_peers(parts, nranks, n, out_f32, out_cast, dtype == FTA_BF16, flags, rank, epoch,
                                                wait_limit_ns, status, static_cast<cudaStream_t>(stream)))
    return cuda_fail(e);
  return FTA_OK;
}

int fta_dbias_sum_peers_sliced(const float* const* parts, void* const* outs, int32_t nranks, int32_t rank, int64_t n,
                               int32_t dtype, void* stream) {
  if (!parts || !outs) return FTA_ERR_NULL;
  if (nranks < 1 || nranks > 64 || rank < 0 || rank >= nranks || n <= 0 || n % 8 != 0) return FTA_ERR_SHAPE;
  if (dtype != FTA_FP16 && dtype != FTA_BF16) return FTA_ERR_DTYPE;
  if ((reinterpret_cast<uintptr_t>(parts) & 7u) || (reinterpret_cast<uintptr_t>(outs) & 7u)) return FTA_ERR_ALIGN;
  if (const int e = fta::launch_dbias_sum_peers_sliced(parts, outs, nranks, rank, n, dtype == FTA_BF16, nullptr, nullptr, 0,
                                                       0, nullptr, static_cast<cudaStream_t>(stream)))
    return cuda_fail(e);
  return FTA_OK;
}

int fta_dbias_sum_peers_sliced_sync(const float* const* parts, void* const* outs, int32_t* const* flags,
                                    const int32_t* my_flags, int32_t nranks, int32_t rank, int32_t epoch, int64_t n,
                                    int32_t dtype, uint64_t wait_limit_ns, int32_t* status, void* stream) {
  if (!parts || !outs || !flags || !my_flags || !status) return FTA_ERR_NULL;
  if (nranks < 1 || nranks > 31 || rank < 0 || rank >= nranks || epoch <= 0 || n <= 0 || n % 8 != 0) return FTA_ERR_SHAPE;
  if (dtype != FTA_FP16 && dtype != FTA_BF16) return FTA_ERR_DTYPE;
  if ((reinterpret_cast<uintptr_t>(parts) & 7u) || (reinterpret_cast<uintptr_t>(outs) & 7u) ||
      (reinterpret_cast<uintptr_t>(flags) & 7u) || (reinterpret_cast<uintptr_t>(my_flags) & 3u))
    return FTA_ERR_ALIGN;
  if (wait_limit_ns == 0) wait_limit_ns = 1000000000ull;
  if (const int e = fta::launch_dbias_sum_peers_sliced(parts, outs, nranks, rank, n, dtype == FTA_BF16, flags, my_flags, epoch,
                                                       wait_limit_ns, status, static_cast<cudaStream_t>(stream)))
    return cuda_fail(e);
  return FTA_OK;
}

int fta_memcpy_2d(void* dst, size_t dst_pitch_bytes, const void* src, size_t src_pitch_bytes, size_t width_bytes,
                  size_t rows, void* stream) {
  if (!dst || !src) return FTA_ERR_NULL;
  if (width_bytes == 0 || rows == 0) return FTA_ERR_SHAPE;
  if (dst_pitch_bytes < width_bytes || src_pitch_bytes < width_bytes) return FTA_ERR_STRIDE;
  const cudaError_t e = cudaMemcpy2DAsync(dst, dst_pitch_bytes, src, src_pitch_bytes, width_bytes, rows,
                                          cudaMemcpyDefault, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? FTA_OK : cuda_fail(e);
}

int fta_profile_backward_kernel(void* start_event, void* stop_event) {
  g_prof_start = static_cast<cudaEvent_t>(start_event);
  g_prof_stop = static_cast<cudaEvent_t>(stop_event);
  return FTA_OK;
}

int fta_read_status(const int32_t* status, int32_t* code_out, void* stream) {
  if (!status) return FTA_ERR_NULL;
  int32_t host = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(&host, status, sizeof(host), cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return cuda_fail(e);
  if (code_out) *code_out = host;
  return host == 0 ? FTA_OK : FTA_ERR_DEVICE;
}

}  // extern "C"
