// Internal launch interface between the C ABI (api.cu) and the kernels.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace fta {

// Records `cuda_error` (a cudaError_t) as the calling thread's last CUDA error, the value
// fta_last_cuda_error() reports; returns FTA_ERR_CUDA.
int record_cuda_error(int cuda_error);

// Every launch_* function below returns cudaSuccess (0) or the cudaError_t of the call that failed
// (the launch itself or an attribute call before it); it leaves no sticky error behind.

// cudaFuncAttributeMaxDynamicSharedMemorySize is a property of a kernel ON ONE DEVICE: a process
// that drives several GPUs has to set it once per device. One flag per device ordinal; two threads
// that race on the same device both make the (idempotent) call.
struct PerDeviceOnce {
  static constexpr int kMaxDevices = 64;
  std::atomic<unsigned char> done[kMaxDevices] = {};
};
template <typename Kernel>
inline cudaError_t ensure_dynamic_smem(PerDeviceOnce& once, Kernel kern, int bytes) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const bool tracked = dev >= 0 && dev < PerDeviceOnce::kMaxDevices;
  if (tracked && once.done[dev].load(std::memory_order_acquire)) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && tracked) once.done[dev].store(1, std::memory_order_release);
  return e;
}

struct FwdArgs {
  CUtensorMap tmQ, tmK, tmV, tmBias;
  void* o;
  void* o_resid;  // nullptr, or the rounding residual of O with O's strides
  float* lse;
  int* status;
  int B, H, L1, L2, D;
  bool bf16;
  long long so[4];  // element strides of O (and of the residual) over (B, H, L1, L2)
  float sm_scale;
};
int launch_fwd(const FwdArgs& a, cudaStream_t stream);
int fwd_rows_per_cta(int D);

struct BwdArgs {
  CUtensorMap tmQ, tmK, tmV, tmDO, tmBiasT;  // tmBiasT: over the key-major copy of the bias
  CUtensorMap tmDQ;    // dq32 as a 3-D float32 tensor (B*H*L1, L2, D), box 128 queries x 32 columns, 128 B swizzle
  CUtensorMap tmPlane; // the partial dBias planes as (nplanes*B*H, L2 keys, L2 queries) float32, same box
  const float* lse;    // (3,B,H,L1,L2): -max, -log2(sum), combined (NaN where inexact)
  const float* delta;  // (B,H,L1,L2)
  float* dq32;         // (B,H,L1,L2,D) float32, zeroed; receives sum over key blocks of dS K
  void* dk;
  void* dv;
  int* status;
  int B, H, L1, L2, D;
  bool bf16;
  long long sdk[4], sdv[4];  // element strides of dK, dV over (B, H, L1, L2)
  float sm_scale;
};
int launch_bwd(const BwdArgs& a, cudaStream_t stream);
int bwd_rows_per_cta(int D);
int bwd_num_planes(int B, int H, int L1, int L2, int D, int num_sms);

// delta[(b,h,i), j] = sum_d (O[.,d] + R[.,d]) * dO[.,d]; `o_resid` (R, strides of O) may be nullptr;
// `delta_pitch` = elements between rows (b,h,i) of delta (L2 rounded up to 128)
int launch_preprocess(const void* o, const void* o_resid, const long long so[4], const void* dout,
                      const long long sdo[4], float* delta, int delta_pitch, int B, int H, int L1, int L2, int D,
                      bool bf16, cudaStream_t stream);

// out[b][h][q][k], (B, H, L2p, L2p) contiguous: the bias where q, k < L2 and the key is kept by
// `key_mask` ((B, L2) bytes, non-zero = keep; nullptr = keep all), -inf for every other key, 0 for
// the kept keys of the padding queries q >= L2
int launch_mask_bias(const void* bias, const long long sb[4], const uint8_t* key_mask, void* out, int B, int H, int L2,
                     int L2p, bool bf16, cudaStream_t stream);

// Backward prologue, one launch: bias_t[bh][k][q] = bias[b][h][q][k] (16-bit elements; `sb` = element
// strides of the bias) and zero-fill of the float32 dQ accumulator (`dq_elems` floats, a multiple of 4)
int launch_bwd_prologue(const void* bias, const long long sb[4], void* bias_t, int B, int H, int L2, float* dq32,
                        long long dq_elems, cudaStream_t stream);

// Backward epilogue, one launch: dq[row, d] = (dtype)(scale * dq32[row, d]) and, for the KEY-MAJOR
// planes the backward kernel writes, (nplanes, B*H, key, query):
// dbias_f32[bh][query][key] = sum_p planes[p][bh][key][query] in plane order, optional rounded copy
int launch_bwd_epilogue(const float* dq32, void* dq, const long long sdq[4], int B, int H, int L1, int L2, int D,
                        float scale, const float* planes, int nplanes, float* dbias_f32, void* dbias_cast, bool bf16,
                        cudaStream_t stream);

// out = sum over r of parts[r][0..n) (rank order), float32 and / or rounded to 16 bits; `parts`: device
// array of `nranks` device pointers (peer mappings included); n a multiple of 8
// `flags` == nullptr: the caller has lined the ranks up; otherwise the kernel does (bounded wait, see the kernel)
int launch_dbias_sum_peers(const float* const* parts, int nranks, long long n, float* out_f32, void* out_cast,
                           bool bf16, int* const* flags, int rank, int epoch, unsigned long long limit_ns, int* status,
                           cudaStream_t stream);
// the same with the work split over the ranks: this rank sums its 1/nranks slice and stores the rounded
// result into every rank's buffer `outs[r]` (device array of nranks device pointers)
// `flags` == nullptr: the caller lines the ranks up before and after; otherwise the kernel does, and a
// one-block kernel behind it holds the stream until every rank's slice has arrived (`my_flags`: this
// rank's own flag array, 2 * nranks + 1 words)
int launch_dbias_sum_peers_sliced(const float* const* parts, void* const* outs, int nranks, int rank, long long n,
                                  bool bf16, int* const* flags, const int* my_flags, int epoch,
                                  unsigned long long limit_ns, int* status, cudaStream_t stream);
// dst[i] = (dtype) src[i], n a multiple of 4
int launch_dbias_cast(const float* src, long long n, void* dst, bool bf16, cudaStream_t stream);

}  // namespace fta
