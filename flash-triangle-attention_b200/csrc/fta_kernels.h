// Internal launch interface between the C ABI (api.cu) and the kernels.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fta {

struct FwdArgs {
  CUtensorMap tmQ, tmK, tmV, tmBias;
  void* o;
  float* lse;
  int* status;
  int B, H, L1, L2, D;
  bool bf16;
  long long so[4];  // element strides of O over (B, H, L1, L2)
  float sm_scale;
};
int launch_fwd(const FwdArgs& a, cudaStream_t stream);
int fwd_rows_per_cta(int D);

struct BwdArgs {
  CUtensorMap tmQ, tmK, tmV, tmDO, tmBiasT;  // tmBiasT: over the key-major copy of the bias
  CUtensorMap tmDQ;    // dq32 as a 2-D float32 tensor (rows, D), box 128 rows x 32 columns, 128 B swizzle
  CUtensorMap tmPlane; // the partial dBias planes as (nplanes*B*H*L2 key rows, L2 queries) float32, same box
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

// delta[row] = sum_d O[row,d] * dO[row,d]
int launch_preprocess(const void* o, const long long so[4], const void* dout, const long long sdo[4],
                      float* delta, int B, int H, int L1, int L2, int D, bool bf16,
                      cudaStream_t stream);

// out[bh][k][q] = bias[b][h][q][k] (16-bit elements); `sb` = element strides of the bias
int launch_transpose_bias(const void* bias, const long long sb[4], void* out, int B, int H, int L2,
                          cudaStream_t stream);

// out_f32[e] = sum_p planes[p][e] (fixed order), optional rounded copy
int launch_dbias_finalize(const float* planes, int nplanes, long long plane_elems, float* out_f32,
                          void* out_cast, bool bf16, cudaStream_t stream);

// The same for the KEY-MAJOR planes the backward kernel writes, (nplanes, B*H, key, query):
// out[bh][query][key] = sum_p planes[p][bh][key][query] in plane order, optional rounded copy
int launch_dbias_finalize_keymajor(const float* planes, int nplanes, int BH, int L2, float* out_f32,
                                   void* out_cast, bool bf16, cudaStream_t stream);

// dq[row, d] = (dtype)(scale * dq32[row, d])
int launch_dq_finalize(const float* dq32, void* dq, const long long sdq[4], int B, int H, int L1,
                       int L2, int D, float scale, bool bf16, cudaStream_t stream);

#ifdef FTA_TRACE
// debug builds only: clock stamps of CTA 0 of the last launch
int trace_read_fwd(unsigned long long* host, int n);
int trace_read_bwd(unsigned long long* host, int n);
#endif

}  // namespace fta
