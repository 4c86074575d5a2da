// Bandwidth-bound kernels around the backward pass. All three are coalesced, 16-byte
// vectorised HBM streams with grid-stride loops sized to the SM count.
//
//  preprocess     : delta[row] = sum_d O[row,d] * dO[row,d]     (reference: _attn_bwd_preprocess,
//                   flash_tt_attn.py:266-288)
//  dbias_finalize : dBias[e] = sum over partial planes, in plane order, plus the rounded copy
//                   (replaces the fp16 atomics into a zeroed buffer, flash_tt_attn.py:425-426, 613)
//  transpose_bias : key-major copy of the pair bias for the backward kernel
//  dq_finalize    : dQ = (dtype)(sm_scale * dQ_f32)             (the scaling of flash_tt_attn.py:430, 549)
#include "fta_kernels.h"
#include "tc05.cuh"

namespace fta {
namespace {

template <bool kBf16>
__device__ __forceinline__ float dot8(const uint4& a, const uint4& b) {
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
  const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float a0, a1, b0, b1;
    unpack2<kBf16>(aw[i], a0, a1);
    unpack2<kBf16>(bw[i], b0, b1);
    s = fmaf(a0, b0, s);
    s = fmaf(a1, b1, s);
  }
  return s;
}

// One thread per 8 elements; D/8 adjacent lanes share a row and reduce with shuffles.
// kDense: both tensors are contiguous, so a row's offset is row * D and the index needs no
// division (the strided form spends more instructions on 64-bit divisions than on the data).
template <int kD, bool kBf16, bool kDense>
__global__ void __launch_bounds__(256) preprocess_kernel(const uint16_t* __restrict__ o,
                                                         const uint16_t* __restrict__ dout,
                                                         float* __restrict__ delta, long long rows,
                                                         int H, int L1, int L2, long long so_b,
                                                         long long so_h, long long so_i, long long so_j,
                                                         long long sd_b, long long sd_h, long long sd_i,
                                                         long long sd_j) {
  constexpr int LPR = kD / 8;  // lanes per row
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = (rows * LPR + 31) / 32 * 32;  // keep warps converged for the shuffles
  for (long long idx = tid; idx < total; idx += nthreads) {
    const long long row = idx / LPR;
    const int part = static_cast<int>(idx % LPR);
    float s = 0.f;
    if (row < rows) {
      long long oo, od;
      if constexpr (kDense) {
        oo = od = row * kD + part * 8;
      } else {
        long long r = row;
        const int j = static_cast<int>(r % L2);
        r /= L2;
        const int i = static_cast<int>(r % L1);
        r /= L1;
        const int h = static_cast<int>(r % H);
        const long long b = r / H;
        oo = b * so_b + h * so_h + i * so_i + j * so_j + part * 8;
        od = b * sd_b + h * sd_h + i * sd_i + j * sd_j + part * 8;
      }
      const uint4 ov = __ldg(reinterpret_cast<const uint4*>(o + oo));
      const uint4 dv = __ldg(reinterpret_cast<const uint4*>(dout + od));
      s = dot8<kBf16>(ov, dv);
    }
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (part == 0 && row < rows) delta[row] = s;
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(256) dbias_finalize_kernel(const float* __restrict__ planes,
                                                             int nplanes, long long plane_elems,
                                                             float* __restrict__ out_f32,
                                                             uint16_t* __restrict__ out_cast) {
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long nvec = plane_elems / 4;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
       v += nthreads) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4* src = reinterpret_cast<const float4*>(planes) + v;
    for (int pl = 0; pl < nplanes; ++pl) {  // fixed order: bit-reproducible
      const float4 x = __ldg(src + static_cast<long long>(pl) * nvec);
      acc.x += x.x;
      acc.y += x.y;
      acc.z += x.z;
      acc.w += x.w;
    }
    if (out_f32) reinterpret_cast<float4*>(out_f32)[v] = acc;
    if (out_cast) {
      uint2 pk;
      pk.x = pack2<kBf16>(acc.x, acc.y);
      pk.y = pack2<kBf16>(acc.z, acc.w);
      reinterpret_cast<uint2*>(out_cast)[v] = pk;
    }
  }
}

// Key-major planes (p, bh, key, query) -> dBias (bh, query, key): 32 x 32 tiles transposed through
// shared memory, the planes summed in index order on the way (bit-reproducible).
template <bool kBf16>
__global__ void __launch_bounds__(256) dbias_finalize_keymajor_kernel(const float* __restrict__ planes,
                                                                      int nplanes, int BH, int L2,
                                                                      float* __restrict__ out_f32,
                                                                      uint16_t* __restrict__ out_cast) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int q0 = blockIdx.x * 32, k0 = blockIdx.y * 32, bh = blockIdx.z;
  const long long plane_stride = static_cast<long long>(BH) * L2 * L2;
  const float* src = planes + (static_cast<long long>(bh) * L2 + k0) * L2 + q0 + tx;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int pl = 0; pl < nplanes; ++pl) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      acc[i] += __ldg(src + static_cast<long long>(pl) * plane_stride + static_cast<long long>(ty + 8 * i) * L2);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) tile[ty + 8 * i][tx] = acc[i];  // [key][query]
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int q = ty + 8 * i;
    const float v = tile[tx][q];
    const long long o = (static_cast<long long>(bh) * L2 + q0 + q) * L2 + k0 + tx;
    if (out_f32) out_f32[o] = v;
    if (out_cast) {
      const uint32_t pk = pack2<kBf16>(v, 0.f);
      out_cast[o] = static_cast<uint16_t>(pk & 0xffffu);
    }
  }
}

template <int kD, bool kBf16, bool kDense>
__global__ void __launch_bounds__(256) dq_finalize_kernel(const float* __restrict__ dq32,
                                                          uint16_t* __restrict__ dq, long long rows,
                                                          int H, int L1, int L2, long long s_b,
                                                          long long s_h, long long s_i, long long s_j,
                                                          float scale) {
  constexpr int LPR = kD / 8;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long total = rows * LPR;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += nthreads) {
    const long long row = idx / LPR;
    const int part = static_cast<int>(idx % LPR);
    const float4 a = __ldg(reinterpret_cast<const float4*>(dq32 + row * kD + part * 8));
    const float4 c = __ldg(reinterpret_cast<const float4*>(dq32 + row * kD + part * 8 + 4));
    long long oo;
    if constexpr (kDense) {
      oo = row * kD + part * 8;
    } else {
      long long r = row;
      const int j = static_cast<int>(r % L2);
      r /= L2;
      const int i = static_cast<int>(r % L1);
      r /= L1;
      const int h = static_cast<int>(r % H);
      const long long b = r / H;
      oo = b * s_b + h * s_h + i * s_i + j * s_j + part * 8;
    }
    uint4 out;
    out.x = pack2<kBf16>(a.x * scale, a.y * scale);
    out.y = pack2<kBf16>(a.z * scale, a.w * scale);
    out.z = pack2<kBf16>(c.x * scale, c.y * scale);
    out.w = pack2<kBf16>(c.z * scale, c.w * scale);
    *reinterpret_cast<uint4*>(dq + oo) = out;
  }
}

// out[bh][k][q] = in[b][h][q][k] for 16-bit elements, 64 x 64 tiles staged in shared memory.
__global__ void __launch_bounds__(256) transpose_bias_kernel(const uint16_t* __restrict__ in,
                                                             uint16_t* __restrict__ out, int H, int L2,
                                                             long long s_b, long long s_h, long long s_q) {
  __shared__ uint16_t tile[64][66];
  const int tiles = L2 / 64;
  const int bh = blockIdx.y;
  const int b = bh / H, h = bh % H;
  const uint16_t* src = in + b * s_b + h * s_h;
  uint16_t* dst = out + static_cast<long long>(bh) * L2 * L2;
  for (int t = blockIdx.x; t < tiles * tiles; t += gridDim.x) {
    const int q0 = (t / tiles) * 64, k0 = (t % tiles) * 64;
    // 256 threads: 4 rows x 64 columns per pass; two 16-bit elements per thread
    for (int i = threadIdx.x; i < 64 * 32; i += 256) {
      const int rr = i / 32, c2 = (i % 32) * 2;
      const uint32_t v = *reinterpret_cast<const uint32_t*>(src + (q0 + rr) * s_q + k0 + c2);
      tile[rr][c2] = static_cast<uint16_t>(v & 0xffffu);
      tile[rr][c2 + 1] = static_cast<uint16_t>(v >> 16);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * 32; i += 256) {
      const int rr = i / 32, c2 = (i % 32) * 2;  // rr = key row of the output, c2 = query column
      const uint32_t v = static_cast<uint32_t>(tile[c2][rr]) | (static_cast<uint32_t>(tile[c2 + 1][rr]) << 16);
      *reinterpret_cast<uint32_t*>(dst + static_cast<long long>(k0 + rr) * L2 + q0 + c2) = v;
    }
    __syncthreads();
  }
}

int grid_for(long long work_items, int threads) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(sms) * 8;  // a multiple of the SM count
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace

int launch_preprocess(const void* o, const long long so[4], const void* dout, const long long sdo[4],
                      float* delta, int B, int H, int L1, int L2, int D, bool bf16,
                      cudaStream_t stream) {
  const long long rows = static_cast<long long>(B) * H * L1 * L2;
  const int grid = grid_for(rows * (D / 8), 256);
  const uint16_t* op = static_cast<const uint16_t*>(o);
  const uint16_t* dp = static_cast<const uint16_t*>(dout);
  auto is_dense = [&](const long long s4[4]) {
    return s4[3] == D && s4[2] == static_cast<long long>(L2) * D && s4[1] == static_cast<long long>(L1) * L2 * D &&
           s4[0] == static_cast<long long>(H) * L1 * L2 * D;
  };
  const bool dense = is_dense(so) && is_dense(sdo);
#define FTA_PRE(DD, BF, DN)                                                                          \
  preprocess_kernel<DD, BF, DN><<<grid, 256, 0, stream>>>(op, dp, delta, rows, H, L1, L2, so[0],      \
                                                          so[1], so[2], so[3], sdo[0], sdo[1], sdo[2], \
                                                          sdo[3])
#define FTA_PRE2(DD, BF) \
  do {                   \
    if (dense) FTA_PRE(DD, BF, true); else FTA_PRE(DD, BF, false); \
  } while (0)
  if (D == 32) {
    if (bf16) FTA_PRE2(32, true); else FTA_PRE2(32, false);
  } else {
    if (bf16) FTA_PRE2(64, true); else FTA_PRE2(64, false);
  }
#undef FTA_PRE2
#undef FTA_PRE
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int launch_transpose_bias(const void* bias, const long long sb[4], void* out, int B, int H, int L2,
                          cudaStream_t stream) {
  const int tiles = (L2 / 64) * (L2 / 64);
  dim3 grid(tiles < 1024 ? tiles : 1024, B * H);
  transpose_bias_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(bias),
                                                  static_cast<uint16_t*>(out), H, L2, sb[0], sb[1], sb[2]);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int launch_dbias_finalize(const float* planes, int nplanes, long long plane_elems, float* out_f32,
                          void* out_cast, bool bf16, cudaStream_t stream) {
  const int grid = grid_for(plane_elems / 4, 256);
  if (bf16)
    dbias_finalize_kernel<true><<<grid, 256, 0, stream>>>(planes, nplanes, plane_elems, out_f32,
                                                          static_cast<uint16_t*>(out_cast));
  else
    dbias_finalize_kernel<false><<<grid, 256, 0, stream>>>(planes, nplanes, plane_elems, out_f32,
                                                           static_cast<uint16_t*>(out_cast));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int launch_dbias_finalize_keymajor(const float* planes, int nplanes, int BH, int L2, float* out_f32,
                                   void* out_cast, bool bf16, cudaStream_t stream) {
  const dim3 grid(L2 / 32, L2 / 32, BH);
  if (bf16)
    dbias_finalize_keymajor_kernel<true><<<grid, 256, 0, stream>>>(planes, nplanes, BH, L2, out_f32,
                                                                   static_cast<uint16_t*>(out_cast));
  else
    dbias_finalize_keymajor_kernel<false><<<grid, 256, 0, stream>>>(planes, nplanes, BH, L2, out_f32,
                                                                    static_cast<uint16_t*>(out_cast));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int launch_dq_finalize(const float* dq32, void* dq, const long long sdq[4], int B, int H, int L1,
                       int L2, int D, float scale, bool bf16, cudaStream_t stream) {
  const long long rows = static_cast<long long>(B) * H * L1 * L2;
  const int grid = grid_for(rows * (D / 8), 256);
  uint16_t* out = static_cast<uint16_t*>(dq);
  const bool dense = sdq[3] == D && sdq[2] == static_cast<long long>(L2) * D &&
                     sdq[1] == static_cast<long long>(L1) * L2 * D && sdq[0] == static_cast<long long>(H) * L1 * L2 * D;
#define FTA_DQ(DD, BF, DN)                                                                              \
  dq_finalize_kernel<DD, BF, DN><<<grid, 256, 0, stream>>>(dq32, out, rows, H, L1, L2, sdq[0], sdq[1], \
                                                           sdq[2], sdq[3], scale)
#define FTA_DQ2(DD, BF) \
  do {                  \
    if (dense) FTA_DQ(DD, BF, true); else FTA_DQ(DD, BF, false); \
  } while (0)
  if (D == 32) {
    if (bf16) FTA_DQ2(32, true); else FTA_DQ2(32, false);
  } else {
    if (bf16) FTA_DQ2(64, true); else FTA_DQ2(64, false);
  }
#undef FTA_DQ2
#undef FTA_DQ
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace fta
