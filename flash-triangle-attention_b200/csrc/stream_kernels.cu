// Bandwidth-bound kernels around the backward pass: coalesced, 16-byte vectorised HBM streams with
// grid-stride loops sized to the SM count.
//
//  preprocess     : delta[row] = sum_d (O[row,d] + R[row,d]) * dO[row,d]   (reference:
//                   _attn_bwd_preprocess, flash_tt_attn.py:266-288; R is the optional rounding
//                   residual of O written by the forward pass)
//  bwd_prologue   : key-major copy of the pair bias for the backward kernel + zero-fill of the
//                   float32 dQ accumulator, one launch (the reference zero-fills its dBias buffer
//                   instead, flash_tt_attn.py:613)
//  bwd_epilogue   : dQ = (dtype)(sm_scale * dQ_f32) (the scaling of flash_tt_attn.py:430, 549) and
//                   dBias = sum over the partial planes in plane order, transposed back to
//                   (query, key), plus the rounded copy (replaces the fp16 atomics into a zeroed
//                   buffer, flash_tt_attn.py:425-426), one launch
//  dbias_cast     : float32 -> 16-bit copy (after a cross-GPU sum)
#include "fta_kernels.h"
#include "tc05.cuh"

#include <type_traits>

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

// (a + r) . b with a + r formed in float32 (exact: two 16-bit values of neighbouring magnitude)
template <bool kBf16>
__device__ __forceinline__ float dot8r(const uint4& a, const uint4& r, const uint4& b) {
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
  const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
  const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float a0, a1, r0, r1, b0, b1;
    unpack2<kBf16>(aw[i], a0, a1);
    unpack2<kBf16>(rw[i], r0, r1);
    unpack2<kBf16>(bw[i], b0, b1);
    s = fmaf(a0 + r0, b0, s);
    s = fmaf(a1 + r1, b1, s);
  }
  return s;
}

// (b, h, i, j) of a flat row index -> element offset under strides s[0..3]
__device__ __forceinline__ long long strided_row_offset(long long row, int H, int L1, int L2, long long s_b,
                                                        long long s_h, long long s_i, long long s_j) {
  const int j = static_cast<int>(row % L2);
  row /= L2;
  const int i = static_cast<int>(row % L1);
  row /= L1;
  const int h = static_cast<int>(row % H);
  const long long b = row / H;
  return b * s_b + h * s_h + i * s_i + j * s_j;
}

// One thread per 8 elements; D/8 adjacent lanes share a row and reduce with shuffles.
// kDense: both tensors are contiguous, so a row's offset is row * D and the index needs no
// division (the strided form spends more instructions on 64-bit divisions than on the data).
template <int kD, bool kBf16, bool kDense, bool kResid>
__global__ void __launch_bounds__(256) preprocess_kernel(const uint16_t* __restrict__ o,
                                                         const uint16_t* __restrict__ o_resid,
                                                         const uint16_t* __restrict__ dout,
                                                         float* __restrict__ delta, int delta_pitch,
                                                         long long rows, int H, int L1, int L2, long long so_b,
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
        oo = strided_row_offset(row, H, L1, L2, so_b, so_h, so_i, so_j) + part * 8;
        od = strided_row_offset(row, H, L1, L2, sd_b, sd_h, sd_i, sd_j) + part * 8;
      }
      const uint4 ov = __ldg(reinterpret_cast<const uint4*>(o + oo));
      const uint4 dv = __ldg(reinterpret_cast<const uint4*>(dout + od));
      if constexpr (kResid) {
        const uint4 rv = __ldg(reinterpret_cast<const uint4*>(o_resid + oo));
        s = dot8r<kBf16>(ov, rv, dv);
      } else {
        s = dot8<kBf16>(ov, dv);
      }
    }
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    // rows of delta are `delta_pitch` apart (L2 rounded up to 128; equal to L2 in the dense case)
    if (part == 0 && row < rows) delta[delta_pitch == L2 ? row : (row / L2) * delta_pitch + row % L2] = s;
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(256) dbias_cast_kernel(const float* __restrict__ src, long long n,
                                                         uint16_t* __restrict__ dst) {
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long nvec = n / 8;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += nthreads) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(src) + 2 * v);
    const float4 c = __ldg(reinterpret_cast<const float4*>(src) + 2 * v + 1);
    uint4 pk;
    pk.x = pack2<kBf16>(a.x, a.y);
    pk.y = pack2<kBf16>(a.z, a.w);
    pk.z = pack2<kBf16>(c.x, c.y);
    pk.w = pack2<kBf16>(c.z, c.w);
    reinterpret_cast<uint4*>(dst)[v] = pk;
  }
  // tail (n is a multiple of 4, not necessarily of 8)
  if (blockIdx.x == 0 && threadIdx.x == 0 && (n & 7)) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(src) + 2 * nvec);
    uint2 pk;
    pk.x = pack2<kBf16>(a.x, a.y);
    pk.y = pack2<kBf16>(a.z, a.w);
    reinterpret_cast<uint2*>(dst)[2 * nvec] = pk;
  }
}

// dBias across GPUs without a library collective: every rank holds its float32 partial in memory
// that its peers can address (NVLink peer mappings), and each rank adds the R partials itself, in
// rank order (the same order on every rank: identical bits everywhere), then rounds once. `parts`
// is a device array of R pointers, entry r = rank r's partial as seen from this GPU. Plain loads
// that skip L1 (the peers rewrite these buffers between launches); 8 elements per thread, grid-stride.
// With `flags` (device array of R pointers: entry r = rank r's array of R 32-bit epoch words, as this GPU
// sees it) the kernel also lines the ranks up itself, no barrier launch needed: block 0 publishes
// "my partial of epoch e is complete" into every rank's word for this rank (the partial was written by
// the previous kernel on the stream; fence + system-scope release), and every block waits until the R
// words of this rank show epoch e before it reads the partials. The wait is bounded (`limit_ns` of the
// global timer): when it runs out the kernel writes 0x1000 | 0x61 to `status` and returns without output.
__device__ __forceinline__ void st_release_sys_u32(int* p, int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys_u32(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <bool kBf16>
__global__ void __launch_bounds__(256) dbias_sum_peers_kernel(const float* const* __restrict__ parts, int nranks,
                                                              long long n, float* __restrict__ out_f32,
                                                              uint16_t* __restrict__ out_cast, int* const* flags,
                                                              int rank, int epoch, unsigned long long limit_ns,
                                                              int* status) {
  if (flags != nullptr) {
    if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < nranks) {
      __threadfence_system();
      st_release_sys_u32(flags[threadIdx.x] + rank, epoch);
    }
    bool ok = true;
    if (static_cast<int>(threadIdx.x) < nranks) {
      const int* mine = flags[rank] + threadIdx.x;
      const unsigned long long t0 = global_timer_ns();
      // epochs only grow; "at least" tolerates a peer that is already a step ahead
      while (ld_acquire_sys_u32(mine) - epoch < 0) {
        if (global_timer_ns() - t0 > limit_ns) {
          ok = false;
          break;
        }
        __nanosleep(100);
      }
    }
    if (!__syncthreads_and(ok)) {
      if (threadIdx.x == 0) atomicCAS(status, kStatusOk, kStatusWaitTimeout | 0x61);
      return;
    }
  }
  // Four 8-element vectors per thread and pass, each rank's eight 16-byte loads issued together: a
  // peer load takes a few microseconds over NVLink, so the bytes in flight decide the rate.
  constexpr int U = 4;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long nvec = n / 8;
  for (long long v0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v0 < nvec; v0 += U * nthreads) {
    float4 acc[U][2];
#pragma unroll
    for (int u = 0; u < U; ++u) acc[u][0] = acc[u][1] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < nranks; ++r) {  // rank order: the same bits on every rank
      const float4* src = reinterpret_cast<const float4*>(parts[r]);
      float4 x[U][2];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long v = v0 + u * nthreads;
        if (v < nvec) {
          x[u][0] = __ldcg(src + 2 * v);
          x[u][1] = __ldcg(src + 2 * v + 1);
        } else {
          x[u][0] = x[u][1] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
          acc[u][hlf].x += x[u][hlf].x;
          acc[u][hlf].y += x[u][hlf].y;
          acc[u][hlf].z += x[u][hlf].z;
          acc[u][hlf].w += x[u][hlf].w;
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long v = v0 + u * nthreads;
      if (v >= nvec) continue;
      if (out_f32) {
        reinterpret_cast<float4*>(out_f32)[2 * v] = acc[u][0];
        reinterpret_cast<float4*>(out_f32)[2 * v + 1] = acc[u][1];
      }
      if (out_cast) {
        uint4 pk;
        pk.x = pack2<kBf16>(acc[u][0].x, acc[u][0].y);
        pk.y = pack2<kBf16>(acc[u][0].z, acc[u][0].w);
        pk.z = pack2<kBf16>(acc[u][1].x, acc[u][1].y);
        pk.w = pack2<kBf16>(acc[u][1].z, acc[u][1].w);
        reinterpret_cast<uint4*>(out_cast)[v] = pk;
      }
    }
  }
}

// The same sum for larger groups, as reduce-scatter + all-gather in one kernel: rank `rank` adds the R
// partials of ITS 1/R slice of the elements (rank order), rounds, and stores the 16-bit result into
// every rank's output buffer (`outs`: device array of R pointers, peer mappings included). Each rank
// then reads (R-1)/R of one partial and writes (R-1)/R of half that over NVLink, whatever R is. The
// full result is in a rank's output buffer once every rank's launch has finished (a second barrier).
// With `flags` the kernel lines the ranks up itself, like dbias_sum_peers_kernel (words [0, R) of a rank's
// flag array: "rank r's partial of this epoch is complete"), and when its last block has stored its last
// vector it publishes "rank `rank`'s slice is in your output buffer" into word R + rank of every
// rank's array (the blocks count themselves out on word 2R of this rank's own array).
// peers_wait_kernel, launched behind it, then holds the stream until all R slices have arrived.
template <bool kBf16>
__global__ void __launch_bounds__(256) dbias_sum_peers_sliced_kernel(const float* const* __restrict__ parts,
                                                                     uint16_t* const* __restrict__ outs, int nranks,
                                                                     int rank, long long n, int* const* flags, int epoch,
                                                                     unsigned long long limit_ns, int* status) {
  __shared__ int s_last;
  if (flags != nullptr) {
    if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < nranks) {
      __threadfence_system();
      st_release_sys_u32(flags[threadIdx.x] + rank, epoch);
    }
    bool ok = true;
    if (static_cast<int>(threadIdx.x) < nranks) {
      const int* mine = flags[rank] + threadIdx.x;
      const unsigned long long t0 = global_timer_ns();
      while (ld_acquire_sys_u32(mine) - epoch < 0) {
        if (global_timer_ns() - t0 > limit_ns) {
          ok = false;
          break;
        }
        __nanosleep(100);
      }
    }
    if (!__syncthreads_and(ok)) {
      if (threadIdx.x == 0) atomicCAS(status, kStatusOk, kStatusWaitTimeout | 0x62);
      return;
    }
  }
  // One 8-element vector per thread and pass; the loads of up to eight ranks are issued together
  // (a peer load is a round trip of a few microseconds: one round trip per eight ranks, not one per
  // rank), then added in rank order.
  constexpr int RB = 8;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long nvec = n / 8;
  const long long per = (nvec + nranks - 1) / nranks;
  const long long v_begin = rank * per, v_end = (v_begin + per < nvec) ? v_begin + per : nvec;
  for (long long v = v_begin + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < v_end; v += nthreads) {
    float4 acc0 = make_float4(0.f, 0.f, 0.f, 0.f), acc1 = acc0;
    for (int r0 = 0; r0 < nranks; r0 += RB) {
      float4 x[RB][2];
#pragma unroll
      for (int k = 0; k < RB; ++k) {
        if (r0 + k < nranks) {
          const float4* src = reinterpret_cast<const float4*>(parts[r0 + k]) + 2 * v;
          x[k][0] = __ldcg(src);
          x[k][1] = __ldcg(src + 1);
        } else {
          x[k][0] = x[k][1] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int k = 0; k < RB; ++k) {
        acc0.x += x[k][0].x; acc0.y += x[k][0].y; acc0.z += x[k][0].z; acc0.w += x[k][0].w;
        acc1.x += x[k][1].x; acc1.y += x[k][1].y; acc1.z += x[k][1].z; acc1.w += x[k][1].w;
      }
    }
    uint4 pk;
    pk.x = pack2<kBf16>(acc0.x, acc0.y);
    pk.y = pack2<kBf16>(acc0.z, acc0.w);
    pk.z = pack2<kBf16>(acc1.x, acc1.y);
    pk.w = pack2<kBf16>(acc1.z, acc1.w);
    for (int r = 0; r < nranks; ++r) reinterpret_cast<uint4*>(outs[r])[v] = pk;
  }
  if (flags != nullptr) {
    __threadfence_system();  // this thread's stores into the peers' buffers are visible system-wide
    __syncthreads();
    if (threadIdx.x == 0) {
      int* counter = flags[rank] + 2 * nranks;
      const int done = atomicAdd(counter, 1);
      s_last = (done == static_cast<int>(gridDim.x) - 1);
      if (s_last) *counter = 0;  // for the next launch (launches of one rank are stream-ordered)
    }
    __syncthreads();
    if (s_last && static_cast<int>(threadIdx.x) < nranks) {
      __threadfence_system();
      st_release_sys_u32(flags[threadIdx.x] + nranks + rank, epoch);
    }
  }
}

// Holds the stream until words [R, 2R) of this rank's flag array have reached `epoch`: every rank's slice
// of the sum is then in this rank's output buffer. One block; bounded like every other wait here.
__global__ void __launch_bounds__(64) peers_wait_kernel(const int* done_words, int nranks, int epoch,
                                                        unsigned long long limit_ns, int* status) {
  bool ok = true;
  if (static_cast<int>(threadIdx.x) < nranks) {
    const unsigned long long t0 = global_timer_ns();
    while (ld_acquire_sys_u32(done_words + threadIdx.x) - epoch < 0) {
      if (global_timer_ns() - t0 > limit_ns) {
        ok = false;
        break;
      }
      __nanosleep(100);
    }
  }
  if (!__syncthreads_and(ok) && threadIdx.x == 0) atomicCAS(status, kStatusOk, kStatusWaitTimeout | 0x63);
}

// Padded, masked copy of the pair bias for problems whose L2 is not a multiple of 128 and / or that
// drop keys with a boolean mask: out (B*H, L2p, L2p), 8 elements (16 bytes) per thread.
template <bool kBf16>
__global__ void __launch_bounds__(256) mask_bias_kernel(const uint16_t* __restrict__ bias, long long s_b, long long s_h,
                                                        long long s_q, const uint8_t* __restrict__ key_mask,
                                                        uint16_t* __restrict__ out, int BH, int H, int L2, int L2p) {
  constexpr uint32_t NEG_INF = kBf16 ? 0xFF80u : 0xFC00u;
  const int vec_per_row = L2p / 8;
  const long long total = static_cast<long long>(BH) * L2p * vec_per_row;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int k8 = static_cast<int>(idx % vec_per_row) * 8;
    const long long rq = idx / vec_per_row;
    const int q = static_cast<int>(rq % L2p);
    const int bh = static_cast<int>(rq / L2p);
    const int b = bh / H, h = bh % H;
    uint32_t w[4] = {0u, 0u, 0u, 0u};
    if (k8 >= L2) {
      w[0] = w[1] = w[2] = w[3] = NEG_INF | (NEG_INF << 16);  // padding keys: never attended
    } else {
      uint4 v = make_uint4(0u, 0u, 0u, 0u);  // padding queries see a zero bias on the real keys
      if (q < L2) v = __ldg(reinterpret_cast<const uint4*>(bias + b * s_b + h * s_h + q * s_q + k8));
      const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
      uint2 m = make_uint2(0x01010101u, 0x01010101u);
      if (key_mask) m = __ldg(reinterpret_cast<const uint2*>(key_mask + static_cast<long long>(b) * L2 + k8));
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t mm = (e < 2 ? m.x : m.y) >> ((e & 1) * 16);
        const uint32_t lo = (mm & 0xffu) ? (vw[e] & 0xffffu) : NEG_INF;
        const uint32_t hi = (mm & 0xff00u) ? (vw[e] >> 16) : NEG_INF;
        w[e] = lo | (hi << 16);
      }
    }
    *reinterpret_cast<uint4*>(out + (static_cast<long long>(bh) * L2p + q) * L2p + k8) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// ------------------------------------------------------------------------------------------------
// Backward prologue. Blocks [0, tr_blocks): out[bh][k][q] = bias[b][h][q][k] (16-bit elements, 64 x 64
// tiles through shared memory, 16-byte global accesses on both sides). Remaining blocks: zero-fill
// of the float32 dQ accumulator, 16 bytes per thread, grid-stride.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) bwd_prologue_kernel(const uint16_t* __restrict__ bias,
                                                           uint16_t* __restrict__ bias_t, int BH, int H, int L2,
                                                           long long s_b, long long s_h, long long s_q,
                                                           int tr_blocks, float4* __restrict__ dq32,
                                                           long long dq_vec) {
  __shared__ uint32_t tile[64][33];  // [query][key pair]; odd pitch in words
  if (static_cast<int>(blockIdx.x) >= tr_blocks) {
    const long long nthreads = static_cast<long long>(gridDim.x - tr_blocks) * blockDim.x;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long v = static_cast<long long>(blockIdx.x - tr_blocks) * blockDim.x + threadIdx.x; v < dq_vec;
         v += nthreads)
      dq32[v] = z;
    return;
  }
  const int tiles = L2 / 64;
  const int per_bh = tiles * tiles;
  for (int t = blockIdx.x; t < per_bh * BH; t += tr_blocks) {
    const int bh = t / per_bh, tt = t % per_bh;
    const int q0 = (tt / tiles) * 64, k0 = (tt % tiles) * 64;
    const uint16_t* src = bias + (bh / H) * s_b + (bh % H) * s_h;
    uint16_t* dst = bias_t + static_cast<long long>(bh) * L2 * L2;
    // 64 query rows x 8 chunks of 8 keys = 512 chunks, two per thread
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int c = threadIdx.x + it * 256;
      const int rr = c >> 3, c8 = (c & 7) * 8;
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + (q0 + rr) * s_q + k0 + c8));
      uint32_t* trow = &tile[rr][c8 >> 1];
      trow[0] = v.x;
      trow[1] = v.y;
      trow[2] = v.z;
      trow[3] = v.w;
    }
    __syncthreads();
    // 64 key rows x 8 chunks of 8 queries; the 8 threads of a key row write 128 contiguous bytes
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int c = threadIdx.x + it * 256;
      const int kk = c >> 3, q8 = (c & 7) * 8;
      const int sh = (kk & 1) * 16;
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t lo = (tile[q8 + 2 * e][kk >> 1] >> sh) & 0xffffu;
        const uint32_t hi = (tile[q8 + 2 * e + 1][kk >> 1] >> sh) & 0xffffu;
        w[e] = lo | (hi << 16);
      }
      *reinterpret_cast<uint4*>(dst + static_cast<long long>(k0 + kk) * L2 + q0 + q8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------------
// Backward epilogue. Blocks [0, dq_blocks): dq = dtype(scale * dq32), 8 elements per thread,
// grid-stride. Remaining blocks: one 64 (key) x 64 (query) tile of dBias each - the key-major
// planes (p, bh, key, query) summed in plane order in registers (float4 loads along the query
// axis), transposed through shared memory, written as (bh, query, key) float32 and 16-bit with
// 16-byte stores along the key axis. Fixed order everywhere: bit-reproducible.
// ------------------------------------------------------------------------------------------------
template <int kD, bool kBf16, bool kDense>
__global__ void __launch_bounds__(256) bwd_epilogue_kernel(const float* __restrict__ dq32, uint16_t* __restrict__ dq,
                                                           long long rows, int H, int L1, int L2, long long s_b,
                                                           long long s_h, long long s_i, long long s_j, float scale,
                                                           int dq_blocks, const float* __restrict__ planes, int nplanes,
                                                           int BH, float* __restrict__ out_f32,
                                                           uint16_t* __restrict__ out_cast) {
  __shared__ float tile[64][65];  // [key][query]
  if (static_cast<int>(blockIdx.x) < dq_blocks) {
    constexpr int LPR = kD / 8;
    const long long nthreads = static_cast<long long>(dq_blocks) * blockDim.x;
    const long long total = rows * LPR;
    for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += nthreads) {
      const long long row = idx / LPR;
      const int part = static_cast<int>(idx % LPR);
      const float4 a = __ldg(reinterpret_cast<const float4*>(dq32 + row * kD + part * 8));
      const float4 c = __ldg(reinterpret_cast<const float4*>(dq32 + row * kD + part * 8 + 4));
      long long oo;
      if constexpr (kDense) oo = row * kD + part * 8;
      else oo = strided_row_offset(row, H, L1, L2, s_b, s_h, s_i, s_j) + part * 8;
      uint4 out;
      out.x = pack2<kBf16>(a.x * scale, a.y * scale);
      out.y = pack2<kBf16>(a.z * scale, a.w * scale);
      out.z = pack2<kBf16>(c.x * scale, c.y * scale);
      out.w = pack2<kBf16>(c.z * scale, c.w * scale);
      *reinterpret_cast<uint4*>(dq + oo) = out;
    }
    return;
  }
  const int tiles = (L2 + 63) / 64;  // L2 is a multiple of 8: an 8-key / 4-query vector is inside or outside as a whole
  int t = blockIdx.x - dq_blocks;
  const int q0 = (t % tiles) * 64;
  t /= tiles;
  const int k0 = (t % tiles) * 64;
  const int bh = t / tiles;
  const long long plane_stride = static_cast<long long>(BH) * L2 * L2;
  // read: thread -> key rows kr, kr + 16, kr + 32, kr + 48, four queries at qc
  const int kr = threadIdx.x >> 4, qc = (threadIdx.x & 15) * 4;
  const float* src = planes + (static_cast<long long>(bh) * L2 + k0 + kr) * L2 + q0 + qc;
  float4 acc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool q_in = q0 + qc < L2;
  // planes added in index order (bit-reproducible); the loads of four planes are in flight together:
  // with one head per GPU there are only (L2/64)^2 of these blocks and up to 24 planes each, a chain
  // of dependent memory latencies when the planes are read one at a time
  auto load = [&](int pl, int i) {
    return __ldg(reinterpret_cast<const float4*>(src + static_cast<long long>(pl) * plane_stride +
                                                 static_cast<long long>(16 * i) * L2));
  };
  int pl = 0;
  for (; pl + 4 <= nplanes; pl += 4) {
    float4 x[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int i = 0; i < 4; ++i)
        x[u][i] = (q_in && k0 + kr + 16 * i < L2) ? load(pl + u, i) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[i].x += x[u][i].x;
        acc[i].y += x[u][i].y;
        acc[i].z += x[u][i].z;
        acc[i].w += x[u][i].w;
      }
  }
  for (; pl < nplanes; ++pl) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (!q_in || k0 + kr + 16 * i >= L2) continue;
      const float4 x = load(pl, i);
      acc[i].x += x.x;
      acc[i].y += x.y;
      acc[i].z += x.z;
      acc[i].w += x.w;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float* trow = &tile[kr + 16 * i][qc];
    trow[0] = acc[i].x;
    trow[1] = acc[i].y;
    trow[2] = acc[i].z;
    trow[3] = acc[i].w;
  }
  __syncthreads();
  // write: 64 queries x 8 groups of 8 keys = 512 items, two per thread
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int c = threadIdx.x + it * 256;
    const int q = c >> 3, k8 = (c & 7) * 8;
    if (q0 + q >= L2 || k0 + k8 >= L2) continue;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = tile[k8 + e][q];
    const long long o = (static_cast<long long>(bh) * L2 + q0 + q) * L2 + k0 + k8;
    if (out_f32) {
      *reinterpret_cast<float4*>(out_f32 + o) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(out_f32 + o + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    if (out_cast) {
      uint4 pk;
      pk.x = pack2<kBf16>(v[0], v[1]);
      pk.y = pack2<kBf16>(v[2], v[3]);
      pk.z = pack2<kBf16>(v[4], v[5]);
      pk.w = pack2<kBf16>(v[6], v[7]);
      *reinterpret_cast<uint4*>(out_cast + o) = pk;
    }
  }
}

int num_sms() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

int grid_for(long long work_items, int threads) {
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(num_sms()) * 8;  // a multiple of the SM count
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

bool is_dense(const long long s4[4], int H, int L1, int L2, int D) {
  return s4[3] == D && s4[2] == static_cast<long long>(L2) * D && s4[1] == static_cast<long long>(L1) * L2 * D &&
         s4[0] == static_cast<long long>(H) * L1 * L2 * D;
}

}  // namespace

int launch_preprocess(const void* o, const void* o_resid, const long long so[4], const void* dout,
                      const long long sdo[4], float* delta, int delta_pitch, int B, int H, int L1, int L2, int D,
                      bool bf16, cudaStream_t stream) {
  const long long rows = static_cast<long long>(B) * H * L1 * L2;
  const int grid = grid_for(rows * (D / 8), 256);
  const uint16_t* op = static_cast<const uint16_t*>(o);
  const uint16_t* rp = static_cast<const uint16_t*>(o_resid);
  const uint16_t* dp = static_cast<const uint16_t*>(dout);
  const bool dense = is_dense(so, H, L1, L2, D) && is_dense(sdo, H, L1, L2, D);
  auto go = [&](auto kern) {
    kern<<<grid, 256, 0, stream>>>(op, rp, dp, delta, delta_pitch, rows, H, L1, L2, so[0], so[1], so[2], so[3],
                                   sdo[0], sdo[1], sdo[2], sdo[3]);
  };
  auto pick = [&](auto d_tag, auto bf_tag) {
    constexpr int DD = decltype(d_tag)::value;
    constexpr bool BF = decltype(bf_tag)::value;
    if (dense) {
      if (rp) go(preprocess_kernel<DD, BF, true, true>);
      else go(preprocess_kernel<DD, BF, true, false>);
    } else {
      if (rp) go(preprocess_kernel<DD, BF, false, true>);
      else go(preprocess_kernel<DD, BF, false, false>);
    }
  };
  using I32 = std::integral_constant<int, 32>;
  using I64 = std::integral_constant<int, 64>;
  if (D == 32) {
    if (bf16) pick(I32{}, std::true_type{}); else pick(I32{}, std::false_type{});
  } else {
    if (bf16) pick(I64{}, std::true_type{}); else pick(I64{}, std::false_type{});
  }
  return static_cast<int>(cudaGetLastError());
}

int launch_mask_bias(const void* bias, const long long sb[4], const uint8_t* key_mask, void* out, int B, int H, int L2,
                     int L2p, bool bf16, cudaStream_t stream) {
  const int grid = grid_for(static_cast<long long>(B) * H * L2p * (L2p / 8), 256);
  if (bf16)
    mask_bias_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(bias), sb[0], sb[1], sb[2], key_mask,
                                                     static_cast<uint16_t*>(out), B * H, H, L2, L2p);
  else
    mask_bias_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(bias), sb[0], sb[1], sb[2], key_mask,
                                                      static_cast<uint16_t*>(out), B * H, H, L2, L2p);
  return static_cast<int>(cudaGetLastError());
}

int launch_bwd_prologue(const void* bias, const long long sb[4], void* bias_t, int B, int H, int L2, float* dq32,
                        long long dq_elems, cudaStream_t stream) {
  const int sms = num_sms();
  const long long tiles = static_cast<long long>(L2 / 64) * (L2 / 64) * B * H;
  const int tr_blocks = static_cast<int>(tiles < 2LL * sms ? tiles : 2LL * sms);
  const int grid = tr_blocks + 6 * sms;
  bwd_prologue_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(bias), static_cast<uint16_t*>(bias_t),
                                                B * H, H, L2, sb[0], sb[1], sb[2], tr_blocks,
                                                reinterpret_cast<float4*>(dq32), dq_elems / 4);
  return static_cast<int>(cudaGetLastError());
}

int launch_bwd_epilogue(const float* dq32, void* dq, const long long sdq[4], int B, int H, int L1, int L2, int D,
                        float scale, const float* planes, int nplanes, float* dbias_f32, void* dbias_cast, bool bf16,
                        cudaStream_t stream) {
  const long long rows = static_cast<long long>(B) * H * L1 * L2;
  const int dq_blocks = grid_for(rows * (D / 8), 256);
  const int db_blocks = ((L2 + 63) / 64) * ((L2 + 63) / 64) * B * H;
  const int grid = dq_blocks + db_blocks;
  uint16_t* out = static_cast<uint16_t*>(dq);
  uint16_t* cast = static_cast<uint16_t*>(dbias_cast);
  const bool dense = is_dense(sdq, H, L1, L2, D);
  auto go = [&](auto kern) {
    kern<<<grid, 256, 0, stream>>>(dq32, out, rows, H, L1, L2, sdq[0], sdq[1], sdq[2], sdq[3], scale, dq_blocks,
                                   planes, nplanes, B * H, dbias_f32, cast);
  };
  auto pick = [&](auto d_tag, auto bf_tag) {
    constexpr int DD = decltype(d_tag)::value;
    constexpr bool BF = decltype(bf_tag)::value;
    if (dense) go(bwd_epilogue_kernel<DD, BF, true>);
    else go(bwd_epilogue_kernel<DD, BF, false>);
  };
  using I32 = std::integral_constant<int, 32>;
  using I64 = std::integral_constant<int, 64>;
  if (D == 32) {
    if (bf16) pick(I32{}, std::true_type{}); else pick(I32{}, std::false_type{});
  } else {
    if (bf16) pick(I64{}, std::true_type{}); else pick(I64{}, std::false_type{});
  }
  return static_cast<int>(cudaGetLastError());
}

int launch_dbias_cast(const float* src, long long n, void* dst, bool bf16, cudaStream_t stream) {
  const int grid = grid_for(n / 8 + 1, 256);
  if (bf16) dbias_cast_kernel<true><<<grid, 256, 0, stream>>>(src, n, static_cast<uint16_t*>(dst));
  else dbias_cast_kernel<false><<<grid, 256, 0, stream>>>(src, n, static_cast<uint16_t*>(dst));
  return static_cast<int>(cudaGetLastError());
}

int launch_dbias_sum_peers(const float* const* parts, int nranks, long long n, float* out_f32, void* out_cast,
                           bool bf16, int* const* flags, int rank, int epoch, unsigned long long limit_ns, int* status,
                           cudaStream_t stream) {
  const int grid = grid_for((n / 8 + 3) / 4, 256);
  uint16_t* oc = static_cast<uint16_t*>(out_cast);
  if (bf16)
    dbias_sum_peers_kernel<true><<<grid, 256, 0, stream>>>(parts, nranks, n, out_f32, oc, flags, rank, epoch, limit_ns, status);
  else
    dbias_sum_peers_kernel<false><<<grid, 256, 0, stream>>>(parts, nranks, n, out_f32, oc, flags, rank, epoch, limit_ns, status);
  return static_cast<int>(cudaGetLastError());
}

int launch_dbias_sum_peers_sliced(const float* const* parts, void* const* outs, int nranks, int rank, long long n,
                                  bool bf16, int* const* flags, const int* my_flags, int epoch,
                                  unsigned long long limit_ns, int* status, cudaStream_t stream) {
  const long long per = (n / 8 + nranks - 1) / nranks;
  const int grid = grid_for(per, 256);
  uint16_t* const* o = reinterpret_cast<uint16_t* const*>(outs);
  if (bf16)
    dbias_sum_peers_sliced_kernel<true><<<grid, 256, 0, stream>>>(parts, o, nranks, rank, n, flags, epoch, limit_ns, status);
  else
    dbias_sum_peers_sliced_kernel<false><<<grid, 256, 0, stream>>>(parts, o, nranks, rank, n, flags, epoch, limit_ns, status);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess && flags != nullptr) {
    peers_wait_kernel<<<1, 64, 0, stream>>>(my_flags + nranks, nranks, epoch, limit_ns, status);
    e = cudaGetLastError();
  }
  return static_cast<int>(e);
}

}  // namespace fta
