// Forward triangle attention for sm_100a: O = softmax(sm_scale * q k^T + bias) v and the
// softmax statistics (row max and log2 of the row sum), the work of the reference's `_attn_fwd` (flash_tt_attn.py:128-264).
//
// One CTA owns a 128-query block `jb` of one (b,h) and walks a residue class of the groups of G
// consecutive L1 rows back to back (loads and MMAs of the next group start while the softmax
// warps finish the current one). Within a group it walks the key blocks once (outer loop) and,
// inside, the G rows (inner loop), so that one 128x128 bias tile staged in shared memory serves
// G score tiles:
//
//   warp 0      : tcgen05 issuer (S = Q K^T into TMEM, O += P V with P read from TMEM)
//   warp 1      : TMA producer  (Q tiles once, K/V ring, bias double buffer)
//   warps 2-3   : idle; warps 0-3 form a warpgroup that hands most of its registers to the
//                 softmax warpgroups (setmaxnreg). The issuer has the lowest warp id so that
//                 the warp scheduler, which prefers older warps, never starves it behind the
//                 long instruction runs of the softmax warps.
//   warps 4-7   : softmax warpgroup 0 -> even rows of the group, S/P buffer 0
//   warps 8-11  : softmax warpgroup 1 -> odd rows of the group,  S/P buffer 1
//
// The producer and issuer loops run warp-uniformly (all 32 lanes) and only the TMA / MMA
// instruction itself is issued by one elected lane, so that descriptors and addresses stay
// in uniform registers.
//
// TMEM (512 columns): S buffers 2 x 128 fp32 columns, P buffers 2 x 64 columns (packed
// 16-bit pairs), O accumulators G x D columns. S and P are separate so that the next
// S = Q K^T of a warpgroup is issued as soon as the warpgroup has copied its S tile to
// registers, and is ready when the warpgroup comes back for it.
// Online softmax state (running max, running sum) lives in registers of the thread that
// owns the query row; the O accumulator is rescaled whenever the row max grew, by the same
// thread, before P is handed to the PV MMA.
#include "fta_kernels.h"
#include "tc05.cuh"

namespace fta {

namespace {

constexpr float kLog2e = 1.4426950408889634f;

template <int kD>
struct FwdCfg {
  static constexpr int G = (kD == 32) ? 4 : 2;       // rows per CTA (even)
  static constexpr int NSTAGE = (kD == 32) ? 6 : 4;  // K/V ring depth
  static constexpr int TILE_B = 128 * kD * 2;        // one 128 x D tile of 16-bit values
  static constexpr int BIAS_B = 128 * 128 * 2;       // one 128 x 128 bias tile
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_KV = OFF_Q + G * TILE_B;
  static constexpr int OFF_BIAS = OFF_KV + NSTAGE * 2 * TILE_B;
  static constexpr int OFF_BAR = OFF_BIAS + 2 * BIAS_B;
  // barrier slots
  static constexpr int B_QFULL = 0;
  static constexpr int B_QEMPTY = B_QFULL + G;
  static constexpr int B_KVFULL = B_QEMPTY + G;
  static constexpr int B_KVEMPTY = B_KVFULL + NSTAGE;
  static constexpr int B_BIASFULL = B_KVEMPTY + NSTAGE;
  static constexpr int B_BIASEMPTY = B_BIASFULL + 2;
  static constexpr int B_SFULL = B_BIASEMPTY + 2;
  static constexpr int B_SFREE = B_SFULL + 2;
  static constexpr int B_PFULL = B_SFREE + 2;
  static constexpr int B_PVDONE = B_PFULL + 2;
  static constexpr int NBAR = B_PVDONE + 2;
  static constexpr int SMEM_BYTES = OFF_BAR + NBAR * 8 + 16 + 1024;  // + tmem slot/abort + align slack
  static constexpr uint64_t SWZ = (kD == 32) ? kSwz64 : kSwz128;
  static constexpr uint32_t SBO = 8 * kD * 2;  // bytes between 8-row groups of a tile
  static constexpr uint32_t TMEM_P = 256;      // first P column
  static constexpr uint32_t TMEM_O = 384;      // first O column
  static_assert(TMEM_O + G * kD <= 512, "TMEM budget");
};

struct FwdParams {
  void* o;
  void* o_resid;  // optional: the part of O lost in rounding to 16 bits, same layout as O
  float* lse;
  int* status;
  int H, L1, L2;
  long long so_b, so_h, so_i, so_j;  // element strides of O (D stride is 1)
  float scale;                       // sm_scale
  int stat_pitch;                    // row pitch of the statistics: L2 rounded up to 128
  long long stat_stride;             // elements between the statistics planes
};

template <int N>
__device__ __forceinline__ float sel(const float (&a)[N], int idx) {
  float r = a[0];
#pragma unroll
  for (int i = 1; i < N; ++i) r = (idx == i) ? a[i] : r;
  return r;
}
template <int N>
__device__ __forceinline__ void put(float (&a)[N], int idx, float v) {
#pragma unroll
  for (int i = 0; i < N; ++i) a[i] = (idx == i) ? v : a[i];
}

template <int kD, bool kBf16>
__global__ void __launch_bounds__(384, 1)
fta_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmBias,
               const FwdParams p) {
  using C = FwdCfg<kD>;
  constexpr int G = C::G;
  extern __shared__ uint8_t smem_raw[];
  // 1 KB alignment by an offset from the shared array itself, so that the compiler keeps the
  // shared address space (ld.shared / st.shared instead of generic accesses)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sQ = smem + C::OFF_Q;
  uint8_t* sKV = smem + C::OFF_KV;
  uint8_t* sBias = smem + C::OFF_BIAS;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::NBAR);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * static_cast<uint32_t>(i); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jb = blockIdx.x, bh = blockIdx.z;
  const int b = bh / p.H, h = bh % p.H;
  const int nkb = (p.L2 + 127) / 128;  // a ragged last key block is padded by the loads (zeros) and masked by the bias (-inf)
  // This CTA walks the row groups blockIdx.y, blockIdx.y + gridDim.y, ... ("units") back to back;
  // loads and MMAs of the next unit start while the softmax warps finish the current one.
  const int ngroups = (p.L1 + G - 1) / G;
  const int nunits = (ngroups - static_cast<int>(blockIdx.y) + static_cast<int>(gridDim.y) - 1) /
                     static_cast<int>(gridDim.y);
  auto unit_i0 = [&](int u) { return (static_cast<int>(blockIdx.y) + u * static_cast<int>(gridDim.y)) * G; };
  // Every unit processes G rows: a short last group is padded with rows past L1, which the TMA
  // loads fill with zeros and the epilogue does not store.
  // (kept a run-time value: as a compile-time constant it changes the code the compiler generates
  // for the softmax loop, measurably for the worse)
  auto unit_gp = [&](int u) { return unit_i0(u) < p.L1 ? G : 0; };
  const WaitCtx w{smem_u32(abort_flag), p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < G; ++i) {
      mbar_init(bar(C::B_QFULL + i), 1);
      mbar_init(bar(C::B_QEMPTY + i), 1);
    }
    for (int i = 0; i < C::NSTAGE; ++i) {
      mbar_init(bar(C::B_KVFULL + i), 1);
      mbar_init(bar(C::B_KVEMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(C::B_BIASFULL + i), 1);
      mbar_init(bar(C::B_BIASEMPTY + i), 8);  // one arrive per softmax warp
      mbar_init(bar(C::B_SFULL + i), 1);
      mbar_init(bar(C::B_SFREE + i), 4);  // one arrive per warp of the warpgroup
      mbar_init(bar(C::B_PFULL + i), 4);
      mbar_init(bar(C::B_PVDONE + i), 1);
    }
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = *tmem_slot;

  if (warp < 4) {
    reg_dec<88>();
    if (warp == 1) {
      // ---------------------------------------------------------------- TMA producer
      if (elect_one()) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmBias);
      }
      bool ok = true;
      int tt = 0, nbias = 0;
      for (int u = 0; u < nunits && ok; ++u) {
        const int i0 = unit_i0(u), Gp = unit_gp(u);
        for (int kb = 0; kb < nkb && ok; ++kb, ++nbias) {
          const int bs = nbias & 1;
          ok = mbar_wait_warp(bar(C::B_BIASEMPTY + bs), ((nbias >> 1) & 1) ^ 1, w, 1);
          if (!ok) break;
          if (elect_one()) {
            mbar_expect_tx(bar(C::B_BIASFULL + bs), C::BIAS_B);
            tma_load_4d(smem_u32(sBias + bs * C::BIAS_B), &tmBias, bar(C::B_BIASFULL + bs), kb * 128,
                        jb * 128, h, b);
            tma_load_4d(smem_u32(sBias + bs * C::BIAS_B + 16384), &tmBias, bar(C::B_BIASFULL + bs),
                        kb * 128 + 64, jb * 128, h, b);
          }
          for (int g = 0; g < Gp; ++g, ++tt) {
            if (kb == 0) {
              // the Q tile of this row slot is free once the last Q K^T of the previous unit is done
              ok = mbar_wait_warp(bar(C::B_QEMPTY + g), (u & 1) ^ 1, w, 11);
              if (!ok) break;
              if (elect_one()) {
                mbar_expect_tx(bar(C::B_QFULL + g), C::TILE_B);
                tma_load_5d(smem_u32(sQ + g * C::TILE_B), &tmQ, bar(C::B_QFULL + g), 0, jb * 128, i0 + g,
                            h, b);
              }
            }
            const int s = tt % C::NSTAGE;
            ok = mbar_wait_warp(bar(C::B_KVEMPTY + s), ((tt / C::NSTAGE) & 1) ^ 1, w, 2);
            if (!ok) break;
            if (elect_one()) {
              mbar_expect_tx(bar(C::B_KVFULL + s), 2 * C::TILE_B);
              tma_load_5d(smem_u32(sKV + s * 2 * C::TILE_B), &tmK, bar(C::B_KVFULL + s), 0, kb * 128,
                          i0 + g, h, b);
              tma_load_5d(smem_u32(sKV + s * 2 * C::TILE_B + C::TILE_B), &tmV, bar(C::B_KVFULL + s), 0,
                          kb * 128, i0 + g, h, b);
            }
          }
        }
      }
    } else if (warp == 0) {
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_qk = umma_idesc_f16(kBf16 ? 1 : 0, 128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_f16(kBf16 ? 1 : 0, 128, kD, 0, 1);
      const uint32_t sQ_a = smem_u32(sQ), sKV_a = smem_u32(sKV);
      bool ok = true;
      // the tile sequence (unit, key block, row) flattened; `tt` = global tile index
      struct TileIt { int u, kb, g, gp, tt; };
      auto it_valid = [&](const TileIt& it) { return it.u < nunits; };
      auto it_next = [&](TileIt& it) {
        ++it.tt;
        if (++it.g == it.gp) {
          it.g = 0;
          if (++it.kb == nkb) {
            it.kb = 0;
            if (++it.u < nunits) it.gp = unit_gp(it.u);
          }
        }
      };
      int nqk[2] = {0, 0}, npv[2] = {0, 0};  // tiles issued per S / P buffer
      // S = Q_g K^T into S buffer g&1, once the buffer's previous tile has been copied out by its
      // warpgroup.
      auto issue_qk = [&](const TileIt& it) -> bool {
        const int g = it.g, s = it.tt % C::NSTAGE, wb = g & 1;
        const int n = nqk[wb];
        if (it.kb == 0 && !mbar_wait_warp(bar(C::B_QFULL + g), it.u & 1, w, 3)) return false;
        if (!mbar_wait_warp(bar(C::B_KVFULL + s), (it.tt / C::NSTAGE) & 1, w, 4)) return false;
        if (n > 0 && !mbar_wait_warp(bar(C::B_SFREE + wb), (n - 1) & 1, w, 9)) return false;
        tc_fence_after_sync();
        const uint64_t dq = umma_smem_desc(sQ_a + g * C::TILE_B, 16, C::SBO, C::SWZ);
        const uint64_t dk = umma_smem_desc(sKV_a + s * 2 * C::TILE_B, 16, C::SBO, C::SWZ);
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < kD / 16; ++ks)
            umma_ss(tbase + wb * 128, dq + ks * 2, dk + ks * 2, idesc_qk, ks > 0);
          umma_commit(bar(C::B_SFULL + wb));
          if (it.kb == nkb - 1) umma_commit(bar(C::B_QEMPTY + g));  // last use of this unit's Q tile
        }
        __syncwarp();
        ++nqk[wb];
        return true;
      };
      TileIt cur{0, 0, 0, nunits > 0 ? unit_gp(0) : 2, 0};
      TileIt ahead = cur;
      for (int k = 0; k < 2 && ok && it_valid(ahead); ++k) {
        ok = issue_qk(ahead);
        it_next(ahead);
      }
      while (ok && it_valid(cur)) {
        const int g = cur.g, s = cur.tt % C::NSTAGE, wb = g & 1;
        if (it_valid(ahead)) {
          ok = issue_qk(ahead);  // waits until the S tile two tiles back has been copied out
          if (!ok) break;
          it_next(ahead);
        }
        ok = mbar_wait_warp(bar(C::B_PFULL + wb), npv[wb] & 1, w, 5);
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t dv = umma_smem_desc(sKV_a + s * 2 * C::TILE_B + C::TILE_B, C::SBO, C::SBO, C::SWZ);
        const uint32_t acc0 = cur.kb > 0 ? 1u : 0u;
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_ts(tbase + C::TMEM_O + g * kD, tbase + C::TMEM_P + wb * 64 + ks * 8,
                    dv + ks * ((2 * C::SBO) >> 4), idesc_pv, ks > 0 ? 1u : acc0);
          umma_commit(bar(C::B_KVEMPTY + s));
          umma_commit(bar(C::B_PVDONE + wb));
        }
        __syncwarp();
        ++npv[wb];
        it_next(cur);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    reg_inc<208>();
    const int wg = (warp >> 2) - 1;
    const int row = (warp & 3) * 32 + lane;  // query row of the tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tbase + wg * 128 + lane_off;
    const uint32_t tP = tbase + C::TMEM_P + wg * 64 + lane_off;
    const f32x2 scale2 = mk2(p.scale, p.scale);
    const f32x2 log2e2 = mk2(kLog2e, kLog2e);
    int n = 0, nbias = 0;
    bool ok = true;
    for (int u = 0; u < nunits && ok; ++u) {
    const int i0 = unit_i0(u);
    const int ngi = unit_gp(u) >> 1;
    float m_used[G / 2], l_run[G / 2];  // running max (natural-log units) and running sum
#pragma unroll
    for (int i = 0; i < G / 2; ++i) {
      m_used[i] = -INFINITY;
      l_run[i] = 0.f;
    }
    for (int kb = 0; kb < nkb && ok; ++kb, ++nbias) {
      const int bs = nbias & 1;
      const uint8_t* brow = sBias + bs * C::BIAS_B + row * 128;
      for (int gi = 0; gi < ngi; ++gi, ++n) {
        const int g = 2 * gi + wg;
        ok = mbar_wait_warp(bar(C::B_SFULL + wg), n & 1, w, 6);
        if (!ok) break;
        if (gi == 0) {
          ok = mbar_wait_warp(bar(C::B_BIASFULL + bs), (nbias >> 1) & 1, w, 7);
          if (!ok) break;
        }
        tc_fence_after_sync();
        uint32_t sr[128];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, sr + c * 32);
        tmem_ld_wait();
        // the S buffer may now be overwritten by the next Q K^T of this warpgroup
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(C::B_SFREE + wg));
        // pass 1: x = s*scale + bias (natural-log units), row max
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const uint4 bv = *reinterpret_cast<const uint4*>(brow + (c >> 3) * 16384 +
                                                            (((c & 7) ^ (row & 7)) << 4));
          const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float b0, b1, x0, x1;
            unpack2<kBf16>(bw[e], b0, b1);
            const f32x2 x = fma2(mk2(__uint_as_float(sr[c * 8 + 2 * e]), __uint_as_float(sr[c * 8 + 2 * e + 1])),
                                 scale2, mk2(b0, b1));
            un2(x, x0, x1);
            sr[c * 8 + 2 * e] = __float_as_uint(x0);
            sr[c * 8 + 2 * e + 1] = __float_as_uint(x1);
            if (e == 0) mx0 = max3(mx0, x0, x1);
            else if (e == 1) mx1 = max3(mx1, x0, x1);
            else if (e == 2) mx2 = max3(mx2, x0, x1);
            else mx3 = max3(mx3, x0, x1);
          }
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        if (gi == ngi - 1) {  // last use of this bias stage by this warp
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(C::B_BIASEMPTY + bs));
        }
        const float m_old = sel(m_used, gi);
        const float l_old = sel(l_run, gi);
        // The reference maximum follows the running row maximum exactly (the O accumulator is rescaled
        // whenever it grows), so the largest probabilities of a row are powers of two times an exactly
        // representable value when they are rounded to 16 bits for the PV MMA. Letting the reference
        // lag (rescaling only after a growth of 2^8) costs the same time here and doubles the error
        // of O and of delta = rowsum(dO * O) on peaked rows, which dBias then sums over all L1 rows.
        const bool need = mx > m_old;
        const float m_new = need ? mx : m_old;
        const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = need ? fast_exp2((m_old - m_safe) * kLog2e) : 1.0f;
        if (kb > 0 && __any_sync(0xffffffffu, need)) {
          // The rescale reads and writes the O accumulator of this row, so the row's previous PV MMA
          // must be done. With two or more rows per warpgroup that was waited for a tile ago; with a
          // single row the previous tile WAS this row.
          if constexpr (G == 2) {
            ok = mbar_wait_warp(bar(C::B_PVDONE + wg), (n - 1) & 1, w, 13);
            if (!ok) break;
            tc_fence_after_sync();
          }
#pragma unroll
          for (int c = 0; c < kD / 32; ++c) {
            uint32_t orr[32];
            const uint32_t ta = tbase + C::TMEM_O + g * kD + c * 32 + lane_off;
            tmem_ld32(ta, orr);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) orr[j] = __float_as_uint(__uint_as_float(orr[j]) * alpha);
            tmem_st32(ta, orr);
          }
        }
        // the P buffer is free once the PV MMA of this warpgroup's previous tile is done
        if (n > 0) {
          ok = mbar_wait_warp(bar(C::B_PVDONE + wg), (n - 1) & 1, w, 10);
          if (!ok) break;
        }
        // pass 2: p = 2^((x - m) * log2e), row sum, pack, hand P to the tensor core through TMEM
        const f32x2 nm2 = mk2(-m_safe, -m_safe);
        f32x2 sum2a = mk2(0.f, 0.f), sum2b = mk2(0.f, 0.f);
        // One fused multiply-add per pair while every row max of the warp is moderate; rows with a
        // huge |max| (keys masked with -1e9) need (x - m) formed first: it is exact when x is close
        // to m whatever their magnitude, whereas x*log2e - m*log2e would round m*log2e to the ulp
        // of 1e9.
        const bool moderate = __all_sync(0xffffffffu, fabsf(m_safe) <= 1.0e4f);
        if (moderate) {
          const float nml = -m_safe * kLog2e;
          const f32x2 nml2 = mk2(nml, nml);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float y0, y1;
              un2(fma2(mk2(__uint_as_float(sr[c * 32 + 2 * j]), __uint_as_float(sr[c * 32 + 2 * j + 1])), log2e2, nml2),
                  y0, y1);
              const float p0 = fast_exp2(y0), p1 = fast_exp2(y1);
              if (j & 1) sum2b = add2(sum2b, mk2(p0, p1));
              else sum2a = add2(sum2a, mk2(p0, p1));
              pk[j] = pack2<kBf16>(p0, p1);
            }
            tmem_st16(tP + c * 16, pk);
          }
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float y0, y1;
              un2(mul2(add2(mk2(__uint_as_float(sr[c * 32 + 2 * j]), __uint_as_float(sr[c * 32 + 2 * j + 1])), nm2),
                       log2e2),
                  y0, y1);
              const float p0 = fast_exp2(y0), p1 = fast_exp2(y1);
              if (j & 1) sum2b = add2(sum2b, mk2(p0, p1));
              else sum2a = add2(sum2a, mk2(p0, p1));
              pk[j] = pack2<kBf16>(p0, p1);
            }
            tmem_st16(tP + c * 16, pk);
          }
        }
        float s0, s1;
        un2(add2(sum2a, sum2b), s0, s1);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(C::B_PFULL + wg));
        const float l_new = l_old * alpha + (s0 + s1);
        put(m_used, gi, m_new);
        put(l_run, gi, l_new);

        if (kb == nkb - 1) {
          // epilogue of row g: wait for the last PV, normalise, store O and the log-sum-exp.
          // (Consumes PVDONE phase n; no later tile of this warpgroup waits for it again.)
          ok = mbar_wait_warp(bar(C::B_PVDONE + wg), n & 1, w, 8);
          if (!ok) break;
          tc_fence_after_sync();
          const int i = i0 + g;
          // a row whose every key is masked has an empty sum: O = 0 and statistics that make the
          // backward pass recompute P = 0
          const float inv = l_new > 0.f ? 1.0f / l_new : 0.f;
          const int j = jb * 128 + row;
          const bool live = i < p.L1 && j < p.L2;  // padding rows of a short group / a ragged query block
          const long long ooff = b * p.so_b + h * p.so_h + static_cast<long long>(i) * p.so_i +
                                 static_cast<long long>(j) * p.so_j;
          uint16_t* optr = reinterpret_cast<uint16_t*>(p.o) + ooff;
          // O - dtype(O), rounded to the same dtype: with it the backward preprocess forms
          // delta = rowsum(dO * O) from O to 16 mantissa bits instead of 8 (bf16)
          uint16_t* rptr = p.o_resid ? reinterpret_cast<uint16_t*>(p.o_resid) + ooff : nullptr;
#pragma unroll
          for (int c = 0; c < kD / 32; ++c) {
            uint32_t orr[32];
            tmem_ld32(tbase + C::TMEM_O + g * kD + c * 32 + lane_off, orr);
            tmem_ld_wait();
            if (live) {
#pragma unroll
              for (int v4 = 0; v4 < 4; ++v4) {
                uint4 ov;
                ov.x = pack2<kBf16>(__uint_as_float(orr[v4 * 8 + 0]) * inv, __uint_as_float(orr[v4 * 8 + 1]) * inv);
                ov.y = pack2<kBf16>(__uint_as_float(orr[v4 * 8 + 2]) * inv, __uint_as_float(orr[v4 * 8 + 3]) * inv);
                ov.z = pack2<kBf16>(__uint_as_float(orr[v4 * 8 + 4]) * inv, __uint_as_float(orr[v4 * 8 + 5]) * inv);
                ov.w = pack2<kBf16>(__uint_as_float(orr[v4 * 8 + 6]) * inv, __uint_as_float(orr[v4 * 8 + 7]) * inv);
                *reinterpret_cast<uint4*>(optr + c * 32 + v4 * 8) = ov;
                if (rptr) {
                  const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w};
                  uint32_t rw[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    float r0, r1;
                    unpack2<kBf16>(ow[e], r0, r1);
                    rw[e] = pack2<kBf16>(__uint_as_float(orr[v4 * 8 + 2 * e]) * inv - r0,
                                         __uint_as_float(orr[v4 * 8 + 2 * e + 1]) * inv - r1);
                  }
                  *reinterpret_cast<uint4*>(rptr + c * 32 + v4 * 8) = make_uint4(rw[0], rw[1], rw[2], rw[3]);
                }
              }
            }
          }
          if (i < p.L1) {
            float m_safe_out = m_safe;
            // softmax statistics for the backward pass: -max (natural-log units) and -log2(sum).
            // Kept apart: their sum in one float would lose log2(sum) when |max| is huge.
            // (queries past L2 in a ragged block get 0 / -inf / -inf: whatever their logits, P = 0)
            const long long ridx = (static_cast<long long>(bh) * p.L1 + i) * p.stat_pitch + j;
            const bool empty = !(l_new > 0.f) || j >= p.L2;
            const float nl = empty ? -INFINITY : -log2f(l_new);
            if (j >= p.L2) m_safe_out = 0.f;
            p.lse[ridx] = -m_safe_out;
            p.lse[p.stat_stride + ridx] = nl;
            // plane 2: both in one number, c = -(max*log2e + log2 sum), for rows where that loses
            // nothing; NaN marks rows whose max is so large (fully masked rows) that the
            // backward pass must use the two parts separately
            p.lse[2 * p.stat_stride + ridx] =
                (fabsf(m_safe_out) > 1.0e4f) ? __int_as_float(0x7fc00000) : fmaf(-m_safe_out, kLog2e, nl);
          }
        }
      }
    }
    }  // units
  }

  // ---------------------------------------------------------------------- tear-down
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) __nanosleep(20000);  // let copies already in flight land before the CTA exits
  if (warp == 0) tmem_dealloc(tbase, 512);
}

template <int kD, bool kBf16>
int launch_fwd_t(const FwdArgs& a, cudaStream_t stream) {
  using C = FwdCfg<kD>;
  static PerDeviceOnce smem_attr;
  auto kern = fta_fwd_kernel<kD, kBf16>;
  if (cudaError_t e = ensure_dynamic_smem(smem_attr, kern, C::SMEM_BYTES)) return static_cast<int>(e);
  FwdParams p;
  p.o = a.o;
  p.o_resid = a.o_resid;
  p.lse = a.lse;
  p.status = a.status;
  p.H = a.H;
  p.L1 = a.L1;
  p.L2 = a.L2;
  p.so_b = a.so[0];
  p.so_h = a.so[1];
  p.so_i = a.so[2];
  p.so_j = a.so[3];
  p.scale = a.sm_scale;
  p.stat_pitch = (a.L2 + 127) / 128 * 128;
  p.stat_stride = static_cast<long long>(a.B) * a.H * a.L1 * p.stat_pitch;
  // Row groups are dealt round-robin to grid.y CTAs per (query block, head). Pick the smallest
  // grid.y whose schedule (waves of one CTA per SM, the longest CTA setting the pace) is within
  // 3 % of the best: few long-lived CTAs amortise their start-up and keep the pipeline full
  // across row groups.
  const int ngroups = (a.L1 + C::G - 1) / C::G;
  const long long per = static_cast<long long>((a.L2 + 127) / 128) * a.B * a.H;
  int sms = 148;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  int best_gy = 1;
  {
    double best = 0.0;
    const int gy_max = ngroups;
    // first pass: best efficiency; second: smallest gy close to it
    for (int pass = 0; pass < 2; ++pass) {
      for (int gy = 1; gy <= gy_max; ++gy) {
        const long long ctas = per * gy;
        const long long waves = (ctas + sms - 1) / sms;
        const int longest = (ngroups + gy - 1) / gy;
        // fixed cost per CTA of about a third of a row group
        const double eff = static_cast<double>(per) * ngroups /
                           (static_cast<double>(waves) * sms * (longest + 0.35));
        if (pass == 0) {
          if (eff > best) best = eff;
        } else if (eff >= 0.97 * best) {
          best_gy = gy;
          break;
        }
      }
    }
  }
  dim3 grid((a.L2 + 127) / 128, best_gy, a.B * a.H);
  kern<<<grid, 384, C::SMEM_BYTES, stream>>>(a.tmQ, a.tmK, a.tmV, a.tmBias, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

int launch_fwd(const FwdArgs& a, cudaStream_t stream) {
  if (a.D == 32) return a.bf16 ? launch_fwd_t<32, true>(a, stream) : launch_fwd_t<32, false>(a, stream);
  return a.bf16 ? launch_fwd_t<64, true>(a, stream) : launch_fwd_t<64, false>(a, stream);
}

int fwd_rows_per_cta(int D) { return D == 32 ? FwdCfg<32>::G : FwdCfg<64>::G; }

}  // namespace fta
