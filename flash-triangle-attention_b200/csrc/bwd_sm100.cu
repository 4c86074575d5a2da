// Backward triangle attention for sm_100a: dQ, dK, dV and dBias, the work of the reference's
// `_attn_bwd` (flash_tt_attn.py:442-550) with each score tile visited ONCE (5 MMAs and one
// exp2 per score instead of the reference's two passes).
//
// A CTA owns one key block `kb` of one (b,h) and the r-th of NP nearly equal blocks of consecutive
// L1 rows, which it walks in groups of G rows. For each group it keeps K/V of the G
// rows in shared memory and dK/dV of the G rows in TMEM, and walks the query blocks `jb`
// (outer) and the G rows (inner):
//
//   S^T  = K Q^T, dP^T = V dO^T                       (tcgen05, operands in smem)
//   P^T  = exp2((S^T*scale + bias^T - max)*log2e - log2 sum),  dS^T = P^T * (dP^T - delta)   (CUDA cores)
//   dV  += P^T dO, dK += dS^T Q                        (A operand read from TMEM)
//   dQ   = dS K                                        (dS staged in smem, M-major)
//
// Four compute warpgroups own one 32-query quarter of the tile each and move in step: one barrier
// per phase collects all sixteen warps, and the issuer answers each with one batch of MMAs (after
// phase 1: dV of this tile and S^T of the NEXT one; after phase 2: dK and the next dP^T), so the
// operands of the next phase are always a whole phase ahead and no warpgroup ever waits for
// another one's share of a tile. The bias is read from a transposed copy (key-major) so that the
// thread that owns a key row reads its query columns with 16-byte shared-memory loads.
//
// dBias: each thread owns one key column and 32 query rows of the (jb,kb) tile and sums dS
// (float32, before rounding) over the G rows in registers. At the end of a query block each
// warpgroup parks its 16 KB box of sums in shared memory that is idle at that moment and the
// store warp adds it to the CTA's PRIVATE float32 plane (plane index r, key-major) with a TMA tile
// reduction. A plane element is only ever touched by one CTA, one addition per group, each
// completed before the next, so the result is bit-exact run to run; the planes are summed in
// fixed order by the finalise kernel.
// dQ leaves the CTA the same way: TMEM -> shared memory -> TMA reduction into a zero-initialised
// float32 buffer (sum over key blocks). Every route out of an SM carries about 20 bytes per
// cycle; the TMA route costs the compute warps nothing but the shared-memory writes.
//
//   warp 0     : tcgen05 issuer (S^T, dP^T, dV, dK; lowest warp id: the scheduler prefers older warps)
//   warp 1     : TMA producer        warp 2 : issuer of the dQ MMAs        warp 3 : store warp (TMA reductions)
//   warps 4-19 : four compute warpgroups, one 32-query quarter of the tile each; quarters 0-1
//                (half 0) also store dV, quarters 2-3 (half 1) store dK
// Producer and issuer loops run warp-uniformly; one elected lane issues the TMA / MMA.
#include "fta_kernels.h"
#include "tc05.cuh"

namespace fta {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kBwdThreads = 640;    // 4 service warps + 16 compute warps
constexpr int kAuxRegs = 64;        // registers per thread of the service warpgroup
constexpr int kComputeRegs = 104;   // 512 * 104 + 128 * 64 == 640 * 96, the CTA's register allotment at launch

template <int kD>
struct BwdCfg {
  static constexpr int G = (kD == 32) ? 3 : 1;  // rows per group (TMEM: 256 + 2*D + 2*D*G <= 512)
  static constexpr int NQ = (kD == 32) ? 3 : 2;  // Q/dO ring depth
  // dQ tiles leave through a shared-memory staging tile and a TMA reduction (D = 32); at D = 64
  // shared memory has no room for the tile and dQ is reduced with red.global from registers
  static constexpr bool DQ_TMA = (kD == 32);
  static constexpr int DQS_B = DQ_TMA ? 128 * 32 * 4 : 0;
  static constexpr int TILE_B = 128 * kD * 2;
  static constexpr int STAGE_B = 2 * TILE_B + 2048;  // Q, dO, -max[128], -log2sum[128], delta[128], c[128]
  static constexpr int BIAS_B = 128 * 128 * 2;
  static constexpr int DS_B = 128 * 128 * 2;
  static constexpr int OFF_KV = 0;
  static constexpr int OFF_QDO = OFF_KV + G * 2 * TILE_B;
  static constexpr int OFF_BIAS = OFF_QDO + NQ * STAGE_B;
  static constexpr int OFF_DS = OFF_BIAS + 2 * BIAS_B;
  static constexpr int OFF_DQS = OFF_DS + DS_B;
  static constexpr int OFF_BAR = OFF_DQS + DQS_B;
  static constexpr int B_KVFULL = 0;
  static constexpr int B_KVFREE = 1;
  static constexpr int B_QDOFULL = 2;
  static constexpr int B_QDOEMPTY = B_QDOFULL + NQ;
  static constexpr int B_BIASFULL = B_QDOEMPTY + NQ;
  static constexpr int B_BIASEMPTY = B_BIASFULL + 2;
  static constexpr int B_SFULL = B_BIASEMPTY + 2;   // S^T of the next tile is in TMEM
  static constexpr int B_DPFULL = B_SFULL + 1;      // dP^T of the next tile is in TMEM
  static constexpr int B_P1FULL = B_DPFULL + 1;     // all sixteen compute warps have written P^T
  static constexpr int B_P2FULL = B_P1FULL + 1;     // ... dS^T (TMEM and the shared-memory staging tile)
  static constexpr int B_DQDONE = B_P2FULL + 1;
  static constexpr int B_ACCFULL = B_DQDONE + 1;
  static constexpr int B_ACCFREE = B_ACCFULL + 1;
  static constexpr int B_DQSFULL = B_ACCFREE + 1;
  static constexpr int B_DQSFREE = B_DQSFULL + 1;
  // dBias flush of query half h: box of its first / second warpgroup written, first box read.
  // One barrier per turn: a single one would see two phases per query block, and the store warp
  // may lag a whole phase behind, which a parity wait cannot tell from being on time.
  static constexpr int B_FLA = B_DQSFREE + 1;
  static constexpr int B_FLB = B_FLA + 2;
  static constexpr int B_DSFREE = B_FLB + 2;  // the two boxes parked in the dS tile have been read
  static constexpr int NBAR = B_DSFREE + 1;
  static constexpr int SMEM_BYTES = OFF_BAR + NBAR * 8 + 16 + 1024;  // + tmem slot / abort flag + alignment slack
  static constexpr uint64_t SWZ = (kD == 32) ? kSwz64 : kSwz128;
  static constexpr uint32_t ROW_B = kD * 2;
  static constexpr uint32_t SBO = 8 * ROW_B;
  // TMEM columns
  static constexpr uint32_t TM_ST = 0;
  static constexpr uint32_t TM_DP = 128;
  static constexpr uint32_t TM_DQ = 256;             // two dQ buffers of kD columns
  static constexpr uint32_t TM_ACC = 256 + 2 * kD;   // dK_g at TM_ACC + g*2*kD, dV_g right after
  static_assert(TM_ACC + G * 2 * kD <= 512, "TMEM budget");
};

struct BwdParams {
  const float* lse;  // three planes: -max (natural-log units), -log2(sum), c (see the forward kernel)
  const float* delta;
  float* dq32;
  void* dk;
  void* dv;
  int* status;
  int H, L1, L2, NP, BH;
  int stat_pitch;  // row pitch of lse / delta: L2 rounded up to 128
  long long sdk[4], sdv[4];
  float scale;  // sm_scale
  long long stat_stride;  // elements between the statistics planes
};

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

template <int kD, bool kBf16>
__global__ void __launch_bounds__(kBwdThreads, 1)
fta_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
               const __grid_constant__ CUtensorMap tmBiasT, const __grid_constant__ CUtensorMap tmDQ,
               const __grid_constant__ CUtensorMap tmPlane, const BwdParams p) {
  using C = BwdCfg<kD>;
  constexpr int G = C::G;
  extern __shared__ uint8_t smem_raw[];
  // 1 KB alignment by an offset from the shared array itself, so that the compiler keeps the
  // shared address space (ld.shared / st.shared instead of generic accesses)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sKV = smem + C::OFF_KV;    // [g][K tile | V tile]
  uint8_t* sQDO = smem + C::OFF_QDO;  // [stage][Q | dO | lse | delta]
  uint8_t* sBias = smem + C::OFF_BIAS;  // [stage][query half][key row][64 queries], 128B swizzle
  uint8_t* sDS = smem + C::OFF_DS;
  uint8_t* sDQ = smem + C::OFF_DQS;  // float32 dQ tile on its way to the TMA reduction
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::NBAR);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * static_cast<uint32_t>(i); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // a ragged last block (L2 not a multiple of 128) is padded: loads fill zeros, the key-major bias
  // copy holds -inf for keys past L2, the statistics give P = 0 for queries past L2, stores are clipped
  const int nkb = (p.L2 + 127) / 128, nq = nkb;
  const int kb = blockIdx.x % nkb;
  const int r = (blockIdx.x / nkb) % p.NP;
  const int bh = blockIdx.x / (nkb * p.NP);
  const int b = bh / p.H, h = bh % p.H;
  // This CTA's rows: the r-th of NP nearly equal blocks of consecutive L1 rows (sizes differ by at
  // most one row, none empty since NP <= L1), walked in groups of G rows with a short last group.
  const int row_begin = static_cast<int>(static_cast<long long>(r) * p.L1 / p.NP);
  const int row_end = static_cast<int>(static_cast<long long>(r + 1) * p.L1 / p.NP);
  const int ngroups = (row_end - row_begin + G - 1) / G;
  const WaitCtx w{smem_u32(abort_flag), p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar(C::B_KVFULL), 1);
    mbar_init(bar(C::B_KVFREE), 2);  // main issuer + dQ issuer
    for (int i = 0; i < C::NQ; ++i) {
      mbar_init(bar(C::B_QDOFULL + i), 1);
      mbar_init(bar(C::B_QDOEMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(C::B_BIASFULL + i), 1);
      mbar_init(bar(C::B_BIASEMPTY + i), 1);   // store warp, once the boxes parked in the stage are read
      mbar_init(bar(C::B_FLA + i), 4);         // the four warps of the warpgroup that wrote the box
      mbar_init(bar(C::B_FLB + i), 4);
    }
    mbar_init(bar(C::B_SFULL), 1);
    mbar_init(bar(C::B_DPFULL), 1);
    mbar_init(bar(C::B_P1FULL), 16);  // one arrive per compute warp
    mbar_init(bar(C::B_P2FULL), 16);
    mbar_init(bar(C::B_DQDONE), 1);
    mbar_init(bar(C::B_ACCFULL), 1);
    mbar_init(bar(C::B_ACCFREE), 16);
    mbar_init(bar(C::B_DQSFULL), 16);
    mbar_init(bar(C::B_DQSFREE), 1);
    mbar_init(bar(C::B_DSFREE), 1);
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
    reg_dec<kAuxRegs>();
    if (warp == 1) {
      // ---------------------------------------------------------------- TMA producer
      if (elect_one()) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmDO);
        tma_prefetch_desc(&tmBiasT);
        tma_prefetch_desc(&tmDQ);
        tma_prefetch_desc(&tmPlane);
      }
      // K/V/Q/dO tiles stream through L2 (each is read within a short window and never again);
      // the bias tiles are re-read by every group and stay
      const uint64_t pol_stream = l2_policy_evict_first(), pol_keep = l2_policy_evict_last();
      bool ok = true;
      int tt = 0, nb = 0;
      for (int n = 0; n < ngroups && ok; ++n) {
        const int i0 = row_begin + n * G;
        const int Gc = min(G, row_end - i0);
        ok = mbar_wait_warp(bar(C::B_KVFREE), (n & 1) ^ 1, w, 0x21);
        if (!ok) break;
        if (elect_one()) {
          mbar_expect_tx(bar(C::B_KVFULL), Gc * 2 * C::TILE_B);
          for (int g = 0; g < Gc; ++g) {
            tma_load_5d_hint(smem_u32(sKV + g * 2 * C::TILE_B), &tmK, bar(C::B_KVFULL), 0, kb * 128, i0 + g, h, b,
                             pol_stream);
            tma_load_5d_hint(smem_u32(sKV + g * 2 * C::TILE_B + C::TILE_B), &tmV, bar(C::B_KVFULL), 0, kb * 128,
                             i0 + g, h, b, pol_stream);
          }
          // K/V of the next group are read by no other CTA: bring them into L2 a whole group ahead
          if (n + 1 < ngroups) {
            const int i1 = row_begin + (n + 1) * G;
            for (int g = 0; g < min(G, row_end - i1); ++g) {
              tma_prefetch_l2_5d(&tmK, 0, kb * 128, i1 + g, h, b);
              tma_prefetch_l2_5d(&tmV, 0, kb * 128, i1 + g, h, b);
            }
          }
        }
        for (int jb = 0; jb < nq && ok; ++jb, ++nb) {
          const int bs = nb & 1;
          ok = mbar_wait_warp(bar(C::B_BIASEMPTY + bs), ((nb >> 1) & 1) ^ 1, w, 0x22);
          if (!ok) break;
          if (elect_one()) {
            // transposed bias: innermost coordinate = query, then key
            mbar_expect_tx(bar(C::B_BIASFULL + bs), C::BIAS_B);
            tma_load_4d_hint(smem_u32(sBias + bs * C::BIAS_B), &tmBiasT, bar(C::B_BIASFULL + bs), jb * 128,
                             kb * 128, h, b, pol_keep);
            tma_load_4d_hint(smem_u32(sBias + bs * C::BIAS_B + 16384), &tmBiasT, bar(C::B_BIASFULL + bs),
                             jb * 128 + 64, kb * 128, h, b, pol_keep);
          }
          for (int g = 0; g < Gc; ++g, ++tt) {
            const int s = tt % C::NQ;
            ok = mbar_wait_warp(bar(C::B_QDOEMPTY + s), ((tt / C::NQ) & 1) ^ 1, w, 0x23);
            if (!ok) break;
            if (elect_one()) {
              uint8_t* st = sQDO + s * C::STAGE_B;
              mbar_expect_tx(bar(C::B_QDOFULL + s), 2 * C::TILE_B + 2048);
              tma_load_5d_hint(smem_u32(st), &tmQ, bar(C::B_QDOFULL + s), 0, jb * 128, i0 + g, h, b, pol_stream);
              tma_load_5d_hint(smem_u32(st + C::TILE_B), &tmDO, bar(C::B_QDOFULL + s), 0, jb * 128, i0 + g, h, b,
                               pol_stream);
              const long long roff = (static_cast<long long>(bh) * p.L1 + i0 + g) * p.stat_pitch + jb * 128;
              bulk_load_1d(smem_u32(st + 2 * C::TILE_B), p.lse + roff, 512, bar(C::B_QDOFULL + s));
              bulk_load_1d(smem_u32(st + 2 * C::TILE_B + 512), p.lse + p.stat_stride + roff, 512,
                           bar(C::B_QDOFULL + s));
              bulk_load_1d(smem_u32(st + 2 * C::TILE_B + 1024), p.delta + roff, 512, bar(C::B_QDOFULL + s));
              bulk_load_1d(smem_u32(st + 2 * C::TILE_B + 1536), p.lse + 2 * p.stat_stride + roff, 512,
                           bar(C::B_QDOFULL + s));
            }
          }
        }
      }
    } else if (warp == 0) {
      // ---------------------------------------------------------------- MMA issuer
      // Two hand-overs per tile: after phase 1 (P^T written) it issues dV and the next tile's S^T;
      // after phase 2 (dS^T written) dK and the next tile's dP^T. The next S^T / dP^T are therefore
      // in flight while the compute warps work through the other phase.
      constexpr int fmt = kBf16 ? 1 : 0;
      constexpr uint32_t idesc_acc = umma_idesc_f16(fmt, 128, kD, 0, 1);  // dV, dK (A in TMEM, B M-major)
      const uint32_t sKV_a = smem_u32(sKV), sQDO_a = smem_u32(sQDO);
      bool ok = true;
      int tt = 0;
      constexpr uint32_t idesc_full = umma_idesc_f16(fmt, 128, 128, 0, 0);  // S^T, dP^T: all 128 queries
      // Descriptors are built from 32-bit low words (address and leading-dimension offset; the high
      // word is a compile-time constant) at the top of a tile, BEFORE the waits, so that a hand-over
      // is wait -> fence -> ten tcgen05.mma + commit back to back by one elected lane.
      constexpr uint32_t HI = (C::SBO >> 4) | (1u << 14) | (static_cast<uint32_t>(C::SWZ) << 29);
      auto mk = [](uint32_t lo) { return (static_cast<uint64_t>(HI) << 32) | lo; };
      auto lo_k = [](uint32_t addr) { return ((addr & 0x3FFFFu) >> 4) | (1u << 16); };            // K-major: lbo = 16 bytes
      auto lo_m = [](uint32_t addr) { return ((addr & 0x3FFFFu) >> 4) | ((C::SBO >> 4) << 16); };  // M-major: lbo = SBO
      constexpr uint32_t KSTEP = (2 * C::SBO) >> 4;  // 16 rows further (M-major operand), in descriptor units
      int slot = 0;  // ring slot of tile tt
      uint32_t ring_par = 0;
      for (int n = 0; n < ngroups && ok; ++n) {
        const int i0 = row_begin + n * G;
        const int Gc = min(G, row_end - i0);
        const int T = nq * Gc;
        ok = mbar_wait_warp(bar(C::B_KVFULL), n & 1, w, 0x32) && mbar_wait_warp(bar(C::B_QDOFULL + slot), ring_par, w, 0x31);
        if (!ok) break;
        tc_fence_after_sync();
        {
          const uint32_t st = sQDO_a + slot * C::STAGE_B;
          if (elect_one()) {
#pragma unroll
            for (int which = 0; which < 2; ++which) {
              const uint64_t dA = mk(lo_k(sKV_a + which * C::TILE_B)), dB = mk(lo_k(st + which * C::TILE_B));
              const uint32_t td = tbase + (which ? C::TM_DP : C::TM_ST);
#pragma unroll
              for (int ks = 0; ks < kD / 16; ++ks) umma_ss(td, dA + ks * 2, dB + ks * 2, idesc_full, ks > 0);
              umma_commit(bar(which ? C::B_DPFULL : C::B_SFULL));
            }
          }
          __syncwarp();
        }
        int g = 0, jb = 0;
        for (int t = 0; t < T && ok; ++t, ++tt) {
          const bool more = t + 1 < T;
          int gn = g + 1;
          if (gn == Gc) gn = 0;
          int slot_n = slot + 1;
          uint32_t par_n = ring_par;
          if (slot_n == C::NQ) {
            slot_n = 0;
            par_n ^= 1u;
          }
          const uint32_t par = tt & 1;
          const uint32_t accf = jb > 0 ? 1u : 0u;
          const uint32_t st = sQDO_a + slot * C::STAGE_B, stn = sQDO_a + slot_n * C::STAGE_B;
          const uint32_t kvn = sKV_a + gn * 2 * C::TILE_B;
          const uint32_t tacc = tbase + C::TM_ACC + g * 2 * kD;
          const uint32_t lo_dO = lo_m(st + C::TILE_B), lo_Q = lo_m(st);
          const uint32_t lo_Kn = lo_k(kvn), lo_Vn = lo_k(kvn + C::TILE_B);
          const uint32_t lo_Qn = lo_k(stn), lo_dOn = lo_k(stn + C::TILE_B);
          asm volatile("" ::"r"(lo_dO), "r"(lo_Q), "r"(lo_Kn), "r"(lo_Vn), "r"(lo_Qn), "r"(lo_dOn), "r"(tacc));
          // phase 1 done: dV, then the next S^T
          ok = mbar_wait_warp(bar(C::B_P1FULL), par, w, 0x33);
          if (ok && t == 0 && n > 0) ok = mbar_wait_warp(bar(C::B_ACCFREE), (n - 1) & 1, w, 0x34);
          if (ok && more) ok = mbar_wait_warp(bar(C::B_QDOFULL + slot_n), par_n, w, 0x35);
          if (!ok) break;
          tc_fence_after_sync();
          if (elect_one()) {
            const uint64_t dB = mk(lo_dO);
            const uint32_t ta = tbase + C::TM_ST;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              umma_ts(tacc + kD, ta + (ks >> 1) * 32 + (ks & 1) * 8, dB + ks * KSTEP, idesc_acc, ks > 0 ? 1u : accf);
            if (more) {
              const uint64_t dA = mk(lo_Kn), dQn = mk(lo_Qn);
#pragma unroll
              for (int ks = 0; ks < kD / 16; ++ks) umma_ss(ta, dA + ks * 2, dQn + ks * 2, idesc_full, ks > 0);
              umma_commit(bar(C::B_SFULL));
            }
          }
          __syncwarp();
          // phase 2 done: dK, then the next dP^T
          ok = mbar_wait_warp(bar(C::B_P2FULL), par, w, 0x39);
          if (!ok) break;
          tc_fence_after_sync();
          if (elect_one()) {
            const uint64_t dB = mk(lo_Q);
            const uint32_t ta = tbase + C::TM_DP;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              umma_ts(tacc, ta + (ks >> 1) * 32 + (ks & 1) * 8, dB + ks * KSTEP, idesc_acc, ks > 0 ? 1u : accf);
            umma_commit(bar(C::B_QDOEMPTY + slot));  // every MMA that reads this Q/dO stage has been issued
            if (more) {
              const uint64_t dA = mk(lo_Vn), dOn = mk(lo_dOn);
#pragma unroll
              for (int ks = 0; ks < kD / 16; ++ks) umma_ss(ta, dA + ks * 2, dOn + ks * 2, idesc_full, ks > 0);
              umma_commit(bar(C::B_DPFULL));
            }
          }
          __syncwarp();
          slot = slot_n;
          ring_par = par_n;
          g = gn;
          if (gn == 0) ++jb;
        }
        if (ok) {
          if (elect_one()) {
            umma_commit(bar(C::B_ACCFULL));
            umma_commit(bar(C::B_KVFREE));
          }
          __syncwarp();
        }
      }
    } else if (warp == 2) {
      // ---------------------------------------------------------------- dQ issuer
      // dQ = dS K needs the dS rows of all four quarters; it writes its own TMEM columns and reads no
      // Q/dO stage, so it is issued from a second warp and does not hold up the main issuer.
      constexpr uint32_t idesc_dq = umma_idesc_f16(kBf16 ? 1 : 0, 128, kD, 1, 1);  // A, B M-major
      const uint32_t sKV_a = smem_u32(sKV), sDS_a = smem_u32(sDS);
      bool ok = true;
      int tt = 0;
      for (int n = 0; n < ngroups && ok; ++n) {
        const int i0 = row_begin + n * G;
        const int Gc = min(G, row_end - i0);
        const int T = nq * Gc;
        ok = mbar_wait_warp(bar(C::B_KVFULL), n & 1, w, 0x36);
        for (int t = 0; t < T && ok; ++t, ++tt) {
          const int g = t % Gc;
          ok = mbar_wait_warp(bar(C::B_P2FULL), tt & 1, w, 0x37);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t dSm = umma_smem_desc(sDS_a, 16384, 1024, kSwz128);
          const uint64_t dKm = umma_smem_desc(sKV_a + g * 2 * C::TILE_B, C::SBO, C::SBO, C::SWZ);
          if (elect_one()) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              umma_ss(tbase + C::TM_DQ + (tt & 1) * kD, dSm + ks * (2048 >> 4), dKm + ks * ((2 * C::SBO) >> 4),
                      idesc_dq, ks > 0);
            umma_commit(bar(C::B_DQDONE));
          }
          __syncwarp();
        }
        if (ok) {
          if (elect_one()) umma_commit(bar(C::B_KVFREE));  // K of this group is no longer read by dQ MMAs
          __syncwarp();
        }
      }
    } else {
      // ---------------------------------------------------------------- store warp
      // Everything that leaves the CTA as a float32 sum goes through shared memory and one TMA
      // tile reduction issued by one thread (whole 128-byte lines, no work for the compute warps):
      //  * each finished dQ tile, staged by the compute warps (D = 32);
      //  * at the end of each query block, the dBias sums of the four warpgroups: 16 KB boxes
      //    (128 keys x 32 queries) written into the bias stage that has just been used up - the two
      //    warpgroups of a query half take turns in that half's 16 KB - and added to (first group:
      //    stored into) this CTA's private key-major plane.
      // The planes (a few tens of MB, added to once per group) must stay in L2 between groups: with
      // default priority the dQ stream evicts them and every addition becomes a DRAM read + write.
      const uint64_t pol_keep = l2_policy_evict_last();
      bool ok = true;
      int k = 0, nb = 0;  // dQ tiles / query blocks so far
      auto dq_event = [&](int irow, int jblk) -> bool {
        if (!mbar_wait_warp(bar(C::B_DQSFULL), k & 1, w, 0x51)) return false;
        if (elect_one()) {
          tma_reduce_add_3d(&tmDQ, smem_u32(sDQ), 0, jblk * 128, bh * p.L1 + irow);
          bulk_commit_group();
          bulk_wait_read_all();  // the staging tile has been read: the compute warps may refill it
          mbar_arrive(bar(C::B_DQSFREE));
        }
        __syncwarp();
        ++k;
        return true;
      };
      for (int n = 0; n < ngroups && ok; ++n) {
        const int i0 = row_begin + n * G;
        const int Gc = min(G, row_end - i0);
        const int pkey = kb * 128, pidx = r * p.BH + bh;  // first key row of this CTA's tile, its plane
        for (int jb = 0; jb < nq && ok; ++jb, ++nb) {
          if constexpr (C::DQ_TMA) {
            for (int g = 0; g < Gc && ok; ++g) {
              if (jb == 0 && g == 0) continue;
              const int pt = jb * Gc + g - 1;
              ok = dq_event(i0 + pt % Gc, pt / Gc);
            }
            if (!ok) break;
          }
          const int bs = nb & 1;
          // second warpgroup of each half: boxes parked in the dS tile (needed again soonest)
          ok = mbar_wait_warp(bar(C::B_FLB + 0), nb & 1, w, 0x52) && mbar_wait_warp(bar(C::B_FLB + 1), nb & 1, w, 0x53);
          if (!ok) break;
          if (elect_one()) {
            for (int hh = 0; hh < 2; ++hh) {
              const uint32_t src = smem_u32(sDS + hh * 16384);
              const int qcol = jb * 128 + (2 * hh + 1) * 32;
              if (n == 0) tma_store_3d_hint(&tmPlane, src, qcol, pkey, pidx, pol_keep);
              else tma_reduce_add_3d_hint(&tmPlane, src, qcol, pkey, pidx, pol_keep);
            }
            bulk_commit_group();
          }
          __syncwarp();
          // first warpgroup of each half: boxes parked in the bias stage
          ok = mbar_wait_warp(bar(C::B_FLA + 0), nb & 1, w, 0x54) && mbar_wait_warp(bar(C::B_FLA + 1), nb & 1, w, 0x55);
          if (!ok) break;
          if (elect_one()) {
            for (int hh = 0; hh < 2; ++hh) {
              const uint32_t src = smem_u32(sBias + bs * C::BIAS_B + hh * 16384);
              const int qcol = jb * 128 + (2 * hh) * 32;
              if (n == 0) tma_store_3d_hint(&tmPlane, src, qcol, pkey, pidx, pol_keep);
              else tma_reduce_add_3d_hint(&tmPlane, src, qcol, pkey, pidx, pol_keep);
            }
            bulk_commit_group();
            bulk_wait_read_le1();  // the older group (dS tile) has been read
            mbar_arrive(bar(C::B_DSFREE));
            bulk_wait_read_all();
            mbar_arrive(bar(C::B_BIASEMPTY + bs));  // the bias stage goes back to the producer
          }
          __syncwarp();
        }
        if (!ok) break;
        if constexpr (C::DQ_TMA) {
          const int pt = nq * Gc - 1;
          ok = dq_event(i0 + pt % Gc, pt / Gc);
        }
        // the next group adds to the plane elements this group wrote: finish these writes first
        if (elect_one()) bulk_wait_all();
        __syncwarp();
      }
      if (elect_one()) bulk_wait_all();
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ compute warpgroups
    // 16 warps = 4 warpgroups; warpgroup qd owns the 32-query quarter qd of the tile (half
    // wh = qd / 2, chunk sub = qd % 2 of that half). Four compute warps per scheduler hide the
    // ALU / MUFU / shared-memory latencies that two could not.
    reg_inc<kComputeRegs>();
    const int qd = (warp >> 2) - 1;
    const int wh = qd >> 1, sub = qd & 1;
    const int key = (warp & 3) * 32 + lane;  // key row of the block == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    // this quarter's 32 fp32 columns of S^T / dP^T; P^T / dS^T overwrite its first 16 columns
    const uint32_t tST = tbase + C::TM_ST + wh * 64 + sub * 32 + lane_off;
    const uint32_t tDP = tbase + C::TM_DP + wh * 64 + sub * 32 + lane_off;
    const f32x2 scale2 = mk2(p.scale, p.scale);
    const f32x2 log2e2 = mk2(kLog2e, kLog2e);
    const f32x2 k1_2 = mk2(p.scale * kLog2e, p.scale * kLog2e);
    const f32x2 neg1_2 = mk2(-1.f, -1.f);
    bool ok = true;
    int tt = 0, nb = 0;
    // reduce this warpgroup's quarter of the columns of one finished dQ tile (TMEM buffer `buf`)
    // into the float32 dQ accumulator; the four warpgroups share the work evenly
    int kdq = 0;  // dQ tiles handed to the store warp so far
    int ring_slot = 0;
    uint32_t ring_phase = 0;
    // `publish`: fence and tell the store warp here; otherwise the caller does both (it shares
    // the fence with its own shared-memory writes)
    auto reduce_dq = [&](int buf, int irow, int jblk, bool publish) -> bool {
      constexpr int W = kD / 4;  // columns per warpgroup
      if constexpr (C::DQ_TMA) {
        // this warpgroup's 8 columns (two 16-byte chunks) of each row of the staging tile, in the
        // 128-byte swizzle the tensor map expects; the tile is free once the store warp says that
        // the previous reduction has read it
        uint32_t qv[8];
        tmem_ld8(tbase + C::TM_DQ + buf * kD + qd * W + lane_off, qv);
        const bool free_ok = kdq == 0 || mbar_wait_warp(bar(C::B_DQSFREE), (kdq - 1) & 1, w, 0x48);
        tmem_ld_wait();
        if (!free_ok) return false;
        const uint32_t rowa = smem_u32(sDQ) + key * 128;
        st_shared_v4(rowa + (((2 * qd) ^ (key & 7)) << 4), qv[0], qv[1], qv[2], qv[3]);
        st_shared_v4(rowa + (((2 * qd + 1) ^ (key & 7)) << 4), qv[4], qv[5], qv[6], qv[7]);
        ++kdq;
        if (publish) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(C::B_DQSFULL));
        }
        return true;
      }
      float* dst = p.dq32 + ((static_cast<long long>(bh) * p.L1 + irow) * p.L2 + jblk * 128 + key) * kD + qd * W;
      const bool q_live = jblk * 128 + key < p.L2;  // here `key` is the TMEM lane = query row of the dQ tile
#pragma unroll
      for (int c = 0; c < W / 8; ++c) {
        uint32_t qv[8];
        tmem_ld8(tbase + C::TM_DQ + buf * kD + qd * W + c * 8 + lane_off, qv);
        tmem_ld_wait();
        if (!q_live) continue;
        red_add_v4(dst + c * 8, __uint_as_float(qv[0]), __uint_as_float(qv[1]), __uint_as_float(qv[2]),
                   __uint_as_float(qv[3]));
        red_add_v4(dst + c * 8 + 4, __uint_as_float(qv[4]), __uint_as_float(qv[5]), __uint_as_float(qv[6]),
                   __uint_as_float(qv[7]));
      }
      return true;
    };
    for (int n = 0; n < ngroups && ok; ++n) {
      const int i0 = row_begin + n * G;
      const int Gc = min(G, row_end - i0);
      for (int jb = 0; jb < nq && ok; ++jb, ++nb) {
        f32x2 acc[16];  // dBias sums: this key column x 32 query rows
#pragma unroll
        for (int c = 0; c < 16; ++c) acc[c] = mk2(0.f, 0.f);
        const int bs = nb & 1;
        ok = mbar_wait_warp(bar(C::B_BIASFULL + bs), (nb >> 1) & 1, w, 0x41);
        if (!ok) break;
        const uint8_t* brow = sBias + bs * C::BIAS_B + wh * 16384 + key * 128;
        for (int g = 0; g < Gc; ++g, ++tt) {
          // Q/dO ring slot and phase of tile tt (tt % NQ, (tt / NQ) & 1) kept as running counters
          const int s = ring_slot;
          const uint32_t ring_par = ring_phase;
          if (++ring_slot == C::NQ) {
            ring_slot = 0;
            ring_phase ^= 1u;
          }
          const uint8_t* st = sQDO + s * C::STAGE_B;
          ok = mbar_wait_warp(bar(C::B_SFULL), tt & 1, w, 0x42);
          if (!ok) break;
          ok = mbar_wait_warp(bar(C::B_QDOFULL + s), ring_par, w, 0x43);  // statistics visible
          if (!ok) break;
          tc_fence_after_sync();
          const float4* nm4 = reinterpret_cast<const float4*>(st + 2 * C::TILE_B) + qd * 8;
          const float4* nl4 = reinterpret_cast<const float4*>(st + 2 * C::TILE_B + 512) + qd * 8;
          const float4* del4 = reinterpret_cast<const float4*>(st + 2 * C::TILE_B + 1024) + qd * 8;
          // ---- phase 1: P^T = exp2((S^T*scale + bias^T - max)*log2e - log2 sum), handed to the dV MMA
          // in the input dtype (pp). Phase 2 forms dS from a half-precision (fp16) copy of P (ph):
          // with bf16 inputs the 8-bit mantissa of the MMA operand would put a rounding error of
          // up to 2^-9 * |dP - delta| into every term of the dBias sums over L1 (0.04 max-abs at
          // 768 rows of N(0,1) inputs, twice the tolerance); fp16 keeps 11 bits for 16 conversions
          // per thread and tile.
          uint32_t ph[16], pp[8];  // pp: one half of the quarter at a time (two 8-column stores)
          const float4* c4 = reinterpret_cast<const float4*>(st + 2 * C::TILE_B + 1536) + qd * 8;
          // one lane per query of the quarter looks at c: NaN = a row that needs the two-part form
          const float cq = reinterpret_cast<const float*>(st + 2 * C::TILE_B + 1536)[qd * 32 + lane];
          const bool robust = __any_sync(0xffffffffu, cq != cq);
          if (!robust) {
            // y = s*scale*log2e + b*log2e + c
            // The 32 columns come in four loads of 8, each issued before the arithmetic on the
            // previous one and waited for after it, so only the first TMEM round trip is exposed.
            uint32_t sv[2][8];
            constexpr int NCH = 4;
            tmem_ld8(tST, sv[0]);
            tmem_ld_wait();
#pragma unroll
            for (int ch = 0; ch < NCH; ++ch) {  // 8-query chunk within the quarter
              if (ch + 1 < NCH) tmem_ld8(tST + (ch + 1) * 8, sv[(ch + 1) & 1]);
              const uint4 bv = *reinterpret_cast<const uint4*>(brow + (((sub * 4 + ch) ^ (key & 7)) << 4));
              const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
              const float4 ca = c4[ch * 2], cb = c4[ch * 2 + 1];
              const f32x2 c2[4] = {mk2(ca.x, ca.y), mk2(ca.z, ca.w), mk2(cb.x, cb.y), mk2(cb.z, cb.w)};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float b0, b1, y0, y1;
                unpack2<kBf16>(bw[e], b0, b1);
                un2(fma2(mk2(__uint_as_float(sv[ch & 1][2 * e]), __uint_as_float(sv[ch & 1][2 * e + 1])), k1_2,
                         fma2(mk2(b0, b1), log2e2, c2[e])),
                    y0, y1);
                const float p0 = fast_exp2(y0), p1 = fast_exp2(y1);
                pp[(ch & 1) * 4 + e] = pack2<kBf16>(p0, p1);
                ph[ch * 4 + e] = kBf16 ? pack_f16x2(p0, p1) : pp[(ch & 1) * 4 + e];
              }
              if (ch + 1 < NCH) tmem_ld_wait();
              // the 16 columns of queries 0-15 (16-31) have been read: P^T of those queries goes over
              // the first (second) 8 of them
              if (ch & 1) tmem_st8(tST + (ch >> 1) * 8, pp);
            }
          } else {
#pragma unroll
          for (int c16 = 0; c16 < 2; ++c16) {
            uint32_t sv[16];
            tmem_ld16(tST + c16 * 16, sv);
            tmem_ld_wait();
#pragma unroll
            for (int c8 = 0; c8 < 2; ++c8) {
              const int ch = c16 * 2 + c8;  // 8-query chunk within the quarter
              const uint4 bv = *reinterpret_cast<const uint4*>(brow + (((sub * 4 + ch) ^ (key & 7)) << 4));
              const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
              const float4 ma = nm4[ch * 2], mb = nm4[ch * 2 + 1];
              const float4 la = nl4[ch * 2], lb = nl4[ch * 2 + 1];
              const f32x2 nm2[4] = {mk2(ma.x, ma.y), mk2(ma.z, ma.w), mk2(mb.x, mb.y), mk2(mb.z, mb.w)};
              const f32x2 nl2[4] = {mk2(la.x, la.y), mk2(la.z, la.w), mk2(lb.x, lb.y), mk2(lb.z, lb.w)};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int idx = c8 * 8 + 2 * e;  // column within the 16-column load
                float b0, b1, y0, y1;
                unpack2<kBf16>(bw[e], b0, b1);
                // x = s*scale + b exactly as the forward pass formed it; (x - max) is then exact
                // for x near the max whatever its magnitude; y = (x - max)*log2e - log2(sum)
                const f32x2 x = fma2(mk2(__uint_as_float(sv[idx]), __uint_as_float(sv[idx + 1])), scale2,
                                     mk2(b0, b1));
                un2(fma2(add2(x, nm2[e]), log2e2, nl2[e]), y0, y1);
                const float p0 = fast_exp2(y0), p1 = fast_exp2(y1);
                pp[c8 * 4 + e] = pack2<kBf16>(p0, p1);
                ph[ch * 4 + e] = kBf16 ? pack_f16x2(p0, p1) : pp[c8 * 4 + e];
              }
            }
            tmem_st8(tST + c16 * 8, pp);
          }
          }
          tmem_st_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(C::B_P1FULL));
          // ---- phase 2: dS^T = P^T * (dP^T - delta), summed into the dBias registers
          ok = mbar_wait_warp(bar(C::B_DPFULL), tt & 1, w, 0x47);
          if (!ok) break;
          tc_fence_after_sync();
          uint32_t dd[16];  // dS^T of this key row, 32 queries, packed 16-bit pairs
          {
            uint32_t dv[2][8];  // four loads of 8 columns, pipelined like phase 1
            constexpr int NCH = 4;
            tmem_ld8(tDP, dv[0]);
            tmem_ld_wait();
#pragma unroll
            for (int ch = 0; ch < NCH; ++ch) {
              if (ch + 1 < NCH) tmem_ld8(tDP + (ch + 1) * 8, dv[(ch + 1) & 1]);
              const float4 da = del4[ch * 2], db = del4[ch * 2 + 1];
              const f32x2 del2[4] = {mk2(da.x, da.y), mk2(da.z, da.w), mk2(db.x, db.y), mk2(db.z, db.w)};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float p0, p1, ds0, ds1;
                unpack2<false>(ph[ch * 4 + e], p0, p1);
                const f32x2 u = fma2(del2[e], neg1_2,
                                     mk2(__uint_as_float(dv[ch & 1][2 * e]), __uint_as_float(dv[ch & 1][2 * e + 1])));
                const f32x2 ds = mul2(mk2(p0, p1), u);
                acc[ch * 4 + e] = add2(acc[ch * 4 + e], ds);
                un2(ds, ds0, ds1);
                dd[ch * 4 + e] = pack2<kBf16>(ds0, ds1);
              }
              if (ch + 1 < NCH) tmem_ld_wait();
            }
          }
          tmem_st16(tDP, dd);
          if (tt > 0) {  // dS staging tile free again: the previous dQ MMA has read it
            ok = mbar_wait_warp(bar(C::B_DQDONE), (tt - 1) & 1, w, 0x44);
            if (!ok) break;
          }
          if (g == 0 && nb > 0) {  // the dBias boxes parked in the dS tile have been read
            ok = mbar_wait_warp(bar(C::B_DSFREE), (nb - 1) & 1, w, 0x4b);
            if (!ok) break;
          }
          // dQ of the previous tile of this group is complete (DQDONE waited above): stage it now,
          // so that one proxy fence covers it and the dS rows below
          const bool stage_dq = C::DQ_TMA && !(jb == 0 && g == 0);
          if (stage_dq) {
            const int pt = jb * Gc + g - 1;
            tc_fence_after_sync();
            ok = reduce_dq((tt - 1) & 1, i0 + pt % Gc, pt / Gc, false);
            if (!ok) break;
          }
          // dS^T row of this key into the M-major staging tile (128-byte swizzle)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 v4 = make_uint4(dd[4 * j], dd[4 * j + 1], dd[4 * j + 2], dd[4 * j + 3]);
            *reinterpret_cast<uint4*>(sDS + wh * 16384 + key * 128 + (((sub * 4 + j) ^ (key & 7)) << 4)) = v4;
          }
          tmem_st_wait();
          fence_proxy_async_smem();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(bar(C::B_P2FULL));
            if (stage_dq) mbar_arrive(bar(C::B_DQSFULL));
          }
          if (!C::DQ_TMA && !(jb == 0 && g == 0)) {
            // dQ of the previous tile of this group is complete (DQDONE waited above)
            const int pt = jb * Gc + g - 1;
            tc_fence_after_sync();
            ok = reduce_dq((tt - 1) & 1, i0 + pt % Gc, pt / Gc, true);
            if (!ok) break;
          }
        }
        if (!ok) break;
        if (jb == nq - 1) {
          // ---- group epilogue, before the dBias boxes so that the dK / dV stores are not queued
          // behind their reductions: last dQ tile, then dK / dV of the G rows
          ok = mbar_wait_warp(bar(C::B_ACCFULL), n & 1, w, 0x45);
          if (!ok) break;
          tc_fence_after_sync();
          {
            ok = mbar_wait_warp(bar(C::B_DQDONE), (tt - 1) & 1, w, 0x46);  // last dQ of the group
            if (!ok) break;
            tc_fence_after_sync();
            const int pt = nq * Gc - 1;
            ok = reduce_dq((tt - 1) & 1, i0 + pt % Gc, pt / Gc, true);
            if (!ok) break;
          }
          {
            // half 0 stores dV, half 1 stores dK (scaled by sm_scale, flash_tt_attn.py:518); the two
            // warpgroups of a half take alternate rows of the group
            const long long* sd = (wh == 0) ? p.sdv : p.sdk;
            uint16_t* base = reinterpret_cast<uint16_t*>(wh == 0 ? p.dv : p.dk) + b * sd[0] + h * sd[1] +
                             static_cast<long long>(kb * 128 + key) * sd[3];
            const float mul = (wh == 0) ? 1.0f : p.scale;
            const bool key_live = kb * 128 + key < p.L2;  // keys past L2 in a ragged block own no output row
            for (int g = sub; g < Gc; g += 2) {
              uint16_t* optr = base + static_cast<long long>(i0 + g) * sd[2];
              const uint32_t ta = tbase + C::TM_ACC + g * 2 * kD + (wh == 0 ? kD : 0) + lane_off;
    #pragma unroll
              for (int c = 0; c < kD / 32; ++c) {
                uint32_t av[32];
                tmem_ld32(ta + c * 32, av);
                tmem_ld_wait();
    #pragma unroll
                for (int v4 = 0; v4 < 4; ++v4) {
                  uint4 ov;
                  ov.x = pack2<kBf16>(__uint_as_float(av[v4 * 8 + 0]) * mul, __uint_as_float(av[v4 * 8 + 1]) * mul);
                  ov.y = pack2<kBf16>(__uint_as_float(av[v4 * 8 + 2]) * mul, __uint_as_float(av[v4 * 8 + 3]) * mul);
                  ov.z = pack2<kBf16>(__uint_as_float(av[v4 * 8 + 4]) * mul, __uint_as_float(av[v4 * 8 + 5]) * mul);
                  ov.w = pack2<kBf16>(__uint_as_float(av[v4 * 8 + 6]) * mul, __uint_as_float(av[v4 * 8 + 7]) * mul);
                  if (key_live) *reinterpret_cast<uint4*>(optr + c * 32 + v4 * 8) = ov;
                }
              }
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(C::B_ACCFREE));
        }
        if (!ok) break;
        // ---- dBias of this query block: the sums go to the store warp as 16 KB boxes parked in
        // shared memory that is idle at this point. The first warpgroup of a half uses that half's
        // part of the bias stage just used up (free once both warpgroups of the half have read
        // their bias values; waiting for their phase-2 arrival rather than the earlier phase-1 one
        // also keeps the two warpgroups of the half in step, which measures faster), the second
        // one that half's part of the dS tile (free once the last dQ MMA has read it).
        if (sub == 0) ok = mbar_wait_warp(bar(C::B_P2FULL), (tt - 1) & 1, w, 0x49);
        else ok = mbar_wait_warp(bar(C::B_DQDONE), (tt - 1) & 1, w, 0x4a);
        if (!ok) break;
        {
          // box: 128 key rows x 32 queries (128 bytes), 128-byte swizzle
          const uint32_t rowa = smem_u32(sub == 0 ? sBias + bs * C::BIAS_B + wh * 16384 : sDS + wh * 16384) + key * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float a0, a1, a2, a3;
            un2(acc[2 * j], a0, a1);
            un2(acc[2 * j + 1], a2, a3);
            st_shared_v4(rowa + ((j ^ (key & 7)) << 4), __float_as_uint(a0), __float_as_uint(a1),
                         __float_as_uint(a2), __float_as_uint(a3));
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar((sub == 0 ? C::B_FLA : C::B_FLB) + wh));
        }
      }
      if (!ok) break;
    }
  }

  // ---------------------------------------------------------------------- tear-down
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) __nanosleep(20000);
  if (warp == 0) tmem_dealloc(tbase, 512);
}

template <int kD, bool kBf16>
int launch_bwd_t(const BwdArgs& a, int NP, cudaStream_t stream) {
  using C = BwdCfg<kD>;
  static PerDeviceOnce smem_attr;
  auto kern = fta_bwd_kernel<kD, kBf16>;
  if (cudaError_t e = ensure_dynamic_smem(smem_attr, kern, C::SMEM_BYTES)) return static_cast<int>(e);
  BwdParams p;
  p.lse = a.lse;
  p.delta = a.delta;
  p.dq32 = a.dq32;
  p.dk = a.dk;
  p.dv = a.dv;
  p.status = a.status;
  p.H = a.H;
  p.L1 = a.L1;
  p.L2 = a.L2;
  p.NP = NP;
  p.BH = a.B * a.H;
  for (int i = 0; i < 4; ++i) {
    p.sdk[i] = a.sdk[i];
    p.sdv[i] = a.sdv[i];
  }
  p.scale = a.sm_scale;
  p.stat_pitch = (a.L2 + 127) / 128 * 128;
  p.stat_stride = static_cast<long long>(a.B) * a.H * a.L1 * p.stat_pitch;
  const int grid = a.B * a.H * NP * ((a.L2 + 127) / 128);
  kern<<<grid, kBwdThreads, C::SMEM_BYTES, stream>>>(a.tmQ, a.tmK, a.tmV, a.tmDO, a.tmBiasT, a.tmDQ, a.tmPlane, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

int bwd_rows_per_cta(int D) { return D == 32 ? BwdCfg<32>::G : BwdCfg<64>::G; }

// Number of private dBias planes == number of row blocks per (b,h,key block). Chosen so that the
// grid (B*H * L2/128 * NP CTAs, one per SM at a time) fills whole waves of the device with
// chains of nearly equal length, with as few planes as that allows.
int bwd_num_planes(int B, int H, int L1, int L2, int D, int num_sms) {
  const int G = bwd_rows_per_cta(D);
  const int ngroups = (L1 + G - 1) / G;
  const long long base = static_cast<long long>(B) * H * ((L2 + 127) / 128);
  const int np_max = ngroups < 64 ? ngroups : 64;
  auto efficiency = [&](int np) {
    const long long ctas = base * np;
    const long long waves = (ctas + num_sms - 1) / num_sms;
    const int chain = (L1 + np - 1) / np;  // rows of the longest chain
    // time ~ waves * chain ; work ~ base * L1 / num_sms
    return (static_cast<double>(base) * L1 / num_sms) / (static_cast<double>(waves) * chain);
  };
  // The planes are updated in place all through the kernel, so their footprint should stay inside
  // the L2 cache. While it does (half of the 126 MB), take the best schedule, and the fewest planes
  // among schedules within 1 % of it; beyond that, the FEWEST planes whose schedule is within 7 % of
  // the best one.
  const long long l2p = (L2 + 127) / 128 * 128;
  const double plane_set_bytes = 4.0 * B * H * static_cast<double>(l2p) * l2p;
  const double budget = 64.0 * 1024 * 1024;
  double best_small = -1.0, best_eff = -1.0;
  for (int np = 1; np <= np_max; ++np) {
    const double e = efficiency(np);
    best_eff = e > best_eff ? e : best_eff;
    if (np * plane_set_bytes <= budget) best_small = e > best_small ? e : best_small;
  }
  if (best_small >= 0.93 * best_eff) {
    for (int np = 1; np <= np_max; ++np)
      if (np * plane_set_bytes <= budget && efficiency(np) >= 0.99 * best_small) return np;
  }
  for (int np = 1; np <= np_max; ++np)
    if (efficiency(np) >= 0.93 * best_eff) return np;
  return 1;
}

int launch_bwd(const BwdArgs& a, cudaStream_t stream) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int NP = bwd_num_planes(a.B, a.H, a.L1, a.L2, a.D, sms);
  if (a.D == 32) return a.bf16 ? launch_bwd_t<32, true>(a, NP, stream) : launch_bwd_t<32, false>(a, NP, stream);
  return a.bf16 ? launch_bwd_t<64, true>(a, NP, stream) : launch_bwd_t<64, false>(a, NP, stream);
}

}  // namespace fta
