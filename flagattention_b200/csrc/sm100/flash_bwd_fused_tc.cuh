// flash_attention backward on tcgen05 in ONE pass over the score tiles (head_dim 64 and 128):
// dK, dV and dQ come out of the same kernel, so S and dP are computed once (five GEMMs per
// 128 x 128 tile) instead of once in a dK/dV kernel and again in a dQ kernel (seven).
//
// One CTA per 128 keys walks the query tiles (and the query heads of its GQA group).  dK and dV
// accumulate in TMEM for the whole walk.  The dQ contribution of a tile, dS K, is a complete
// 128 x D product of its own: it is accumulated in TMEM for the tile, read back by four
// reduction warps and added into an fp32 workspace in global memory with vector reductions
// (`cp.reduce.async.bulk`); a small kernel scales and converts the workspace afterwards.  The
// order of those additions is not fixed, so dQ is reproducible only to fp32 rounding.
//
//   warp 0       TMA producer
//   warp 1       MMA issuer (one thread); every MMA is 128 x 128 x 16 (128 x 64 x 16 at D = 64)
//   warps 2..17  element-wise stage, one thread per (accumulator row, 32 columns)
//   warps 18..21 dQ reduction: TMEM -> shared-memory staging -> cp.reduce.async.bulk
//   warp 22      stages lse / delta of every tile in shared memory
//
// TMEM (512 columns):  S^T, then dP^T | dQ | dK | dV.
//   The two score products of a tile share one 128-column region: dP^T is issued as soon as the
//   element-wise warps hold S^T in registers, S^T of the next tile as soon as they hold dP^T.
//   dQ has columns of its own, so its slow read-out never holds a GEMM back.
// Shared memory:       K, V resident | Q ring | dO ring | one 16-bit 128 x 128 tile "PD" | dQ staging.
//   PD holds P^T (A operand of dV += P^T dO), then dS^T of the same tile: the K-major A operand of
//   dK += dS^T Q and, under a second descriptor, the MN-major A operand of dQ = dS K.
//
// Issue order of a tile (tensor pipe, in order):   dP^T(t) | dV(t) | S^T(t+1) | dQ(t) | dK(t)
// Element-wise order:                              phase 1 (t) | phase 2 (t)
//   phase 1: P^T = exp2(S^T * scale - L) -> PD       phase 2: dS^T = P^T * (dP^T - delta) -> PD
#pragma once

#include "flash_bwd_tc.cuh"

namespace fa {
namespace tc {

template <int D>
struct FusedBwdCfg {
  static constexpr int BM = 128, BN = 128, NQ = 2, NDO = (D == 128 ? 1 : 2);
  static constexpr int KSUB = D / 64;
  static constexpr int kTile = 128 * D * 2;            // any 128-row operand tile
  static constexpr int kK = 0;
  static constexpr int kV = kTile;
  static constexpr int kQ0 = 2 * kTile;                // Q ring
  static constexpr int kDO0 = kQ0 + NQ * kTile;        // dO ring
  static constexpr int kPD = kDO0 + NDO * kTile;       // P^T / dS^T: 128 key rows x 128 queries x 2 B
  static constexpr int kPdBytes = 128 * 128 * 2;
  // dQ staging: two buffers of a quarter of a dQ tile, fp32, as D/16 runs of (128 queries x 4)
  static constexpr int kQuarter = (D / 16) * 2048;
  static constexpr int kStage = kPD + kPdBytes;
  static constexpr int kBars = kStage + 2 * kQuarter;
  static constexpr int kMisc = kBars + 24 * 8;
  static constexpr int kStats = kMisc + 16;            // -lse*log2e [128] | -delta [128] of a tile
  static constexpr int kTotal = kStats + 2 * 128 * 4 + 1024;
  static constexpr int kTmemCols = 512;
  static constexpr int kColA = 0, kColQ = 128, kColDK = 256, kColDV = 256 + D;
  static_assert(kTotal <= 232448, "shared memory budget");
};

enum FusedBar { FB_KV_FULL = 0, FB_Q_FULL = 1, FB_Q_FREE = 3, FB_DO_FULL = 5, FB_DO_FREE = 7,
                FB_S_FULL = 9, FB_S_LOADED = 10, FB_DP_FULL = 11, FB_DP_LOADED = 12,
                FB_PT_FULL = 13, FB_PT_FREE = 14, FB_DS_FULL = 15, FB_DS_FREE = 16,
                FB_DQ_FULL = 17, FB_DQ_FREE = 18, FB_DONE = 19, FB_LSE_FULL = 20, FB_DLT_FULL = 21, FB_V_FULL = 22 };

struct FusedBwdParams {
  BwdTcParams base;
  float *dq_acc;   // (B, H, Mpad / 128, D / 4, 128, 4) fp32, zeroed before the launch
  int Mpad;        // M rounded up to a multiple of 128
};

// fp32 add of `bytes` contiguous bytes of shared memory into global memory, done by the copy
// engine: it does not pass through the load/store queue of the SM and nobody waits for it.
__device__ __forceinline__ void bulk_reduce_add_f32(float *dst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;\n" ::"l"(dst),
               "r"(smem_src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
}
// waits until all but the newest group have finished READING their shared-memory source
__device__ __forceinline__ void bulk_wait_read_1() {
  asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory");
}
// waits until every group has finished reading its shared-memory source (what a CTA owes before
// it gives its shared memory back; the additions themselves complete by the end of the grid)
__device__ __forceinline__ void bulk_wait_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
}
// barrier among the four reduction warps (barrier 0 belongs to __syncthreads)
__device__ __forceinline__ void red_warps_sync() {
  asm volatile("bar.sync 1, 128;\n" ::: "memory");
}
// the same barrier with a vote: true iff `ok` holds in all 128 threads
__device__ __forceinline__ bool red_warps_all(bool ok) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "bar.red.and.pred q, 1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}\n"
      : "=r"(out)
      : "r"((uint32_t)ok)
      : "memory");
  return out != 0;
}

// barrier 2 with a vote: the 16 element-wise warps (512 threads)
__device__ __forceinline__ bool ew_warps_all(bool ok) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "bar.red.and.pred q, 2, 512, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}\n"
      : "=r"(out)
      : "r"((uint32_t)ok)
      : "memory");
  return out != 0;
}

// one box of a (d, l, h, b) tensor map, shared memory -> global memory; rows past the tensor's
// end are dropped by the copy engine
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, uint32_t smem_src, int c0, int c1,
                                             int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];\n"
      :
      : "l"(map), "r"(smem_src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// warps: 0 TMA producer, 1 MMA issuer, 2..17 element-wise, 18..21 dQ reduction (one per TMEM
// lane slice), 22 statistics
constexpr int kFusedThreads = kBwdThreads + 5 * 32;   // 736

template <typename T, int D>
__global__ void __launch_bounds__(kFusedThreads, 1)
    flash_bwd_fused_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                              const __grid_constant__ CUtensorMap map_do,
                              const __grid_constant__ CUtensorMap map_k,
                              const __grid_constant__ CUtensorMap map_v,
                              const __grid_constant__ CUtensorMap map_dk,
                              const __grid_constant__ CUtensorMap map_dv, const FusedBwdParams fp) {
  using C = FusedBwdCfg<D>;
  constexpr int BM = C::BM, BN = C::BN, KSUB = C::KSUB, NQ = C::NQ, NDO = C::NDO;
  const BwdTcParams &p = fp.base;
  extern __shared__ uint8_t smem_unaligned[];
  const uint32_t smem = (smem_u32(smem_unaligned) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_unaligned + (smem - smem_u32(smem_unaligned));
  auto bar = [&](int i) { return smem + C::kBars + i * 8; };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + C::kMisc);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + C::kMisc + 8);
  const AbortCtx actx{abort_flag, p.status};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const CtaCoord cta = grouped_cta(blockIdx.x, p.num_blocks, p.B * p.Hk, p.group_size);
  const int nb = cta.blk, hk = cta.pair % p.Hk, b = cta.pair / p.Hk;
  const int G = p.H / p.Hk;
  const int n0 = nb * BN;
  const int p_seq = p.N - p.M;
  const int num_m_tiles = (p.M + BM - 1) / BM;
  int mt_lo = 0;
  if (p.causal) mt_lo = max(0, n0 - p_seq) / BM;
  int mt_hi = num_m_tiles;
  if (p.mode == 1) {  // query tiles that hold a near pair
    const int lim = p.w - p_seq + n0 + BN - 1;
    mt_hi = min(mt_hi, lim <= 0 ? 0 : (lim + BM - 1) / BM);
  } else if (p.mode == 2) {  // query tiles that hold a far pair
    const int lim = p.w - p_seq + n0 - (BM - 1);
    mt_lo = max(mt_lo, lim <= 0 ? 0 : (lim + BM - 1) / BM);
  }
  const int tiles = max(0, mt_hi - mt_lo);
  const int T_tiles = tiles * G;

  if (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) return;

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar(FB_KV_FULL), 1);   // K
    mbar_init(bar(FB_V_FULL), 1);
    for (int s = 0; s < NQ; ++s) {
      mbar_init(bar(FB_Q_FULL + s), 1);
      mbar_init(bar(FB_Q_FREE + s), 1);
    }
    for (int s = 0; s < NDO; ++s) {
      mbar_init(bar(FB_DO_FULL + s), 1);
      mbar_init(bar(FB_DO_FREE + s), 1);
    }
    mbar_init(bar(FB_S_FULL), 1);
    mbar_init(bar(FB_S_LOADED), kEwWarps);
    mbar_init(bar(FB_DP_FULL), 1);
    mbar_init(bar(FB_DP_LOADED), kEwWarps);
    mbar_init(bar(FB_PT_FULL), kEwWarps);
    mbar_init(bar(FB_PT_FREE), 1);
    mbar_init(bar(FB_DS_FULL), kEwWarps);
    mbar_init(bar(FB_DS_FREE), 1);
    mbar_init(bar(FB_DQ_FULL), 1);
    mbar_init(bar(FB_DQ_FREE), 4);
    mbar_init(bar(FB_DONE), 1);
    mbar_init(bar(FB_LSE_FULL), 1);
    mbar_init(bar(FB_DLT_FULL), 1);
    fence_barrier_init();
    // The loads of the first tile go out right here, before the TMEM allocation and the CTA-wide
    // barrier below, so that their latency (the first bytes of K, V, Q, dO come from HBM) runs
    // under the rest of the set-up.  K and Q first: S^T of the first tile needs only those.
    if (T_tiles > 0) {
      const int h0 = hk * G, m00 = mt_lo * BM;
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_v);
      tma_prefetch_desc(&map_do);
      tma_prefetch_desc(&map_dk);
      tma_prefetch_desc(&map_dv);
      mbar_expect_tx(bar(FB_KV_FULL), C::kTile);
      for (int s = 0; s < KSUB; ++s)
        tma_load_4d(smem + C::kK + s * BN * 128, &map_k, bar(FB_KV_FULL), s * 64, n0, hk, b);
      mbar_expect_tx(bar(FB_Q_FULL), C::kTile);
      for (int s = 0; s < KSUB; ++s)
        tma_load_4d(smem + C::kQ0 + s * BM * 128, &map_q, bar(FB_Q_FULL), s * 64, m00, h0, b);
      mbar_expect_tx(bar(FB_V_FULL), C::kTile);
      for (int s = 0; s < KSUB; ++s)
        tma_load_4d(smem + C::kV + s * BN * 128, &map_v, bar(FB_V_FULL), s * 64, n0, hk, b);
      mbar_expect_tx(bar(FB_DO_FULL), C::kTile);
      for (int s = 0; s < KSUB; ++s)
        tma_load_4d(smem + C::kDO0 + s * BM * 128, &map_do, bar(FB_DO_FULL), s * 64, m00, h0, b);
    }
  }
  if (warp == 0) {
    tmem_alloc(smem + C::kMisc, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ producer -----------------------------------
    if (lane == 0 && T_tiles > 0) {
      // (tile 0 was requested during set-up)
      int issued_q = 1, issued_do = 1;
      bool ok = true;
      int sq = 0, phq = 1, sd = 0, phd = 1;   // slot and the "free" parity to wait for
      int h = hk * G, mt = mt_lo;
      for (int t = 0; t < T_tiles; ++t) {
        const int m0 = mt * BM;
        if (t > 0) {
          ok = mbar_wait(bar(FB_Q_FREE + sq), phq, actx, 711);
          if (!ok) break;
          mbar_expect_tx(bar(FB_Q_FULL + sq), C::kTile);
          for (int s = 0; s < KSUB; ++s)
            tma_load_4d(smem + C::kQ0 + sq * C::kTile + s * BM * 128, &map_q, bar(FB_Q_FULL + sq),
                        s * 64, m0, h, b);
          ++issued_q;
          ok = mbar_wait(bar(FB_DO_FREE + sd), phd, actx, 712);
          if (!ok) break;
          mbar_expect_tx(bar(FB_DO_FULL + sd), C::kTile);
          for (int s = 0; s < KSUB; ++s)
            tma_load_4d(smem + C::kDO0 + sd * C::kTile + s * BM * 128, &map_do, bar(FB_DO_FULL + sd),
                        s * 64, m0, h, b);
          ++issued_do;
        }
        if (++sq == NQ) sq = 0, phq ^= 1;
        if (++sd == NDO) sd = 0, phd ^= 1;
        if (++mt == mt_hi) mt = mt_lo, ++h;
      }
      if (!ok) {
        // let copies already in flight land before the CTA gives its shared memory back
        const long long t0 = clock64();
        for (int i = max(0, issued_q - NQ); i < issued_q; ++i)
          while (!mbar_try_wait(bar(FB_Q_FULL + i % NQ), (i / NQ) & 1) && clock64() - t0 < 2000000) {}
        for (int i = max(0, issued_do - NDO); i < issued_do; ++i)
          while (!mbar_try_wait(bar(FB_DO_FULL + i % NDO), (i / NDO) & 1) && clock64() - t0 < 2000000) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    if (lane == 0 && T_tiles > 0) {
      constexpr uint32_t idesc_s = instr_desc_f16(BN, BM, TcElem<T>::kFormat, 0, 0);   // S^T, dP^T
      constexpr uint32_t idesc_acc = instr_desc_f16(BN, D, TcElem<T>::kFormat, 0, 1);  // dV, dK
      constexpr uint32_t idesc_dq = instr_desc_f16(BM, D, TcElem<T>::kFormat, 1, 1);   // dQ
      constexpr uint32_t kTile16 = C::kTile >> 4;
      const uint32_t k_lo = smem_desc_lo(smem + C::kK, 0), v_lo = smem_desc_lo(smem + C::kV, 0);
      const uint32_t k_mn_lo = smem_desc_lo(smem + C::kK, BN * 128);     // K as MN-major B of dQ
      const uint32_t q_k_lo = smem_desc_lo(smem + C::kQ0, 0);            // Q as K-major B operand
      const uint32_t q_mn_lo = smem_desc_lo(smem + C::kQ0, BM * 128);     // Q as MN-major B operand
      const uint32_t do_k_lo = smem_desc_lo(smem + C::kDO0, 0);
      const uint32_t do_mn_lo = smem_desc_lo(smem + C::kDO0, BM * 128);
      const uint32_t pd_k_lo = smem_desc_lo(smem + C::kPD, 0);            // P^T / dS^T, K-major A
      const uint32_t pd_mn_lo = smem_desc_lo(smem + C::kPD, BN * 128);    // dS, MN-major A of dQ
      bool ok = mbar_wait(bar(FB_KV_FULL), 0, actx, 811);
      // S^T = K Q^T into the score columns
      auto issue_s = [&](int sq, int phq) -> bool {
        if (!mbar_wait(bar(FB_Q_FULL + sq), phq, actx, 812)) return false;
        tc_fence_after();
        const uint32_t b_lo = q_k_lo + sq * kTile16;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off16 = ((k / 4) * 128 * 128 + (k % 4) * 32) >> 4;
          mma_ss_lo(tmem + C::kColA, k_lo + off16, b_lo + off16, idesc_s, k > 0 ? 1u : 0u);
        }
        mma_commit(bar(FB_S_FULL));
        return true;
      };
      if (ok) ok = issue_s(0, 0);
      int sq = 0, phq = 0, sd = 0, phd = 0;
      for (int t = 0; t < T_tiles && ok; ++t) {
        int nsq = sq + 1, nphq = phq;
        if (nsq == NQ) nsq = 0, nphq ^= 1;
        const uint32_t acc = t > 0 ? 1u : 0u;
        const uint32_t par = t & 1;
        // dP^T(t) = V dO^T over S^T(t), once every element-wise warp holds S^T(t) in registers
        ok = mbar_wait(bar(FB_S_LOADED), par, actx, 813);
        if (ok && t == 0) ok = mbar_wait(bar(FB_V_FULL), 0, actx, 820);
        if (ok) ok = mbar_wait(bar(FB_DO_FULL + sd), phd, actx, 814);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t b_lo = do_k_lo + sd * kTile16;
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t off16 = ((k / 4) * 128 * 128 + (k % 4) * 32) >> 4;
            mma_ss_lo(tmem + C::kColA, v_lo + off16, b_lo + off16, idesc_s, k > 0 ? 1u : 0u);
          }
          mma_commit(bar(FB_DP_FULL));
        }
        // dV += P^T(t) dO(t), P^T from shared memory
        ok = mbar_wait(bar(FB_PT_FULL), par, actx, 815);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t b_lo = do_mn_lo + sd * kTile16;
#pragma unroll
          for (int kk = 0; kk < BM / 16; ++kk) {
            const uint32_t a_off16 = ((kk / 4) * 128 * 128 + (kk % 4) * 32) >> 4;
            mma_ss_lo(tmem + C::kColDV, pd_k_lo + a_off16, b_lo + ((kk * 16 * 128) >> 4), idesc_acc,
                      kk > 0 ? 1u : acc);
          }
          mma_commit(bar(FB_DO_FREE + sd));
          mma_commit(bar(FB_PT_FREE));
        }
        // S^T(t+1), once every element-wise warp holds dP^T(t) in registers
        if (t + 1 < T_tiles) {
          ok = mbar_wait(bar(FB_DP_LOADED), par, actx, 816);
          if (!ok) break;
          tc_fence_after();
          ok = issue_s(nsq, nphq);
          if (!ok) break;
        }
        // dQ(t) = dS(t) K, a fresh accumulator: the read-out of dQ(t-1) must be over
        ok = mbar_wait(bar(FB_DS_FULL), par, actx, 817);
        if (ok && t > 0) ok = mbar_wait(bar(FB_DQ_FREE), (t - 1) & 1, actx, 818);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint32_t off16 = (kk * 16 * 128) >> 4;
          mma_ss_lo(tmem + C::kColQ, pd_mn_lo + off16, k_mn_lo + off16, idesc_dq, kk > 0 ? 1u : 0u);
        }
        mma_commit(bar(FB_DQ_FULL));
        // dK += dS^T(t) Q(t)
        {
          const uint32_t b_lo = q_mn_lo + sq * kTile16;
#pragma unroll
          for (int kk = 0; kk < BM / 16; ++kk) {
            const uint32_t a_off16 = ((kk / 4) * 128 * 128 + (kk % 4) * 32) >> 4;
            mma_ss_lo(tmem + C::kColDK, pd_k_lo + a_off16, b_lo + ((kk * 16 * 128) >> 4), idesc_acc,
                      kk > 0 ? 1u : acc);
          }
          mma_commit(bar(FB_Q_FREE + sq));
          mma_commit(bar(FB_DS_FREE));
        }
        sq = nsq, phq = nphq;
        if (++sd == NDO) sd = 0, phd ^= 1;
      }
      if (ok) {
        mma_commit(bar(FB_DONE));
        mbar_wait(bar(FB_DONE), 0, actx, 819);
      }
    }
  } else if (warp == 2 + kEwWarps + 4) {
    // ------------------------------ statistics warp ----------------------------
    // -lse * log2(e) and -delta of the 128 queries of every tile go through shared memory, where
    // the element-wise threads read them as broadcast vectors (every thread needs the values of
    // all its 32 query columns; fetching them lane by lane and shuffling costs 64 shuffles per
    // thread and tile in a load/store queue that is already the busiest unit).  Queries past M
    // get lse = +inf, which makes their P exactly zero.  One buffer each: lse(t) may be written
    // once phase 1 of tile t - 1 is over, delta(t) once phase 2 of tile t - 1 is.
    float4 *lse_s = reinterpret_cast<float4 *>(smem_gen + C::kStats);
    float4 *dlt_s = lse_s + 32;
    int h = hk * G, mt = mt_lo;
    bool ok = true;
    for (int t = 0; t < T_tiles; ++t) {
      const int m = mt * BM + lane * 4;
      const int64_t li = ((int64_t)b * p.H + h) * p.M + m;
      if (++mt == mt_hi) mt = mt_lo, ++h;
      float l[4], d[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        l[j] = m + j < p.M ? -p.lse[li + j] * kLog2e : -INFINITY;
        d[j] = m + j < p.M ? -p.delta[li + j] : 0.f;
      }
      if (t > 0) ok = mbar_wait(bar(FB_PT_FULL), (t - 1) & 1, actx, 951);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      lse_s[lane] = make_float4(l[0], l[1], l[2], l[3]);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(FB_LSE_FULL));
      if (t > 0) ok = mbar_wait(bar(FB_DS_FULL), (t - 1) & 1, actx, 952);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      dlt_s[lane] = make_float4(d[0], d[1], d[2], d[3]);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(FB_DLT_FULL));
    }
  } else if (warp >= 2 + kEwWarps) {
    // ------------------------------ dQ reduction warps --------------------------
    // dQ(t) = dS K is a complete 128 x D product per tile.  These four warps (one per TMEM lane
    // slice = 32 query rows) move it out of TMEM a quarter of the columns at a time into a
    // shared-memory staging buffer, from where the copy engine adds it to the fp32 workspace
    // (`cp.reduce.async.bulk`, 2 KB runs).  An SM retires fp32 reductions at about 26 bytes per
    // clock whoever issues them, so the 64 KB of a tile take about as long as its GEMMs; issued
    // as `red` instructions they fill the load/store queue and stall every warp of the SM that
    // shuffles or touches shared memory.  Two staging buffers: a quarter drains while the next
    // is staged.
    const int slice = warp & 3;
    const int row = slice * 32 + lane;
    const uint32_t tlane = tmem + ((uint32_t)(slice * 32) << 16);
    const bool issuer = (warp == 2 + kEwWarps) && lane == 0;
    constexpr int QC = D / 4;                 // columns per quarter
    int h = hk * G, mt = mt_lo;
    int buf = 0;
    bool ok = true;
    for (int t = 0; t < T_tiles; ++t) {
      // the tile's block of the workspace: D / 4 runs of (128 queries x 4 columns), contiguous
      float *dst = fp.dq_acc + (((int64_t)b * p.H + h) * (fp.Mpad / BM) + mt) * (int64_t)(BM * D);
      if (++mt == mt_hi) mt = mt_lo, ++h;
      // every wait is bounded, so all four warps reach the vote; they leave together or not at all
      ok = red_warps_all(mbar_wait(bar(FB_DQ_FULL), t & 1, actx, 921));
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int qd = 0; qd < 4; ++qd) {
        uint32_t qr[QC];
        if (QC == 32) tmem_ld32(tlane + C::kColQ + qd * QC, *reinterpret_cast<uint32_t(*)[32]>(qr));
        else tmem_ld16(tlane + C::kColQ + qd * QC, qr);
        tmem_wait_ld();
        if (qd == 3) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(FB_DQ_FREE));   // dQ(t+1) may overwrite the columns
        }
        // the copy engine must have read what this buffer held two quarters ago
        if (issuer) bulk_wait_read_1();
        red_warps_sync();
        uint8_t *stage = smem_gen + C::kStage + buf * C::kQuarter + row * 16;
#pragma unroll
        for (int g = 0; g < QC / 4; ++g)
          *reinterpret_cast<uint4 *>(stage + g * 2048) =
              make_uint4(qr[4 * g], qr[4 * g + 1], qr[4 * g + 2], qr[4 * g + 3]);
        fence_proxy_async_smem();
        red_warps_sync();
        if (issuer) {
          // one contiguous run per quarter; rows past M hold zeros and land in padding
          bulk_reduce_add_f32(dst + qd * (C::kQuarter / 4), smem + C::kStage + buf * C::kQuarter,
                              C::kQuarter);
          bulk_commit();
        }
        buf ^= 1;
      }
    }
    if (issuer) bulk_wait_read_all();   // shared memory must outlive the copy engine's reads
  } else {
    // ------------------------------ element-wise warps --------------------------
    const int ew = warp - 2;
    const int slice = warp & 3, cg = ew >> 2;       // TMEM lane slice, 32-column group
    const int row = slice * 32 + lane;              // accumulator row of this thread
    const int key = n0 + row;
    const uint32_t tlane = tmem + ((uint32_t)(slice * 32) << 16);
    const float qk_scale = p.sm_scale * kLog2e;
    const bool key_ok = key < p.N;
    // this thread's 64 bytes of a PD row: sub-tile cg / 2, 16-byte chunks (cg & 1) * 4 .. + 3
    uint8_t *pd_row = smem_gen + C::kPD + (cg >> 1) * (128 * 128) + row * 128;
    const int pd_chunk0 = (cg & 1) * 4, pd_xor = row & 7;
    auto store_pd = [&](const uint32_t (&pk)[16]) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4 *>(pd_row + (((pd_chunk0 + j) ^ pd_xor) << 4)) =
            make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
    };
    bool ok = true;

    // -lse * log2(e) / -delta of this thread's 32 query columns, as staged by the statistics warp
    const float4 *lse_s = reinterpret_cast<const float4 *>(smem_gen + C::kStats) + cg * 8;
    const float4 *dlt_s = lse_s + 32;
    int mt = mt_lo;   // query tile of the current tile

    for (int t = 0; t < T_tiles; ++t) {
      const int m0 = mt * BM;
      if (++mt == mt_hi) mt = mt_lo;

      // ---- phase 1: P^T = exp2(S^T * scale - lse) -> PD ----
      ok = mbar_wait(bar(FB_LSE_FULL), t & 1, actx, 910);
      if (ok) ok = mbar_wait(bar(FB_S_FULL), t & 1, actx, 911);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float pv[32];
      uint32_t sr[32];
      tmem_ld32(tlane + C::kColA + cg * 32, sr);
      // while the load is in flight: the masks
      // Tiles away from every boundary (sequence end, causal diagonal, piecewise threshold) need no
      // masking at all; the others mask with one unsigned range check per element:
      // column c is visible iff cmin <= c < cmin + cwidth.
      bool interior = (n0 + BN <= p.N) && (!p.causal || m0 + p_seq >= n0 + BN - 1);
      if (p.mode == 1) interior = interior && (m0 + BM - 1 + p_seq - n0 < p.w);
      if (p.mode == 2) interior = interior && (m0 + p_seq - (n0 + BN - 1) >= p.w);
      int cmin = 0, cmax = 32;
      if (p.causal) cmin = max(cmin, key - p_seq - m0 - cg * 32);
      if (p.mode) {
        const int cnear = p.w + key - p_seq - m0 - cg * 32;  // columns below it are near pairs
        if (p.mode == 1) cmax = min(cmax, cnear);
        else cmin = max(cmin, cnear);
      }
      if (!key_ok) cmin = 32;
      const unsigned cwidth = (unsigned)max(cmax - cmin, 0);
      {
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(FB_S_LOADED));   // dP^T(t) may overwrite S^T(t)
        // packed fp32 pairs: one FMA per two elements
        const uint64_t scale2 = f2_pack(qk_scale, qk_scale);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 l4 = lse_s[i];
          f2_unpack(f2_fma(f2_pack(__uint_as_float(sr[4 * i]), __uint_as_float(sr[4 * i + 1])), scale2,
                           f2_pack(l4.x, l4.y)),
                    pv[4 * i], pv[4 * i + 1]);
          f2_unpack(f2_fma(f2_pack(__uint_as_float(sr[4 * i + 2]), __uint_as_float(sr[4 * i + 3])),
                           scale2, f2_pack(l4.z, l4.w)),
                    pv[4 * i + 2], pv[4 * i + 3]);
        }
      }
      if (!interior) {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          pv[c] = ((unsigned)(c - cmin) < cwidth) ? pv[c] : -INFINITY;  // exp2(-inf) = 0
      }
      {
        uint32_t pk[16];
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          pv[c] = ex2(pv[c]);
          pv[c + 1] = ex2(pv[c + 1]);
          pk[c >> 1] = TcElem<T>::pack(pv[c], pv[c + 1]);
        }
        // PD still holds dS^T(t-1) until dQ(t-1) and dK(t-1) have read it
        if (t > 0) ok = mbar_wait(bar(FB_DS_FREE), (t - 1) & 1, actx, 912);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        store_pd(pk);
      }
      // ---- phase 2: dS^T = P^T * (dP^T - delta) -> PD ----
      // Its operands are there by now (dP^T(t) was issued as soon as S^T(t) had been read), so the
      // first TMEM load goes out before the proxy fence of phase 1 and hides behind it.
      ok = mbar_wait(bar(FB_DLT_FULL), t & 1, actx, 909);
      if (ok) ok = mbar_wait(bar(FB_DP_FULL), t & 1, actx, 913);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr0[16];
      tmem_ld16(tlane + C::kColA + cg * 32, sr0);
      fence_proxy_async_smem();   // the MMA reads PD through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(FB_PT_FULL));
      {
        uint32_t pk[16];
        // P * (dP - delta) of 16 columns, two elements per instruction
        auto half_ds = [&](int hf, const uint32_t (&sr)[16]) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 d4 = dlt_s[hf * 4 + i];
            const int c = 4 * i;
            float e0, e1, e2, e3;
            f2_unpack(f2_mul(f2_pack(pv[hf * 16 + c], pv[hf * 16 + c + 1]),
                             f2_add(f2_pack(__uint_as_float(sr[c]), __uint_as_float(sr[c + 1])),
                                    f2_pack(d4.x, d4.y))),
                      e0, e1);
            f2_unpack(f2_mul(f2_pack(pv[hf * 16 + c + 2], pv[hf * 16 + c + 3]),
                             f2_add(f2_pack(__uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3])),
                                    f2_pack(d4.z, d4.w))),
                      e2, e3);
            pk[hf * 8 + 2 * i] = TcElem<T>::pack(e0, e1);
            pk[hf * 8 + 2 * i + 1] = TcElem<T>::pack(e2, e3);
          }
        };
        tmem_wait_ld();            // first 16 columns (requested before the fence above)
        half_ds(0, sr0);
        {
          uint32_t sr1[16];
          tmem_ld16(tlane + C::kColA + cg * 32 + 16, sr1);
          tmem_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(FB_DP_LOADED));   // S^T(t+1) may overwrite dP^T(t)
          half_ds(1, sr1);
        }
        // PD still holds P^T(t) until dV(t) has read it
        ok = mbar_wait(bar(FB_PT_FREE), t & 1, actx, 914);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        store_pd(pk);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(FB_DS_FULL));
    }

    // ---- write-out of dV and dK: warp (slice, cg) owns columns cg * D / 4 .. of its 32 rows ----
    // dV is final once its last product has been committed (the PT_FREE wait that ended the loop),
    // so it is converted and handed to the copy engine while dQ and dK of the last tile still run
    // on the tensor cores; dK follows after the last commit.  The tiles are staged in the shared
    // memory of V and K (both dead by then) in the layout of their own loads, and leave as bulk
    // tensor stores, which also drop the rows past N.  Two cases keep per-thread global stores:
    // a dV that is added to (the second launch of a piecewise backward) and a CTA without tiles.
    constexpr int QC = D / 4;
    const int col0 = cg * QC;
    auto load_cols = [&](uint32_t col_base, uint32_t (&ov)[QC]) {
      if (QC == 32) tmem_ld32(tlane + col_base + col0, *reinterpret_cast<uint32_t(*)[32]>(ov));
      else tmem_ld16(tlane + col_base + col0, ov);
      tmem_wait_ld();
    };
    auto pack8 = [&](const uint32_t *ov, float scale) {
      return make_uint4(
          TcElem<T>::pack(__uint_as_float(ov[0]) * scale, __uint_as_float(ov[1]) * scale),
          TcElem<T>::pack(__uint_as_float(ov[2]) * scale, __uint_as_float(ov[3]) * scale),
          TcElem<T>::pack(__uint_as_float(ov[4]) * scale, __uint_as_float(ov[5]) * scale),
          TcElem<T>::pack(__uint_as_float(ov[6]) * scale, __uint_as_float(ov[7]) * scale));
    };
    auto stage = [&](int region, const uint32_t (&ov)[QC], float scale) {
      uint8_t *base = smem_gen + region + (col0 / 64) * (128 * 128) + row * 128;
      const int ch0 = (col0 % 64) / 8;
#pragma unroll
      for (int j = 0; j < QC / 8; ++j)
        *reinterpret_cast<uint4 *>(base + (((ch0 + j) ^ (row & 7)) << 4)) = pack8(ov + 8 * j, scale);
    };
    auto direct = [&](void *out, const Strides &so, uint32_t (&ov)[QC], float scale, bool add) {
      if (!key_ok) return;
      T *orow = row_ptr_mut<T>(out, so, b, hk, key) + col0;
#pragma unroll
      for (int j = 0; j < QC / 8; ++j) {
        if (add) {
          const uint4 old = *reinterpret_cast<const uint4 *>(orow + j * 8);
          const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
          for (int e2 = 0; e2 < 4; ++e2) {
            const float2 f = TcElem<T>::unpack(ow[e2]);
            ov[8 * j + 2 * e2] = __float_as_uint(__uint_as_float(ov[8 * j + 2 * e2]) + f.x);
            ov[8 * j + 2 * e2 + 1] = __float_as_uint(__uint_as_float(ov[8 * j + 2 * e2 + 1]) + f.y);
          }
        }
        *reinterpret_cast<uint4 *>(orow + j * 8) = pack8(ov + 8 * j, scale);
      }
    };
    const bool elected = ew == 0 && lane == 0;
    if (T_tiles > 0) {
      // every element-wise warp runs both votes below, whatever happened to its own waits
      uint32_t ov[QC];
      const bool bulk_dv = !p.dv_accumulate;
      if (ok) {
        tc_fence_after();
        load_cols(C::kColDV, ov);
        if (bulk_dv) {
          stage(C::kV, ov, 1.f);
          fence_proxy_async_smem();
        } else {
          direct(p.dv, p.sdv, ov, 1.f, true);
        }
      }
      ok = ew_warps_all(ok);
      if (ok && bulk_dv && elected) {
#pragma unroll
        for (int s = 0; s < KSUB; ++s)
          tma_store_4d(&map_dv, smem + C::kV + s * BN * 128, s * 64, n0, hk, b);
        bulk_commit();
      }
      if (ok) ok = mbar_wait(bar(FB_DONE), 0, actx, 916);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        load_cols(C::kColDK, ov);
        stage(C::kK, ov, p.sm_scale);
        fence_proxy_async_smem();
      }
      ok = ew_warps_all(ok);
      if (elected) {
        if (ok) {
#pragma unroll
          for (int s = 0; s < KSUB; ++s)
            tma_store_4d(&map_dk, smem + C::kK + s * BN * 128, s * 64, n0, hk, b);
          bulk_commit();
        }
        bulk_wait_read_all();   // shared memory must outlive the copy engine's reads
      }
    } else if (ok) {
      uint32_t ov[QC];
#pragma unroll
      for (int i = 0; i < QC; ++i) ov[i] = 0u;
      direct(p.dk, p.sdk, ov, 1.f, false);
      if (!p.dv_accumulate) direct(p.dv, p.sdv, ov, 1.f, false);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, C::kTmemCols);
  }
}

// dq = dq_acc * scale, converted to 16 bits.  Block = 32 queries x 8 warps; warp w converts the
// sixteen-column groups w, w + 8, ... of its 32 rows (lane = row: the fp32 reads are 512-byte
// runs, and a thread writes one whole 32-byte sector of its row).
template <typename T, int D>
__global__ void __launch_bounds__(256)
    dq_convert_kernel(const float *__restrict__ acc, void *dq, Strides sdq, int H, int M, int Mpad,
                      float scale) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int m = blockIdx.x * 32 + lane;
  const int h = blockIdx.y, b = blockIdx.z;
  if (m >= M) return;
  // workspace layout (B, H, Mpad / 128, D / 4, 128, 4)
  const float *src = acc + (((int64_t)b * H + h) * (Mpad / 128) + m / 128) * (int64_t)(128 * D) +
                     (m % 128) * 4;
  T *orow = row_ptr_mut<T>(dq, sdq, b, h, m);
#pragma unroll
  for (int g = w; g < D / 16; g += 8) {
    float4 f[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = *reinterpret_cast<const float4 *>(src + (4 * g + i) * 512);
    uint4 v[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      v[i].x = TcElem<T>::pack(f[2 * i].x * scale, f[2 * i].y * scale);
      v[i].y = TcElem<T>::pack(f[2 * i].z * scale, f[2 * i].w * scale);
      v[i].z = TcElem<T>::pack(f[2 * i + 1].x * scale, f[2 * i + 1].y * scale);
      v[i].w = TcElem<T>::pack(f[2 * i + 1].z * scale, f[2 * i + 1].w * scale);
    }
    *reinterpret_cast<uint4 *>(orow + g * 16) = v[0];
    *reinterpret_cast<uint4 *>(orow + g * 16 + 8) = v[1];
  }
}

}  // namespace tc
}  // namespace fa
