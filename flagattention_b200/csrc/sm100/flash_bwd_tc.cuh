// flash_attention backward on tcgen05 for head_dim 64 and 128: the dK/dV kernel
// and the dQ kernel.  No global atomics; P is recomputed from the saved
// log-normaliser, so the element-wise warps need no row statistics.
//
// Skeleton (both kernels):
//   warp 0       TMA producer
//   warp 1       MMA issuer (one thread); every MMA is 128 x 128 x 16
//   warps 2..17  element-wise stage, one thread per (accumulator row, 32 columns),
//                four warps per TMEM lane slice
//
// All score tiles are 128 x 128 and live once in TMEM.  The four (three) GEMMs of
// a tile are issued in an order that staggers the two TMEM score buffers, so the
// tensor pipe always has a GEMM of the neighbouring tile to run while the
// element-wise warps work:
//   dK/dV:  dV(t) | S^T(t+1) | dK(t) | dP^T(t+1)       P^T over S^T, dS^T over dP^T
//   dQ:     S(t+1) | dP(t+1) | dQ(t)                   dP double-buffered, dS over dP
// Phase 1 of the element-wise stage (P = exp2(S*scale - L)) runs as soon as S is
// complete, phase 2 (dS = P * (dP - delta)) as soon as dP is.
#pragma once

#include "../attn_params.cuh"
#include "tc_common.cuh"

namespace fa {
namespace tc {

struct BwdTcParams {
  const float *lse, *delta;
  void *dq, *dk, *dv;
  Strides sdq, sdk, sdv;
  int B, H, Hk, M, N;
  int causal;
  float sm_scale;
  // piecewise_attention runs each kernel twice: mode 1 = near branch (pairs whose distance
  // (m + N - M) - n is below w, scored with q1.k1), mode 2 = far branch (distance >= w, q2.k2);
  // every launch only visits tiles that hold a pair of its branch and masks the others out.
  // mode 0 = flash_attention.
  int mode, w;
  int dv_accumulate;  // dK/dV kernel: add dV to what `dv` already holds (second piecewise launch)
  int *status;
  int num_blocks, group_size;  // launch order of the two-kernel backward, see grouped_cta()
};

constexpr int kEwWarps = 16;                       // element-wise warps
constexpr int kBwdThreads = (2 + kEwWarps) * 32;   // 576

// Stores 32 accumulator columns (fp32 in `ov`, scaled) as 16-bit values to global memory.
template <typename T>
__device__ __forceinline__ void store_row32(T *dst, const uint32_t (&ov)[32], float scale) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 v;
    v.x = TcElem<T>::pack(__uint_as_float(ov[8 * i + 0]) * scale, __uint_as_float(ov[8 * i + 1]) * scale);
    v.y = TcElem<T>::pack(__uint_as_float(ov[8 * i + 2]) * scale, __uint_as_float(ov[8 * i + 3]) * scale);
    v.z = TcElem<T>::pack(__uint_as_float(ov[8 * i + 4]) * scale, __uint_as_float(ov[8 * i + 5]) * scale);
    v.w = TcElem<T>::pack(__uint_as_float(ov[8 * i + 6]) * scale, __uint_as_float(ov[8 * i + 7]) * scale);
    *reinterpret_cast<uint4 *>(dst + i * 8) = v;
  }
}

// ===========================================================================
// dK / dV: one CTA per 128 keys, query tiles of 128, loops over the query
// heads of a GQA group
// ===========================================================================
template <int D>
struct DkdvTcCfg {
  static constexpr int BM = 128, BN = 128, NQ = 3, NDO = 2;
  static constexpr int KSUB = D / 64;
  static constexpr int kTile = 128 * D * 2;            // any 128-row operand tile
  static constexpr int kK = 0;
  static constexpr int kV = kTile;
  static constexpr int kQ0 = 2 * kTile;                // Q ring: NQ x (Q tile)
  static constexpr int kDO0 = kQ0 + NQ * kTile;        // dO ring: NDO x (dO tile)
  static constexpr int kBars = kDO0 + NDO * kTile;
  static constexpr int kStats = kBars + 24 * 8;        // lse[128] | delta[128] of the current tile
  static constexpr int kMisc = kStats + 2 * 128 * 4;
  static constexpr int kTotal = kMisc + 16 + 1024;
  static constexpr int kTmemCols = 512;
  static constexpr int kColS = 0, kColDP = 128, kColDK = 256, kColDV = 256 + D;
  static_assert(kTotal <= 232448, "shared memory budget");
};

enum DkdvBar { KV_KV_FULL = 0, KV_Q_FULL = 1, KV_Q_FREE = 4, KV_DO_FULL = 7, KV_DO_FREE = 9,
               KV_S_FULL = 11, KV_DP_FULL = 12, KV_P1 = 13, KV_P2 = 14, KV_DONE = 15,
               KV_LSE_FULL = 16, KV_DLT_FULL = 17 };

// the dK/dV kernel has one more warp, which stages lse / delta of every tile in shared memory
constexpr int kDkdvThreads = kBwdThreads + 32;

template <typename T, int D>
__global__ void __launch_bounds__(kDkdvThreads, 1)
    flash_bwd_dkdv_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                             const __grid_constant__ CUtensorMap map_do,
                             const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, const BwdTcParams p) {
  using C = DkdvTcCfg<D>;
  constexpr int BM = C::BM, BN = C::BN, KSUB = C::KSUB, NQ = C::NQ, NDO = C::NDO;
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
  if (p.mode == 1) {  // query tiles that hold a near pair: m0 < w - p_seq + n0 + BN - 1
    const int lim = p.w - p_seq + n0 + BN - 1;
    mt_hi = min(mt_hi, lim <= 0 ? 0 : (lim + BM - 1) / BM);
  } else if (p.mode == 2) {  // query tiles that hold a far pair: m0 >= w - p_seq + n0 - (BM - 1)
    const int lim = p.w - p_seq + n0 - (BM - 1);
    mt_lo = max(mt_lo, lim <= 0 ? 0 : (lim + BM - 1) / BM);
  }
  const int tiles = max(0, mt_hi - mt_lo);
  const int T_tiles = tiles * G;

  if (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) return;

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar(KV_KV_FULL), 1);
    for (int s = 0; s < NQ; ++s) {
      mbar_init(bar(KV_Q_FULL + s), 1);
      mbar_init(bar(KV_Q_FREE + s), 1);
    }
    for (int s = 0; s < NDO; ++s) {
      mbar_init(bar(KV_DO_FULL + s), 1);
      mbar_init(bar(KV_DO_FREE + s), 1);
    }
    mbar_init(bar(KV_S_FULL), 1);
    mbar_init(bar(KV_DP_FULL), 1);
    mbar_init(bar(KV_P1), kEwWarps);
    mbar_init(bar(KV_P2), kEwWarps);
    mbar_init(bar(KV_DONE), 1);
    mbar_init(bar(KV_LSE_FULL), 1);
    mbar_init(bar(KV_DLT_FULL), 1);
    fence_barrier_init();
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
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_do);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      mbar_expect_tx(bar(KV_KV_FULL), 2 * C::kTile);
      for (int s = 0; s < KSUB; ++s) {
        tma_load_4d(smem + C::kK + s * BN * 128, &map_k, bar(KV_KV_FULL), s * 64, n0, hk, b);
        tma_load_4d(smem + C::kV + s * BN * 128, &map_v, bar(KV_KV_FULL), s * 64, n0, hk, b);
      }
      int issued_q = 0, issued_do = 0;
      bool ok = true;
      for (int t = 0; t < T_tiles; ++t) {
        const int h = hk * G + t / tiles, m0 = (mt_lo + t % tiles) * BM;
        const int sq = t % NQ, sd = t % NDO;
        ok = mbar_wait(bar(KV_Q_FREE + sq), ((t / NQ) & 1) ^ 1, actx, 701);
        if (!ok) break;
        mbar_expect_tx(bar(KV_Q_FULL + sq), C::kTile);
        for (int s = 0; s < KSUB; ++s)
          tma_load_4d(smem + C::kQ0 + sq * C::kTile + s * BM * 128, &map_q, bar(KV_Q_FULL + sq),
                      s * 64, m0, h, b);
        ++issued_q;
        ok = mbar_wait(bar(KV_DO_FREE + sd), ((t / NDO) & 1) ^ 1, actx, 702);
        if (!ok) break;
        mbar_expect_tx(bar(KV_DO_FULL + sd), C::kTile);
        for (int s = 0; s < KSUB; ++s)
          tma_load_4d(smem + C::kDO0 + sd * C::kTile + s * BM * 128, &map_do, bar(KV_DO_FULL + sd),
                      s * 64, m0, h, b);
        ++issued_do;
      }
      if (!ok) {
        // let copies already in flight land before the CTA gives its shared memory back
        const long long t0 = clock64();
        for (int i = max(0, issued_q - NQ); i < issued_q; ++i)
          while (!mbar_try_wait(bar(KV_Q_FULL + i % NQ), (i / NQ) & 1) && clock64() - t0 < 2000000) {}
        for (int i = max(0, issued_do - NDO); i < issued_do; ++i)
          while (!mbar_try_wait(bar(KV_DO_FULL + i % NDO), (i / NDO) & 1) && clock64() - t0 < 2000000) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    // The issuing thread is on the critical path of every MMA, so the loop keeps its own work
    // minimal: descriptor low words are precomputed per operand, ring positions and barrier
    // parities are running counters, and each MMA costs two integer adds besides itself.
    if (lane == 0 && T_tiles > 0) {
      constexpr uint32_t idesc_s = instr_desc_f16(BN, BM, TcElem<T>::kFormat, 0, 0);   // 128 x 128
      constexpr uint32_t idesc_acc = instr_desc_f16(BN, D, TcElem<T>::kFormat, 0, 1);  // 128 x D
      constexpr uint32_t kTile16 = C::kTile >> 4;
      const uint32_t k_lo = smem_desc_lo(smem + C::kK, 0), v_lo = smem_desc_lo(smem + C::kV, 0);
      const uint32_t q_k_lo = smem_desc_lo(smem + C::kQ0, 0);            // Q as K-major B operand
      const uint32_t q_mn_lo = smem_desc_lo(smem + C::kQ0, BM * 128);     // Q as MN-major B operand
      const uint32_t do_k_lo = smem_desc_lo(smem + C::kDO0, 0);
      const uint32_t do_mn_lo = smem_desc_lo(smem + C::kDO0, BM * 128);
      bool ok = mbar_wait(bar(KV_KV_FULL), 0, actx, 801);
      // S^T(t) = K Q(t)^T, Q(t) in ring slot sq whose barrier is in phase phq
      auto issue_s = [&](int sq, int phq) -> bool {
        if (!mbar_wait(bar(KV_Q_FULL + sq), phq, actx, 802)) return false;
        tc_fence_after();
        const uint32_t b_lo = q_k_lo + sq * kTile16;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off16 = ((k / 4) * 128 * 128 + (k % 4) * 32) >> 4;
          mma_ss_lo(tmem + C::kColS, k_lo + off16, b_lo + off16, idesc_s, k > 0 ? 1u : 0u);
        }
        mma_commit(bar(KV_S_FULL));
        return true;
      };
      // dP^T(t) = V dO(t)^T
      auto issue_dp = [&](int sd, int phd) -> bool {
        if (!mbar_wait(bar(KV_DO_FULL + sd), phd, actx, 803)) return false;
        tc_fence_after();
        const uint32_t b_lo = do_k_lo + sd * kTile16;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off16 = ((k / 4) * 128 * 128 + (k % 4) * 32) >> 4;
          mma_ss_lo(tmem + C::kColDP, v_lo + off16, b_lo + off16, idesc_s, k > 0 ? 1u : 0u);
        }
        mma_commit(bar(KV_DP_FULL));
        return true;
      };
      if (ok) ok = issue_s(0, 0);
      if (ok) ok = issue_dp(0, 0);
      // ring positions / phases of tile t (sq, phq, sd, phd) and of tile t + 1 (n*)
      int sq = 0, phq = 0, sd = 0, phd = 0;
      for (int t = 0; t < T_tiles && ok; ++t) {
        int nsq = sq + 1, nphq = phq, nsd = sd + 1, nphd = phd;
        if (nsq == NQ) nsq = 0, nphq ^= 1;
        if (nsd == NDO) nsd = 0, nphd ^= 1;
        const uint32_t acc = t > 0 ? 1u : 0u;
        // dV += P^T(t) dO(t)
        ok = mbar_wait(bar(KV_P1), t & 1, actx, 804);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t b_lo = do_mn_lo + sd * kTile16;
#pragma unroll
          for (int kk = 0; kk < BM / 16; ++kk)
            mma_ts_lo(tmem + C::kColDV, tmem + C::kColS + (kk >> 1) * 32 + (kk & 1) * 8,
                      b_lo + ((kk * 16 * 128) >> 4), idesc_acc, kk > 0 ? 1u : acc);
          mma_commit(bar(KV_DO_FREE + sd));
        }
        if (t + 1 < T_tiles) ok = issue_s(nsq, nphq);
        if (!ok) break;
        // dK += dS^T(t) Q(t)
        ok = mbar_wait(bar(KV_P2), t & 1, actx, 805);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t b_lo = q_mn_lo + sq * kTile16;
#pragma unroll
          for (int kk = 0; kk < BM / 16; ++kk)
            mma_ts_lo(tmem + C::kColDK, tmem + C::kColDP + (kk >> 1) * 32 + (kk & 1) * 8,
                      b_lo + ((kk * 16 * 128) >> 4), idesc_acc, kk > 0 ? 1u : acc);
          mma_commit(bar(KV_Q_FREE + sq));
        }
        if (t + 1 < T_tiles) ok = issue_dp(nsd, nphd);
        sq = nsq, phq = nphq, sd = nsd, phd = nphd;
      }
      if (ok) {
        mma_commit(bar(KV_DONE));
        mbar_wait(bar(KV_DONE), 0, actx, 806);
      }
    }
  } else if (warp == 2 + kEwWarps) {
    // ------------------------------ statistics warp ----------------------------
    // lse (in the base-2 domain) and delta of the 128 queries of every tile go through shared
    // memory, where the element-wise threads read them as broadcast vectors: every thread needs
    // the values of all its 32 query columns.  Queries past M get lse = +inf, which makes their P
    // exactly zero.  One buffer each: lse(t) may be written once phase 1 of tile t - 1 is over,
    // delta(t) once phase 2 of tile t - 1 is.
    float4 *lse_s = reinterpret_cast<float4 *>(smem_gen + C::kStats);
    float4 *dlt_s = lse_s + 32;
    bool ok = true;
    for (int t = 0; t < T_tiles; ++t) {
      const int h = hk * G + t / tiles, m0 = (mt_lo + t % tiles) * BM;
      const int m = m0 + lane * 4;
      const int64_t li = ((int64_t)b * p.H + h) * p.M + m;
      float l[4], d[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        l[j] = m + j < p.M ? p.lse[li + j] * kLog2e : INFINITY;
        d[j] = m + j < p.M ? p.delta[li + j] : 0.f;
      }
      if (t > 0) ok = mbar_wait(bar(KV_P1), (t - 1) & 1, actx, 951);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      lse_s[lane] = make_float4(l[0], l[1], l[2], l[3]);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(KV_LSE_FULL));
      if (t > 0) ok = mbar_wait(bar(KV_P2), (t - 1) & 1, actx, 952);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      dlt_s[lane] = make_float4(d[0], d[1], d[2], d[3]);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(KV_DLT_FULL));
    }
  } else {
    // ------------------------------ element-wise warps --------------------------
    const int ew = warp - 2;
    const int slice = warp & 3, cg = ew >> 2;       // TMEM lane slice, 32-column group
    const int key = n0 + slice * 32 + lane;
    const uint32_t tlane = tmem + ((uint32_t)(slice * 32) << 16);
    const float qk_scale = p.sm_scale * kLog2e;
    const bool key_ok = key < p.N;
    // lse / delta of this thread's 32 query columns, as staged by the statistics warp
    const float4 *lse_s = reinterpret_cast<const float4 *>(smem_gen + C::kStats) + cg * 8;
    const float4 *dlt_s = lse_s + 32;
    bool ok = true;

    for (int t = 0; t < T_tiles; ++t) {
      const int m0 = (mt_lo + t % tiles) * BM;
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

      // ---- phase 1: P^T = exp2(S^T * scale - lse), written over S^T ----
      ok = mbar_wait(bar(KV_LSE_FULL), t & 1, actx, 900);
      if (ok) ok = mbar_wait(bar(KV_S_FULL), t & 1, actx, 901);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[32];
      tmem_ld32(tlane + C::kColS + cg * 32, sr);
      tmem_wait_ld();
      float pv[32];
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 l4 = lse_s[i];
        pv[4 * i + 0] = fmaf(__uint_as_float(sr[4 * i + 0]), qk_scale, -l4.x);
        pv[4 * i + 1] = fmaf(__uint_as_float(sr[4 * i + 1]), qk_scale, -l4.y);
        pv[4 * i + 2] = fmaf(__uint_as_float(sr[4 * i + 2]), qk_scale, -l4.z);
        pv[4 * i + 3] = fmaf(__uint_as_float(sr[4 * i + 3]), qk_scale, -l4.w);
      }
      if (!interior) {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          pv[c] = ((unsigned)(c - cmin) < cwidth) ? pv[c] : -INFINITY;  // exp2(-inf) = 0
      }
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        pv[c] = ex2(pv[c]);
        pv[c + 1] = ex2(pv[c + 1]);
        pk[c >> 1] = TcElem<T>::pack(pv[c], pv[c + 1]);
      }
      tmem_st16(tlane + C::kColS + cg * 32, pk);  // inside this thread's own columns
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(KV_P1));

      // ---- phase 2: dS^T = P^T * (dP^T - delta), written over dP^T ----
      ok = mbar_wait(bar(KV_DLT_FULL), t & 1, actx, 902);
      if (ok) ok = mbar_wait(bar(KV_DP_FULL), t & 1, actx, 903);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      tmem_ld32(tlane + C::kColDP + cg * 32, sr);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 d4 = dlt_s[i];
        pk[2 * i] = TcElem<T>::pack(pv[4 * i] * (__uint_as_float(sr[4 * i]) - d4.x),
                                    pv[4 * i + 1] * (__uint_as_float(sr[4 * i + 1]) - d4.y));
        pk[2 * i + 1] = TcElem<T>::pack(pv[4 * i + 2] * (__uint_as_float(sr[4 * i + 2]) - d4.z),
                                        pv[4 * i + 3] * (__uint_as_float(sr[4 * i + 3]) - d4.w));
      }
      tmem_st16(tlane + C::kColDP + cg * 32, pk);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(KV_P2));
    }

    if (ok && T_tiles > 0) {
      ok = mbar_wait(bar(KV_DONE), 0, actx, 904);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      // warps of column groups 0 / 1 store dK, groups 2 / 3 store dV; each thread half a row
      const int which = cg >> 1, half = cg & 1;
      constexpr int COLS = D / 2;
      T *orow = which == 0 ? row_ptr_mut<T>(p.dk, p.sdk, b, hk, key)
                           : row_ptr_mut<T>(p.dv, p.sdv, b, hk, key);
      const float scale = which == 0 ? p.sm_scale : 1.f;
      const uint32_t col_base = which == 0 ? C::kColDK : C::kColDV;
#pragma unroll
      for (int c = 0; c < COLS / 32; ++c) {
        uint32_t ov[32];
        const int col0 = half * COLS + c * 32;
        if (T_tiles > 0) {
          tmem_ld32(tlane + col_base + col0, ov);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = 0u;
        }
        if (which == 1 && p.dv_accumulate && key_ok) {
          // second piecewise launch: add the first launch's dV
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4 old = *reinterpret_cast<const uint4 *>(orow + col0 + i * 8);
            const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
              const float2 f = TcElem<T>::unpack(ow[e2]);
              ov[8 * i + 2 * e2] = __float_as_uint(__uint_as_float(ov[8 * i + 2 * e2]) + f.x);
              ov[8 * i + 2 * e2 + 1] = __float_as_uint(__uint_as_float(ov[8 * i + 2 * e2 + 1]) + f.y);
            }
          }
        }
        if (key_ok) store_row32<T>(orow + col0, ov, scale);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, C::kTmemCols);
  }
}

// ===========================================================================
// dQ: one CTA per 128 query rows, key tiles of 128
// ===========================================================================
template <int D>
struct DqTcCfg {
  static constexpr int BM = 128, BN = 128, NK = 3, NV = 2;
  static constexpr int KSUB = D / 64;
  static constexpr int kTile = 128 * D * 2;
  static constexpr int kQ = 0;
  static constexpr int kDO = kTile;
  static constexpr int kK0 = 2 * kTile;              // K ring
  static constexpr int kV0 = kK0 + NK * kTile;       // V ring
  static constexpr int kBars = kV0 + NV * kTile;
  static constexpr int kMisc = kBars + 24 * 8;
  static constexpr int kTotal = kMisc + 16 + 1024;
  static constexpr int kTmemCols = 512;
  // S | dP0 | dP1 | dQ
  static constexpr int kColS = 0, kColDP = 128, kColDQ = 384;
};

enum DqBar { DQ_QDO_FULL = 0, DQ_K_FULL = 1, DQ_K_FREE = 4, DQ_V_FULL = 7, DQ_V_FREE = 9,
             DQ_S_FULL = 11, DQ_S_CONSUMED = 12, DQ_DP_FULL = 13, DQ_DS_READY = 15, DQ_DONE = 17 };

template <typename T, int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
    flash_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                           const __grid_constant__ CUtensorMap map_do,
                           const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, const BwdTcParams p) {
  using C = DqTcCfg<D>;
  constexpr int BM = C::BM, BN = C::BN, KSUB = C::KSUB, NK = C::NK, NV = C::NV;
  extern __shared__ uint8_t smem_unaligned[];
  const uint32_t smem = (smem_u32(smem_unaligned) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_unaligned + (smem - smem_u32(smem_unaligned));
  auto bar = [&](int i) { return smem + C::kBars + i * 8; };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + C::kMisc);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + C::kMisc + 8);
  const AbortCtx actx{abort_flag, p.status};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const CtaCoord cta = grouped_cta(blockIdx.x, p.num_blocks, p.B * p.H, p.group_size);
  const int mb = p.num_blocks - 1 - cta.blk;  // heaviest causal tiles first
  const int b = cta.pair / p.H, h = cta.pair % p.H;
  const int hk = h / (p.H / p.Hk);
  const int m0 = mb * BM;
  const int p_seq = p.N - p.M;
  int n_hi = p.N;
  if (p.causal) n_hi = min(n_hi, p_seq + m0 + BM);
  const int T_all = n_hi > 0 ? (n_hi + BN - 1) / BN : 0;
  // piecewise: key tiles [0, jf) are entirely far, [jn, T) entirely near
  int t_lo = 0, t_hi = T_all, jf = 0, jn = 0;
  if (p.mode) {
    const int x = m0 + p_seq - (BN - 1) - p.w, y = m0 + BM - 1 + p_seq - p.w;
    jf = x < 0 ? 0 : min(T_all, x / BN + 1);
    jn = y < 0 ? 0 : min(T_all, y / BN + 1);
    if (p.mode == 1) t_lo = jf; else t_hi = jn;
  }
  const int T_tiles = max(0, t_hi - t_lo);

  if (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) return;

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar(DQ_QDO_FULL), 1);
    for (int s = 0; s < NK; ++s) {
      mbar_init(bar(DQ_K_FULL + s), 1);
      mbar_init(bar(DQ_K_FREE + s), 1);
    }
    for (int s = 0; s < NV; ++s) {
      mbar_init(bar(DQ_V_FULL + s), 1);
      mbar_init(bar(DQ_V_FREE + s), 1);
    }
    mbar_init(bar(DQ_S_FULL), 1);
    mbar_init(bar(DQ_S_CONSUMED), kEwWarps);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(DQ_DP_FULL + s), 1);
      mbar_init(bar(DQ_DS_READY + s), kEwWarps);
    }
    mbar_init(bar(DQ_DONE), 1);
    fence_barrier_init();
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
    // ------------------------------ TMA producer --------------------------------
    if (lane == 0 && T_tiles > 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_do);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      mbar_expect_tx(bar(DQ_QDO_FULL), 2 * C::kTile);
      for (int s = 0; s < KSUB; ++s) {
        tma_load_4d(smem + C::kQ + s * BM * 128, &map_q, bar(DQ_QDO_FULL), s * 64, m0, h, b);
        tma_load_4d(smem + C::kDO + s * BM * 128, &map_do, bar(DQ_QDO_FULL), s * 64, m0, h, b);
      }
      int issued_k = 0, issued_v = 0;
      bool ok = true;
      for (int t = 0; t < T_tiles; ++t) {
        const int sk = t % NK, sv = t % NV, n0 = (t_lo + t) * BN;
        ok = mbar_wait(bar(DQ_K_FREE + sk), ((t / NK) & 1) ^ 1, actx, 401);
        if (!ok) break;
        mbar_expect_tx(bar(DQ_K_FULL + sk), C::kTile);
        for (int s = 0; s < KSUB; ++s)
          tma_load_4d(smem + C::kK0 + sk * C::kTile + s * BN * 128, &map_k, bar(DQ_K_FULL + sk),
                      s * 64, n0, hk, b);
        ++issued_k;
        ok = mbar_wait(bar(DQ_V_FREE + sv), ((t / NV) & 1) ^ 1, actx, 402);
        if (!ok) break;
        mbar_expect_tx(bar(DQ_V_FULL + sv), C::kTile);
        for (int s = 0; s < KSUB; ++s)
          tma_load_4d(smem + C::kV0 + sv * C::kTile + s * BN * 128, &map_v, bar(DQ_V_FULL + sv),
                      s * 64, n0, hk, b);
        ++issued_v;
      }
      if (!ok) {
        const long long t0 = clock64();
        for (int i = max(0, issued_k - NK); i < issued_k; ++i)
          while (!mbar_try_wait(bar(DQ_K_FULL + i % NK), (i / NK) & 1) && clock64() - t0 < 2000000) {}
        for (int i = max(0, issued_v - NV); i < issued_v; ++i)
          while (!mbar_try_wait(bar(DQ_V_FULL + i % NV), (i / NV) & 1) && clock64() - t0 < 2000000) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ----------------------------------
    if (lane == 0 && T_tiles > 0) {
      constexpr uint32_t idesc_s = instr_desc_f16(BM, BN, TcElem<T>::kFormat, 0, 0);
      constexpr uint32_t idesc_dq = instr_desc_f16(BM, D, TcElem<T>::kFormat, 0, 1);
      constexpr uint32_t kTile16 = C::kTile >> 4;
      const uint32_t q_lo = smem_desc_lo(smem + C::kQ, 0), do_lo = smem_desc_lo(smem + C::kDO, 0);
      const uint32_t k_k_lo = smem_desc_lo(smem + C::kK0, 0);            // K as K-major B operand
      const uint32_t k_mn_lo = smem_desc_lo(smem + C::kK0, BN * 128);     // K as MN-major B operand
      const uint32_t v_k_lo = smem_desc_lo(smem + C::kV0, 0);
      bool ok = mbar_wait(bar(DQ_QDO_FULL), 0, actx, 501);
      auto issue_s = [&](int sk, int phk) -> bool {  // S(t) = Q K(t)^T
        if (!mbar_wait(bar(DQ_K_FULL + sk), phk, actx, 502)) return false;
        tc_fence_after();
        const uint32_t b_lo = k_k_lo + sk * kTile16;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off16 = ((k / 4) * 128 * 128 + (k % 4) * 32) >> 4;
          mma_ss_lo(tmem + C::kColS, q_lo + off16, b_lo + off16, idesc_s, k > 0 ? 1u : 0u);
        }
        mma_commit(bar(DQ_S_FULL));
        return true;
      };
      auto issue_dp = [&](int sv, int phv, int buf) -> bool {  // dP(t) = dO V(t)^T into buffer `buf`
        if (!mbar_wait(bar(DQ_V_FULL + sv), phv, actx, 503)) return false;
        tc_fence_after();
        const uint32_t b_lo = v_k_lo + sv * kTile16;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off16 = ((k / 4) * 128 * 128 + (k % 4) * 32) >> 4;
          mma_ss_lo(tmem + C::kColDP + buf * 128, do_lo + off16, b_lo + off16, idesc_s,
                    k > 0 ? 1u : 0u);
        }
        mma_commit(bar(DQ_DP_FULL + buf));
        mma_commit(bar(DQ_V_FREE + sv));
        return true;
      };
      if (ok) ok = issue_s(0, 0);
      if (ok) ok = issue_dp(0, 0, 0);
      int sk = 0, phk = 0, sv = 0, phv = 0;   // ring positions / phases of tile t
      for (int t = 0; t < T_tiles && ok; ++t) {
        int nsk = sk + 1, nphk = phk, nsv = sv + 1, nphv = phv;
        if (nsk == NK) nsk = 0, nphk ^= 1;
        if (nsv == NV) nsv = 0, nphv ^= 1;
        const int buf = t & 1;
        if (t + 1 < T_tiles) {
          // S(t) has been pulled into registers: its TMEM tile can take S(t+1)
          ok = mbar_wait(bar(DQ_S_CONSUMED), t & 1, actx, 504);
          if (ok) ok = issue_s(nsk, nphk);
          if (ok) ok = issue_dp(nsv, nphv, buf ^ 1);
          if (!ok) break;
        }
        ok = mbar_wait(bar(DQ_DS_READY + buf), (t >> 1) & 1, actx, 505);
        if (!ok) break;
        tc_fence_after();
        const uint32_t b_lo = k_mn_lo + sk * kTile16;
        const uint32_t acc = t > 0 ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_ts_lo(tmem + C::kColDQ, tmem + C::kColDP + buf * 128 + (kk >> 1) * 32 + (kk & 1) * 8,
                    b_lo + ((kk * 16 * 128) >> 4), idesc_dq, kk > 0 ? 1u : acc);
        mma_commit(bar(DQ_K_FREE + sk));
        sk = nsk, phk = nphk, sv = nsv, phv = nphv;
      }
      if (ok) {
        mma_commit(bar(DQ_DONE));
        mbar_wait(bar(DQ_DONE), 0, actx, 506);
      }
    }
  } else {
    // ------------------------------ element-wise warps ---------------------------
    const int ew = warp - 2;
    const int slice = warp & 3, cg = ew >> 2;
    const int row = m0 + slice * 32 + lane;
    const uint32_t tlane = tmem + ((uint32_t)(slice * 32) << 16);
    const float qk_scale = p.sm_scale * kLog2e;
    const int64_t li = ((int64_t)b * p.H + h) * p.M + row;
    // rows past M get lse = +inf, which makes every P of the row exactly zero
    const float lse2 = row < p.M ? p.lse[li] * kLog2e : INFINITY;
    const float dlt = row < p.M ? p.delta[li] : 0.f;
    bool ok = true;

    for (int t = 0; t < T_tiles; ++t) {
      const int buf = t & 1, j = t_lo + t, n0 = j * BN;
      // ---- phase 1: P = exp2(S * scale - lse), kept in registers ----
      ok = mbar_wait(bar(DQ_S_FULL), t & 1, actx, 601);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[32];
      tmem_ld32(tlane + C::kColS + cg * 32, sr);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(DQ_S_CONSUMED));
      // Tiles away from every boundary (sequence end, causal diagonal, piecewise threshold) need no
      // masking; the others mask with one unsigned range check per element: key column c of this
      // thread's 32 columns is visible iff lo <= c < lo + width.
      bool interior = (n0 + BN <= p.N) && (!p.causal || n0 + BN - 1 <= m0 + p_seq);
      if (p.mode == 1) interior = interior && j >= jn;
      if (p.mode == 2) interior = interior && j < jf;
      float pv[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) pv[c] = fmaf(__uint_as_float(sr[c]), qk_scale, -lse2);
      if (!interior) {
        int lo = 0, hi = p.N - n0;
        if (p.causal) hi = min(hi, row + p_seq - n0 + 1);
        hi = min(hi - cg * 32, 32);
        if (p.mode) {
          const int cfar = row + p_seq - p.w - n0 - cg * 32;  // columns <= cfar are far pairs
          if (p.mode == 2) hi = min(hi, cfar + 1);
          else lo = max(lo, cfar + 1);
        }
        const unsigned width = (unsigned)max(hi - lo, 0);
#pragma unroll
        for (int c = 0; c < 32; ++c)
          pv[c] = ((unsigned)(c - lo) < width) ? pv[c] : -INFINITY;  // exp2(-inf) = 0
      }
#pragma unroll
      for (int c = 0; c < 32; ++c) pv[c] = ex2(pv[c]);
      // ---- phase 2: dS = P * (dP - delta), written over dP ----
      ok = mbar_wait(bar(DQ_DP_FULL + buf), (t >> 1) & 1, actx, 602);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      tmem_ld32(tlane + C::kColDP + buf * 128 + cg * 32, sr);
      tmem_wait_ld();
      uint32_t pk[16];
#pragma unroll
      for (int c = 0; c < 32; c += 2)
        pk[c >> 1] = TcElem<T>::pack(pv[c] * (__uint_as_float(sr[c]) - dlt),
                                     pv[c + 1] * (__uint_as_float(sr[c + 1]) - dlt));
      tmem_st16(tlane + C::kColDP + buf * 128 + cg * 32, pk);  // inside this thread's own columns
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(DQ_DS_READY + buf));
    }

    if (ok && T_tiles > 0) {
      ok = mbar_wait(bar(DQ_DONE), 0, actx, 603);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && cg < 2) {
      tc_fence_after();
      T *orow = row_ptr_mut<T>(p.dq, p.sdq, b, h, row);
      constexpr int COLS = D / 2;  // column groups 0 and 1 each store half a row
#pragma unroll
      for (int c = 0; c < COLS / 32; ++c) {
        uint32_t ov[32];
        const int col0 = cg * COLS + c * 32;
        if (T_tiles > 0) {
          tmem_ld32(tlane + C::kColDQ + col0, ov);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = 0u;
        }
        if (row < p.M) store_row32<T>(orow + col0, ov, p.sm_scale);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, C::kTmemCols);
  }
}

}  // namespace tc
}  // namespace fa
