// total_attention on tcgen05 (head_dim 64 and 128): tot[b, h, n] = sum over queries m of
// P[m, n] = exp(sm_scale * q_m . k_n - lse_m), the column sums of the attention matrix recomputed
// from the saved log-normaliser.
//
// One CTA per 128 keys of one (batch, query head) walks the query tiles that see them:
//   warp 0       TMA producer: K once, Q tiles through a two-stage ring
//   warp 1       MMA issuer (one thread): S^T = K Q^T (128 keys x 128 queries, fp32) into one of two
//                TMEM buffers, so the product of tile t + 1 runs under the exponentials of tile t
//   warps 2..17  element-wise, one thread per (key row, 32 query columns): tcgen05.ld of its slice,
//                exp2(S^T * scale - lse), masked, summed into a register that lives for the whole walk
//   warp 18      stages -lse * log2(e) of every tile in shared memory (broadcast reads)
// At the end the four column groups of a key row are added through shared memory and the 128
// sums are written.  One exponential per score bounds the kernel (the ex2 unit, not the tensor
// pipe).
#pragma once

#include "../attn_params.cuh"
#include "tc_common.cuh"

namespace fa {
namespace tc {

struct TotalTcParams {
  const float *lse;
  float *total;
  int B, H, Hk, M, N;
  int causal;
  float sm_scale;
  int *status;
};

template <int D>
struct TotalTcCfg {
  static constexpr int BM = 128, BN = 128, NQ = 2;
  static constexpr int KSUB = D / 64;
  static constexpr int kTile = 128 * D * 2;
  static constexpr int kK = 0;
  static constexpr int kQ0 = kTile;
  static constexpr int kBars = kQ0 + NQ * kTile;
  static constexpr int kMisc = kBars + 16 * 8;           // tmem base, abort flag
  static constexpr int kLse = kMisc + 16;                // 2 x 128 floats
  static constexpr int kSums = kLse + 2 * 128 * 4;       // 4 x 128 floats
  static constexpr int kTotal = kSums + 4 * 128 * 4 + 1024;
  static constexpr int kTmemCols = 256;
  static constexpr int kEwWarps = 16;
  static constexpr int kThreads = (2 + kEwWarps + 1) * 32;   // 608
};

enum TotalBar { TB_K_FULL = 0, TB_Q_FULL = 1, TB_Q_FREE = 3, TB_S_FULL = 5, TB_S_FREE = 7,
                TB_LSE_FULL = 9, TB_LSE_FREE = 11 };

template <typename T, int D>
__global__ void __launch_bounds__(TotalTcCfg<D>::kThreads, 1)
    total_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                              const __grid_constant__ CUtensorMap map_k, const TotalTcParams p) {
  using C = TotalTcCfg<D>;
  constexpr int BM = C::BM, BN = C::BN, KSUB = C::KSUB, NQ = C::NQ;
  extern __shared__ uint8_t smem_unaligned[];
  const uint32_t smem = (smem_u32(smem_unaligned) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_unaligned + (smem - smem_u32(smem_unaligned));
  auto bar = [&](int i) { return smem + C::kBars + i * 8; };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + C::kMisc);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + C::kMisc + 8);
  const AbortCtx actx{abort_flag, p.status};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * BN;
  const int b = blockIdx.y / p.H, h = blockIdx.y % p.H;
  const int hk = h / (p.H / p.Hk);
  const int p_seq = p.N - p.M;
  const int num_m_tiles = (p.M + BM - 1) / BM;
  int mt_lo = 0;
  if (p.causal) mt_lo = max(0, n0 - p_seq) / BM;
  const int T_tiles = max(0, num_m_tiles - mt_lo);

  if (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) return;

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar(TB_K_FULL), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(TB_Q_FULL + s), 1);
      mbar_init(bar(TB_Q_FREE + s), 1);
      mbar_init(bar(TB_S_FULL + s), 1);
      mbar_init(bar(TB_S_FREE + s), C::kEwWarps);
      mbar_init(bar(TB_LSE_FULL + s), 1);
      mbar_init(bar(TB_LSE_FREE + s), C::kEwWarps);
    }
    fence_barrier_init();
    if (T_tiles > 0) {
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_q);
      mbar_expect_tx(bar(TB_K_FULL), C::kTile);
      for (int s = 0; s < KSUB; ++s)
        tma_load_4d(smem + C::kK + s * BN * 128, &map_k, bar(TB_K_FULL), s * 64, n0, hk, b);
      mbar_expect_tx(bar(TB_Q_FULL), C::kTile);
      for (int s = 0; s < KSUB; ++s)
        tma_load_4d(smem + C::kQ0 + s * BM * 128, &map_q, bar(TB_Q_FULL), s * 64, mt_lo * BM, h, b);
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
      int issued = 1;
      bool ok = true;
      for (int t = 1; t < T_tiles; ++t) {
        const int sq = t % NQ, ph = (t / NQ) & 1;
        ok = mbar_wait(bar(TB_Q_FREE + sq), ph ^ 1, actx, 1011);
        if (!ok) break;
        mbar_expect_tx(bar(TB_Q_FULL + sq), C::kTile);
        for (int s = 0; s < KSUB; ++s)
          tma_load_4d(smem + C::kQ0 + sq * C::kTile + s * BM * 128, &map_q, bar(TB_Q_FULL + sq),
                      s * 64, (mt_lo + t) * BM, h, b);
        ++issued;
      }
      if (!ok) {
        // let copies already in flight land before the CTA gives its shared memory back
        const long long t0 = clock64();
        for (int i = max(0, issued - NQ); i < issued; ++i)
          while (!mbar_try_wait(bar(TB_Q_FULL + i % NQ), (i / NQ) & 1) && clock64() - t0 < 2000000) {}
        while (!mbar_try_wait(bar(TB_K_FULL), 0) && clock64() - t0 < 2000000) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    if (lane == 0 && T_tiles > 0) {
      constexpr uint32_t idesc_s = instr_desc_f16(BN, BM, TcElem<T>::kFormat, 0, 0);
      constexpr uint32_t kTile16 = C::kTile >> 4;
      const uint32_t k_lo = smem_desc_lo(smem + C::kK, 0);
      const uint32_t q_lo = smem_desc_lo(smem + C::kQ0, 0);
      bool ok = mbar_wait(bar(TB_K_FULL), 0, actx, 1021);
      for (int t = 0; t < T_tiles && ok; ++t) {
        const int sq = t % NQ, phq = (t / NQ) & 1, sb = t & 1, phs = (t >> 1) & 1;
        ok = mbar_wait(bar(TB_Q_FULL + sq), phq, actx, 1022);
        // the buffer still holds S^T of two tiles ago until every element-wise warp has read it
        if (ok) ok = mbar_wait(bar(TB_S_FREE + sb), phs ^ 1, actx, 1023);
        if (!ok) break;
        tc_fence_after();
        const uint32_t b_lo = q_lo + sq * kTile16;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off16 = ((k / 4) * 128 * 128 + (k % 4) * 32) >> 4;
          mma_ss_lo(tmem + sb * 128, k_lo + off16, b_lo + off16, idesc_s, k > 0 ? 1u : 0u);
        }
        mma_commit(bar(TB_S_FULL + sb));
        mma_commit(bar(TB_Q_FREE + sq));
      }
      // the last commits' arrives must land before this CTA's shared memory is given back
      if (ok) mbar_wait(bar(TB_Q_FREE + (T_tiles - 1) % NQ), ((T_tiles - 1) / NQ) & 1, actx, 1024);
    }
  } else if (warp == 2 + C::kEwWarps) {
    // ------------------------------ statistics warp ----------------------------
    // -lse * log2(e) of the 128 queries of a tile, two buffers; queries past M get -inf (P = 0)
    bool ok = true;
    for (int t = 0; t < T_tiles; ++t) {
      const int sb = t & 1, phs = (t >> 1) & 1;
      const int m = (mt_lo + t) * BM + lane * 4;
      const int64_t li = ((int64_t)b * p.H + h) * p.M + m;
      float l[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) l[j] = m + j < p.M ? -p.lse[li + j] * kLog2e : -INFINITY;
      ok = mbar_wait(bar(TB_LSE_FREE + sb), phs ^ 1, actx, 1031);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      reinterpret_cast<float4 *>(smem_gen + C::kLse)[sb * 32 + lane] = make_float4(l[0], l[1], l[2], l[3]);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(TB_LSE_FULL + sb));
    }
  } else {
    // ------------------------------ element-wise warps --------------------------
    const int ew = warp - 2;
    const int slice = warp & 3, cg = ew >> 2;       // TMEM lane slice, 32-column group
    const int row = slice * 32 + lane;              // key row of this thread
    const int key = n0 + row;
    const uint32_t tlane = tmem + ((uint32_t)(slice * 32) << 16);
    const float qk_scale = p.sm_scale * kLog2e;
    float sum = 0.f;
    bool ok = true;
    for (int t = 0; t < T_tiles; ++t) {
      const int sb = t & 1, phs = (t >> 1) & 1;
      const int m0 = (mt_lo + t) * BM;
      ok = mbar_wait(bar(TB_LSE_FULL + sb), phs, actx, 1041);
      if (ok) ok = mbar_wait(bar(TB_S_FULL + sb), phs, actx, 1042);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[32];
      tmem_ld32(tlane + sb * 128 + cg * 32, sr);
      // while the load is in flight: query column c of this thread's 32 is visible iff
      // cmin <= c (causal); tiles below the diagonal need no mask at all
      const bool interior = !p.causal || m0 + p_seq >= n0 + BN - 1;
      const int cmin = p.causal ? key - p_seq - m0 - cg * 32 : 0;
      const float4 *lse_s = reinterpret_cast<const float4 *>(smem_gen + C::kLse) + sb * 32 + cg * 8;
      float pv[32];
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(TB_S_FREE + sb));
      const uint64_t scale2 = f2_pack(qk_scale, qk_scale);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 l4 = lse_s[i];
        f2_unpack(f2_fma(f2_pack(__uint_as_float(sr[4 * i]), __uint_as_float(sr[4 * i + 1])), scale2,
                         f2_pack(l4.x, l4.y)),
                  pv[4 * i], pv[4 * i + 1]);
        f2_unpack(f2_fma(f2_pack(__uint_as_float(sr[4 * i + 2]), __uint_as_float(sr[4 * i + 3])), scale2,
                         f2_pack(l4.z, l4.w)),
                  pv[4 * i + 2], pv[4 * i + 3]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(TB_LSE_FREE + sb));
      if (!interior) {
#pragma unroll
        for (int c = 0; c < 32; ++c) pv[c] = (c >= cmin) ? pv[c] : -INFINITY;   // exp2(-inf) = 0
      }
      float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 32; c += 4) {
        part[0] += ex2(pv[c]);
        part[1] += ex2(pv[c + 1]);
        part[2] += ex2(pv[c + 2]);
        part[3] += ex2(pv[c + 3]);
      }
      sum += (part[0] + part[1]) + (part[2] + part[3]);
    }
    // the four column groups of a key row meet in shared memory
    float *sums = reinterpret_cast<float *>(smem_gen + C::kSums);
    sums[cg * 128 + row] = ok ? sum : 0.f;
    asm volatile("bar.sync 1, %0;\n" ::"n"(C::kEwWarps * 32) : "memory");
    if (cg == 0 && ok && key < p.N)
      p.total[((int64_t)b * p.H + h) * p.N + key] =
          (sums[row] + sums[128 + row]) + (sums[256 + row] + sums[384 + row]);
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
