// flash_attention backward on tcgen05 for head_dim 64 and 128: the dQ kernel
// and the dK/dV kernel.  No global atomics; P is recomputed from the saved
// log-normaliser, so the softmax warps need no row statistics and two warps
// share each TMEM lane slice, splitting the tile's columns between them.
//
// Both kernels use the same skeleton as the forward kernel:
//   warp 0      TMA producer
//   warp 1      MMA issuer (one thread)
//   warps 2..9  element-wise stage: P = exp2(S*scale - L), dS = P*(dP - delta),
//               written back to TMEM as 16-bit A operands of the next GEMMs
// with S / dP double-buffered in TMEM so the tensor pipe computes tile j+1
// while the element-wise warps work on tile j.
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
  int *status;
};

// ===========================================================================
// dQ: one CTA per 128 query rows, key tiles of 64
// ===========================================================================
template <int D>
struct DqTcCfg {
  static constexpr int BM = 128, BN = 64, NSTAGE = 3;
  static constexpr int KSUB = D / 64;
  static constexpr int kQBytes = BM * D * 2;
  static constexpr int kKVBytes = BN * D * 2;
  static constexpr int kQ = 0;
  static constexpr int kDO = kQBytes;
  static constexpr int kStage0 = 2 * kQBytes;           // stage: K | V
  static constexpr int kStageBytes = 2 * kKVBytes;
  static constexpr int kBars = kStage0 + NSTAGE * kStageBytes;
  static constexpr int kMisc = kBars + 16 * 8;
  static constexpr int kTotal = kMisc + 16 + 1024;
  static constexpr int kTmemCols = 512;
  // S0 | S1 | dP0 | dP1 | dQ
  static constexpr int kColS = 0, kColDP = 128, kColDQ = 256;
  static constexpr int kThreads = 320;
};

enum DqBar { DQ_QDO_FULL = 0, DQ_KV_FULL = 1, DQ_KV_FREE = 4, DQ_SDP_FULL = 7, DQ_DS_READY = 9,
             DQ_DONE = 11 };

template <typename T, int D>
__global__ void __launch_bounds__(DqTcCfg<D>::kThreads, 1)
    flash_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                           const __grid_constant__ CUtensorMap map_do,
                           const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, const BwdTcParams p) {
  using C = DqTcCfg<D>;
  constexpr int BM = C::BM, BN = C::BN, KSUB = C::KSUB, NS = C::NSTAGE;
  extern __shared__ uint8_t smem_unaligned[];
  const uint32_t smem = (smem_u32(smem_unaligned) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_unaligned + (smem - smem_u32(smem_unaligned));
  auto bar = [&](int i) { return smem + C::kBars + i * 8; };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + C::kMisc);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + C::kMisc + 8);
  const AbortCtx actx{abort_flag, p.status};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mb = gridDim.x - 1 - blockIdx.x;
  const int b = blockIdx.y / p.H, h = blockIdx.y % p.H;
  const int hk = h / (p.H / p.Hk);
  const int m0 = mb * BM;
  const int p_seq = p.N - p.M;
  int n_hi = p.N;
  if (p.causal) n_hi = min(n_hi, p_seq + m0 + BM);
  const int T_tiles = n_hi > 0 ? (n_hi + BN - 1) / BN : 0;

  if (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) return;

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar(DQ_QDO_FULL), 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar(DQ_KV_FULL + s), 1);
      mbar_init(bar(DQ_KV_FREE + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(DQ_SDP_FULL + s), 1);
      mbar_init(bar(DQ_DS_READY + s), 8);
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
    if (lane == 0 && T_tiles > 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_do);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      mbar_expect_tx(bar(DQ_QDO_FULL), 2 * C::kQBytes);
      for (int s = 0; s < KSUB; ++s) {
        tma_load_4d(smem + C::kQ + s * BM * 128, &map_q, bar(DQ_QDO_FULL), s * 64, m0, h, b);
        tma_load_4d(smem + C::kDO + s * BM * 128, &map_do, bar(DQ_QDO_FULL), s * 64, m0, h, b);
      }
      int issued = 0;
      bool ok = true;
      for (int j = 0; j < T_tiles; ++j) {
        const int st = j % NS, ph = (j / NS) & 1, n0 = j * BN;
        ok = mbar_wait(bar(DQ_KV_FREE + st), ph ^ 1, actx, 401);
        if (!ok) break;
        mbar_expect_tx(bar(DQ_KV_FULL + st), C::kStageBytes);
        const uint32_t base = smem + C::kStage0 + st * C::kStageBytes;
        for (int s = 0; s < KSUB; ++s) {
          tma_load_4d(base + s * BN * 128, &map_k, bar(DQ_KV_FULL + st), s * 64, n0, hk, b);
          tma_load_4d(base + C::kKVBytes + s * BN * 128, &map_v, bar(DQ_KV_FULL + st), s * 64, n0,
                      hk, b);
        }
        ++issued;
      }
      if (!ok) {
        const long long t0 = clock64();
        for (int i = max(0, issued - NS); i < issued; ++i)
          while (!mbar_try_wait(bar(DQ_KV_FULL + i % NS), (i / NS) & 1) &&
                 clock64() - t0 < 2000000) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && T_tiles > 0) {
      constexpr uint32_t idesc_s = instr_desc_f16(BM, BN, TcElem<T>::kFormat, 0, 0);
      constexpr uint32_t idesc_dq = instr_desc_f16(BM, D, TcElem<T>::kFormat, 0, 1);
      bool ok = mbar_wait(bar(DQ_QDO_FULL), 0, actx, 501);
      auto issue_sdp = [&](int j) -> bool {
        const int st = j % NS, ph = (j / NS) & 1, buf = j & 1;
        if (!mbar_wait(bar(DQ_KV_FULL + st), ph, actx, 502)) return false;
        tc_fence_after();
        const uint32_t kbase = smem + C::kStage0 + st * C::kStageBytes;
        const uint32_t vbase = kbase + C::kKVBytes;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off_a = (k / 4) * BM * 128 + (k % 4) * 32;
          const uint32_t off_b = (k / 4) * BN * 128 + (k % 4) * 32;
          mma_ss(tmem + C::kColS + buf * 64, smem_desc_sw128(smem + C::kQ + off_a, 0, 1024),
                 smem_desc_sw128(kbase + off_b, 0, 1024), idesc_s, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off_a = (k / 4) * BM * 128 + (k % 4) * 32;
          const uint32_t off_b = (k / 4) * BN * 128 + (k % 4) * 32;
          mma_ss(tmem + C::kColDP + buf * 64, smem_desc_sw128(smem + C::kDO + off_a, 0, 1024),
                 smem_desc_sw128(vbase + off_b, 0, 1024), idesc_s, k > 0 ? 1u : 0u);
        }
        mma_commit(bar(DQ_SDP_FULL + buf));
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int j = 0; j < T_tiles && ok; ++j) {
        if (j + 1 < T_tiles) ok = issue_sdp(j + 1);
        if (!ok) break;
        const int st = j % NS, buf = j & 1;
        ok = mbar_wait(bar(DQ_DS_READY + buf), (j >> 1) & 1, actx, 503);
        if (!ok) break;
        tc_fence_after();
        const uint32_t kbase = smem + C::kStage0 + st * C::kStageBytes;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_ts(tmem + C::kColDQ, tmem + C::kColDP + buf * 64 + (kk >> 1) * 32 + (kk & 1) * 8,
                 smem_desc_sw128(kbase + kk * 16 * 128, BN * 128, 1024), idesc_dq,
                 (j > 0 || kk > 0) ? 1u : 0u);
        mma_commit(bar(DQ_KV_FREE + st));
      }
      if (ok) {
        mma_commit(bar(DQ_DONE));
        mbar_wait(bar(DQ_DONE), 0, actx, 504);
      }
    }
  } else {
    const int ew = warp - 2;                  // 0..7
    const int slice = warp & 3, half = ew >> 2;
    const int row = m0 + slice * 32 + lane;
    const uint32_t tlane = tmem + ((uint32_t)(slice * 32) << 16);
    const float qk_scale = p.sm_scale * kLog2e;
    const int64_t li = ((int64_t)b * p.H + h) * p.M + row;
    // rows past M get lse = +inf, which makes every P of the row exactly zero
    const float lse2 = row < p.M ? p.lse[li] * kLog2e : INFINITY;
    const float dlt = row < p.M ? p.delta[li] : 0.f;
    bool ok = true;

    for (int j = 0; j < T_tiles; ++j) {
      const int buf = j & 1, n0 = j * BN;
      ok = mbar_wait(bar(DQ_SDP_FULL + buf), (j >> 1) & 1, actx, 601);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[32], dr[32];
      tmem_ld32(tlane + C::kColS + buf * 64 + half * 32, sr);
      tmem_ld32(tlane + C::kColDP + buf * 64 + half * 32, dr);
      tmem_wait_ld();
      const bool need_mask = (n0 + BN > p.N) || (p.causal && (n0 + BN - 1 > m0 + p_seq));
      int limit = BN;
      if (need_mask) {
        limit = p.N - n0;
        if (p.causal) limit = min(limit, row + p_seq - n0 + 1);
      }
      limit -= half * 32;
      uint32_t pk[16];
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        float p0 = ex2(fmaf(__uint_as_float(sr[c]), qk_scale, -lse2));
        float p1 = ex2(fmaf(__uint_as_float(sr[c + 1]), qk_scale, -lse2));
        if (c >= limit) p0 = 0.f;
        if (c + 1 >= limit) p1 = 0.f;
        const float d0 = p0 * (__uint_as_float(dr[c]) - dlt);
        const float d1 = p1 * (__uint_as_float(dr[c + 1]) - dlt);
        pk[c >> 1] = TcElem<T>::pack(d0, d1);
      }
      tmem_st16(tlane + C::kColDP + buf * 64 + half * 32, pk);  // inside this thread's own columns
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(DQ_DS_READY + buf));  // one arrival per warp
    }

    if (ok && T_tiles > 0) {
      ok = mbar_wait(bar(DQ_DONE), 0, actx, 602);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      T *orow = row_ptr_mut<T>(p.dq, p.sdq, b, h, row);
      constexpr int COLS = D / 2;  // this thread's half of the row
#pragma unroll
      for (int c = 0; c < COLS / 32; ++c) {
        uint32_t ov[32];
        const int col0 = half * COLS + c * 32;
        if (T_tiles > 0) {
          tmem_ld32(tlane + C::kColDQ + col0, ov);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = 0u;
        }
        if (row < p.M) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = TcElem<T>::pack(__uint_as_float(ov[8 * i + 0]) * p.sm_scale, __uint_as_float(ov[8 * i + 1]) * p.sm_scale);
            v.y = TcElem<T>::pack(__uint_as_float(ov[8 * i + 2]) * p.sm_scale, __uint_as_float(ov[8 * i + 3]) * p.sm_scale);
            v.z = TcElem<T>::pack(__uint_as_float(ov[8 * i + 4]) * p.sm_scale, __uint_as_float(ov[8 * i + 5]) * p.sm_scale);
            v.w = TcElem<T>::pack(__uint_as_float(ov[8 * i + 6]) * p.sm_scale, __uint_as_float(ov[8 * i + 7]) * p.sm_scale);
            *reinterpret_cast<uint4 *>(orow + col0 + i * 8) = v;
          }
        }
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
// dK / dV: one CTA per 128 keys, query tiles of 64, loops over the query
// heads of a GQA group
// ===========================================================================
template <int D>
struct DkdvTcCfg {
  static constexpr int BM = 64, BN = 128, NSTAGE = 3;
  static constexpr int KSUB = D / 64;
  static constexpr int kKVBytes = BN * D * 2;
  static constexpr int kQBytes = BM * D * 2;
  static constexpr int kK = 0;
  static constexpr int kV = kKVBytes;
  static constexpr int kStage0 = 2 * kKVBytes;           // stage: Q | dO | lse[BM] | delta[BM]
  static constexpr int kStLse = 2 * kQBytes;
  static constexpr int kStDelta = kStLse + BM * 4;
  static constexpr int kStageBytes = 2 * kQBytes + 1024;  // keeps every stage 1024-byte aligned
  static constexpr int kBars = kStage0 + NSTAGE * kStageBytes;
  static constexpr int kMisc = kBars + 16 * 8;
  static constexpr int kTotal = kMisc + 16 + 1024;
  static constexpr int kTmemCols = 512;
  // S^T0 | S^T1 | dP^T0 | dP^T1 | dK | dV
  static constexpr int kColS = 0, kColDP = 128, kColDK = 256, kColDV = 256 + D;
  static constexpr int kThreads = 320;
};

enum DkdvBar { KV_KV_FULL = 0, KV_QDO_FULL = 1, KV_QDO_FREE = 4, KV_SDP_FULL = 7, KV_PDS_READY = 9,
               KV_DONE = 11 };

template <typename T, int D>
__global__ void __launch_bounds__(DkdvTcCfg<D>::kThreads, 1)
    flash_bwd_dkdv_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                             const __grid_constant__ CUtensorMap map_do,
                             const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, const BwdTcParams p) {
  using C = DkdvTcCfg<D>;
  constexpr int BM = C::BM, BN = C::BN, KSUB = C::KSUB, NS = C::NSTAGE;
  extern __shared__ uint8_t smem_unaligned[];
  const uint32_t smem = (smem_u32(smem_unaligned) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_unaligned + (smem - smem_u32(smem_unaligned));
  auto bar = [&](int i) { return smem + C::kBars + i * 8; };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + C::kMisc);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + C::kMisc + 8);
  const AbortCtx actx{abort_flag, p.status};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nb = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = p.H / p.Hk;
  const int n0 = nb * BN;
  const int p_seq = p.N - p.M;
  const int num_m_tiles = (p.M + BM - 1) / BM;
  int mt_lo = 0;
  if (p.causal) mt_lo = max(0, n0 - p_seq) / BM;
  const int tiles = max(0, num_m_tiles - mt_lo);
  const int T_tiles = tiles * G;

  if (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) return;

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar(KV_KV_FULL), 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar(KV_QDO_FULL + s), 2);  // the TMA transaction + the warp that stored lse / delta
      mbar_init(bar(KV_QDO_FREE + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(KV_SDP_FULL + s), 1);
      mbar_init(bar(KV_PDS_READY + s), 8);
    }
    mbar_init(bar(KV_DONE), 1);
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
    // whole warp: lane 0 drives TMA, all lanes stage lse / delta of the tile
    if (T_tiles > 0) {
      if (lane == 0) {
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_do);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        mbar_expect_tx(bar(KV_KV_FULL), 2 * C::kKVBytes);
        for (int s = 0; s < KSUB; ++s) {
          tma_load_4d(smem + C::kK + s * BN * 128, &map_k, bar(KV_KV_FULL), s * 64, n0, hk, b);
          tma_load_4d(smem + C::kV + s * BN * 128, &map_v, bar(KV_KV_FULL), s * 64, n0, hk, b);
        }
      }
      int issued = 0;
      bool ok = true;
      for (int t = 0; t < T_tiles; ++t) {
        const int st = t % NS, ph = (t / NS) & 1;
        const int h = hk * G + t / tiles, m0 = (mt_lo + t % tiles) * BM;
        ok = mbar_wait(bar(KV_QDO_FREE + st), ph ^ 1, actx, 701);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint32_t base = smem + C::kStage0 + st * C::kStageBytes;
        if (lane == 0) {
          mbar_expect_tx(bar(KV_QDO_FULL + st), 2 * C::kQBytes);
          for (int s = 0; s < KSUB; ++s) {
            tma_load_4d(base + s * BM * 128, &map_q, bar(KV_QDO_FULL + st), s * 64, m0, h, b);
            tma_load_4d(base + C::kQBytes + s * BM * 128, &map_do, bar(KV_QDO_FULL + st), s * 64,
                        m0, h, b);
          }
        }
        float *lse_s = reinterpret_cast<float *>(smem_gen + C::kStage0 + st * C::kStageBytes + C::kStLse);
        float *dlt_s = reinterpret_cast<float *>(smem_gen + C::kStage0 + st * C::kStageBytes + C::kStDelta);
        const int64_t lbase = ((int64_t)b * p.H + h) * p.M;
#pragma unroll
        for (int i = 0; i < BM / 32; ++i) {
          const int qm = m0 + lane + i * 32;
          // queries past M get lse = +inf, which makes their P exactly zero
          lse_s[lane + i * 32] = qm < p.M ? p.lse[lbase + qm] * kLog2e : INFINITY;
          dlt_s[lane + i * 32] = qm < p.M ? p.delta[lbase + qm] : 0.f;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(KV_QDO_FULL + st));  // after every lane stored its lse / delta
        ++issued;
      }
      if (!ok && lane == 0) {
        const long long t0 = clock64();
        for (int i = max(0, issued - NS); i < issued; ++i)
          while (!mbar_try_wait(bar(KV_QDO_FULL + i % NS), (i / NS) & 1) &&
                 clock64() - t0 < 2000000) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && T_tiles > 0) {
      constexpr uint32_t idesc_s = instr_desc_f16(BN, BM, TcElem<T>::kFormat, 0, 0);  // 128 x 64
      constexpr uint32_t idesc_acc = instr_desc_f16(BN, D, TcElem<T>::kFormat, 0, 1); // 128 x D
      bool ok = mbar_wait(bar(KV_KV_FULL), 0, actx, 801);
      auto issue_sdp = [&](int t) -> bool {
        const int st = t % NS, ph = (t / NS) & 1, buf = t & 1;
        if (!mbar_wait(bar(KV_QDO_FULL + st), ph, actx, 802)) return false;
        tc_fence_after();
        const uint32_t qbase = smem + C::kStage0 + st * C::kStageBytes;
        const uint32_t dobase = qbase + C::kQBytes;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off_a = (k / 4) * BN * 128 + (k % 4) * 32;
          const uint32_t off_b = (k / 4) * BM * 128 + (k % 4) * 32;
          mma_ss(tmem + C::kColS + buf * 64, smem_desc_sw128(smem + C::kK + off_a, 0, 1024),
                 smem_desc_sw128(qbase + off_b, 0, 1024), idesc_s, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off_a = (k / 4) * BN * 128 + (k % 4) * 32;
          const uint32_t off_b = (k / 4) * BM * 128 + (k % 4) * 32;
          mma_ss(tmem + C::kColDP + buf * 64, smem_desc_sw128(smem + C::kV + off_a, 0, 1024),
                 smem_desc_sw128(dobase + off_b, 0, 1024), idesc_s, k > 0 ? 1u : 0u);
        }
        mma_commit(bar(KV_SDP_FULL + buf));
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int t = 0; t < T_tiles && ok; ++t) {
        if (t + 1 < T_tiles) ok = issue_sdp(t + 1);
        if (!ok) break;
        const int st = t % NS, buf = t & 1;
        ok = mbar_wait(bar(KV_PDS_READY + buf), (t >> 1) & 1, actx, 803);
        if (!ok) break;
        tc_fence_after();
        const uint32_t qbase = smem + C::kStage0 + st * C::kStageBytes;
        const uint32_t dobase = qbase + C::kQBytes;
#pragma unroll
        for (int kk = 0; kk < BM / 16; ++kk)
          mma_ts(tmem + C::kColDV, tmem + C::kColS + buf * 64 + (kk >> 1) * 32 + (kk & 1) * 8,
                 smem_desc_sw128(dobase + kk * 16 * 128, BM * 128, 1024), idesc_acc,
                 (t > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < BM / 16; ++kk)
          mma_ts(tmem + C::kColDK, tmem + C::kColDP + buf * 64 + (kk >> 1) * 32 + (kk & 1) * 8,
                 smem_desc_sw128(qbase + kk * 16 * 128, BM * 128, 1024), idesc_acc,
                 (t > 0 || kk > 0) ? 1u : 0u);
        mma_commit(bar(KV_QDO_FREE + st));
      }
      if (ok) {
        mma_commit(bar(KV_DONE));
        mbar_wait(bar(KV_DONE), 0, actx, 804);
      }
    }
  } else {
    const int ew = warp - 2;
    const int slice = warp & 3, half = ew >> 2;
    const int key = n0 + slice * 32 + lane;
    const uint32_t tlane = tmem + ((uint32_t)(slice * 32) << 16);
    const float qk_scale = p.sm_scale * kLog2e;
    const bool key_ok = key < p.N;
    bool ok = true;

    for (int t = 0; t < T_tiles; ++t) {
      const int st = t % NS, buf = t & 1;
      const int m0 = (mt_lo + t % tiles) * BM;
      ok = mbar_wait(bar(KV_SDP_FULL + buf), (t >> 1) & 1, actx, 901);
      // acquire the producer lanes' lse / delta stores of this stage (complete long ago)
      ok = ok && mbar_wait(bar(KV_QDO_FULL + st), (t / NS) & 1, actx, 903);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[32], dr[32];
      tmem_ld32(tlane + C::kColS + buf * 64 + half * 32, sr);
      tmem_ld32(tlane + C::kColDP + buf * 64 + half * 32, dr);
      tmem_wait_ld();
      const float *lse_s = reinterpret_cast<const float *>(smem_gen + C::kStage0 + st * C::kStageBytes + C::kStLse) + half * 32;
      const float *dlt_s = reinterpret_cast<const float *>(smem_gen + C::kStage0 + st * C::kStageBytes + C::kStDelta) + half * 32;
      // first visible query column of this key row inside the tile (causal), in this half
      int cmin = 0;
      if (p.causal) cmin = key - p_seq - m0 - half * 32;
      if (!key_ok) cmin = 64;
      uint32_t pp[16], ds[16];
#pragma unroll
      for (int c4 = 0; c4 < 8; ++c4) {
        const float4 l4 = *reinterpret_cast<const float4 *>(lse_s + c4 * 4);
        const float4 d4 = *reinterpret_cast<const float4 *>(dlt_s + c4 * 4);
        const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
        const float dv4[4] = {d4.x, d4.y, d4.z, d4.w};
        float pv[4], dsv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c = c4 * 4 + i;
          float pe = ex2(fmaf(__uint_as_float(sr[c]), qk_scale, -lv[i]));
          if (c < cmin) pe = 0.f;
          pv[i] = pe;
          dsv[i] = pe * (__uint_as_float(dr[c]) - dv4[i]);
        }
        pp[c4 * 2] = TcElem<T>::pack(pv[0], pv[1]);
        pp[c4 * 2 + 1] = TcElem<T>::pack(pv[2], pv[3]);
        ds[c4 * 2] = TcElem<T>::pack(dsv[0], dsv[1]);
        ds[c4 * 2 + 1] = TcElem<T>::pack(dsv[2], dsv[3]);
      }
      tmem_st16(tlane + C::kColS + buf * 64 + half * 32, pp);
      tmem_st16(tlane + C::kColDP + buf * 64 + half * 32, ds);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(KV_PDS_READY + buf));  // one arrival per warp
    }

    if (ok && T_tiles > 0) {
      ok = mbar_wait(bar(KV_DONE), 0, actx, 902);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      constexpr int COLS = D / 2;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
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
          if (key_ok) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = TcElem<T>::pack(__uint_as_float(ov[8 * i + 0]) * scale, __uint_as_float(ov[8 * i + 1]) * scale);
              v.y = TcElem<T>::pack(__uint_as_float(ov[8 * i + 2]) * scale, __uint_as_float(ov[8 * i + 3]) * scale);
              v.z = TcElem<T>::pack(__uint_as_float(ov[8 * i + 4]) * scale, __uint_as_float(ov[8 * i + 5]) * scale);
              v.w = TcElem<T>::pack(__uint_as_float(ov[8 * i + 6]) * scale, __uint_as_float(ov[8 * i + 7]) * scale);
              *reinterpret_cast<uint4 *>(orow + col0 + i * 8) = v;
            }
          }
        }
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
