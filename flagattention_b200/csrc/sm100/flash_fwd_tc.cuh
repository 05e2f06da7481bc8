// flash_attention forward on the 5th-generation tensor cores (tcgen05) for
// head_dim 64 and 128.
//
// One CTA owns 128 query rows of one (batch, head) and walks the visible keys
// in tiles of 64.  Warp roles:
//   warp 0      TMA producer: Q once, then K and V tiles through two 2-stage rings
//   warp 1      MMA issuer (one thread): S = Q K^T into a double-buffered TMEM
//               tile, O += P V with P read back from TMEM
//   warps 2..5  softmax, one thread per query row: tcgen05.ld of its S row,
//               running max / sum, P written over S in TMEM as 16-bit pairs,
//               lazy rescale of the O accumulator, final normalise + store
// S(j+1) is issued before P(j) V(j), so the tensor pipe computes the next
// scores while the softmax warps work on the current tile; two CTAs per SM
// (256 of the 512 TMEM columns each) overlap each other's remaining gaps.
#pragma once

#include "../attn_params.cuh"
#include "tc_common.cuh"

namespace fa {
namespace tc {

struct FwdTcParams {
  void *o;
  float *lse;
  Strides so;
  int B, H, Hk, M, N;
  int causal;
  float sm_scale;
  int w;  // piecewise distance threshold (PW kernels only)
  int *status;
  int num_m_blocks, group_size;  // launch order, see grouped_cta()
};

template <int D>
struct FwdTcCfg {
  static constexpr int BM = 128, BN = 64;
  static constexpr int KSUB = D / 64;                 // 64-column (128-byte) sub-tiles per row
  static constexpr int kQBytes = BM * D * 2;
  static constexpr int kKVBytes = BN * D * 2;
  static constexpr int kQ = 0;
  static constexpr int kK = kQBytes;                  // 2 stages
  static constexpr int kV = kK + 2 * kKVBytes;        // 2 stages
  static constexpr int kBars = kV + 2 * kKVBytes;     // 16 mbarriers
  static constexpr int kMisc = kBars + 16 * 8;        // tmem base, abort flag
  static constexpr int kTotal = kMisc + 16 + 1024;    // + slack to align the base to 1024 bytes
  static constexpr int kTmemCols = 256;               // S0 | S1 | O, rounded to a power of two
  static constexpr int kColS0 = 0, kColS1 = 64, kColO = 128;
  static constexpr int kThreads = 192;
};

enum FwdBar { Q_FULL = 0, K_FULL = 1, K_FREE = 3, V_FULL = 5, V_FREE = 7, S_FULL = 9, P_READY = 11,
              PV_DONE = 13, Q_FREE = 15 };

// PW = piecewise_attention: the score of (m, n) is q2.k2 when (m + N - M) - n >= w, else q.k.
// The key tiles of a CTA are then walked as a list of (tile, branch) entries: first every tile
// that holds a far pair with (q2, k2), then every tile that holds a near pair with (q, k).  A
// tile that straddles the threshold appears twice, each time masked to its own branch, so each
// entry is an ordinary flash tile and the online softmax simply sees a few more tiles.  Q is
// re-loaded once, at the switch from the far to the near entries.
template <typename T, int D, bool PW>
__global__ void __launch_bounds__(FwdTcCfg<D>::kThreads, 2)
    flash_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                        const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v,
                        const __grid_constant__ CUtensorMap map_q2,
                        const __grid_constant__ CUtensorMap map_k2, const FwdTcParams p) {
  using C = FwdTcCfg<D>;
  constexpr int BM = C::BM, BN = C::BN, KSUB = C::KSUB;
  extern __shared__ uint8_t smem_unaligned[];
  const uint32_t smem = (smem_u32(smem_unaligned) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_unaligned + (smem - smem_u32(smem_unaligned));
  auto bar = [&](int i) { return smem + C::kBars + i * 8; };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + C::kMisc);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + C::kMisc + 8);
  const AbortCtx actx{abort_flag, p.status};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const CtaCoord cta = grouped_cta(blockIdx.x, p.num_m_blocks, p.B * p.H, p.group_size);
  const int mb = p.num_m_blocks - 1 - cta.blk;  // heaviest causal tiles first
  const int b = cta.pair / p.H, h = cta.pair % p.H;
  const int hk = h / (p.H / p.Hk);
  const int m0 = mb * BM;
  const int p_seq = p.N - p.M;
  int n_hi = p.N;
  if (p.causal) n_hi = min(n_hi, p_seq + m0 + BM);
  const int T_tiles = n_hi > 0 ? (n_hi + BN - 1) / BN : 0;
  // piecewise schedule: tiles [0, jf) are entirely far, [jn, T) entirely near, [jf, jn) straddle
  int jf = 0, jn = 0;
  if (PW) {
    const int x = m0 + p_seq - (BN - 1) - p.w, y = m0 + BM - 1 + p_seq - p.w;
    jf = x < 0 ? 0 : min(T_tiles, x / BN + 1);
    jn = y < 0 ? 0 : min(T_tiles, y / BN + 1);
  }
  const int E2 = jn;                    // entries of the far branch: tiles 0 .. jn-1
  const int E = E2 + (T_tiles - jf);    // then the near branch: tiles jf .. T-1
  const bool reload_q = PW && E2 > 0 && E2 < E;

  // a wait that ran out earlier (this launch or a previous one) poisons the device status word:
  // do no work until the host has read and cleared it
  if (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) return;

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar(Q_FULL), 1);
    mbar_init(bar(Q_FREE), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(K_FULL + s), 1);
      mbar_init(bar(K_FREE + s), 1);
      mbar_init(bar(V_FULL + s), 1);
      mbar_init(bar(V_FREE + s), 1);
      mbar_init(bar(S_FULL + s), 1);
      mbar_init(bar(P_READY + s), 4);
      mbar_init(bar(PV_DONE + s), 1);
    }
    fence_barrier_init();
    // The loads of Q and of the first K / V tile go out right here, before the TMEM allocation
    // and the CTA-wide barrier below, so that their latency runs under the rest of the set-up.
    if (E > 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      const bool far0 = PW && E2 > 0;
      const int n00 = ((PW && E2 == 0) ? jf : 0) * BN;
      mbar_expect_tx(bar(Q_FULL), C::kQBytes);
      for (int s = 0; s < KSUB; ++s)
        tma_load_4d(smem + C::kQ + s * BM * 128, far0 ? &map_q2 : &map_q, bar(Q_FULL), s * 64, m0, h, b);
      mbar_expect_tx(bar(K_FULL), C::kKVBytes);
      for (int s = 0; s < KSUB; ++s)
        tma_load_4d(smem + C::kK + s * BN * 128, far0 ? &map_k2 : &map_k, bar(K_FULL), s * 64, n00, hk, b);
      mbar_expect_tx(bar(V_FULL), C::kKVBytes);
      for (int s = 0; s < KSUB; ++s)
        tma_load_4d(smem + C::kV + s * BN * 128, &map_v, bar(V_FULL), s * 64, n00, hk, b);
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
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && E > 0) {
      // Q and tile 0 were requested during set-up
      int issued_k = 1, issued_v = 1;
      bool ok = true;
      for (int e = 1; e < E && ok; ++e) {
        const bool far = PW && e < E2;
        const int j = (PW && e >= E2) ? jf + (e - E2) : e;
        const int st = e & 1, ph = (e >> 1) & 1, n0 = j * BN;
        if (reload_q && e == E2) {
          // every S of the far branch has been computed: swap q2 for q
          ok = mbar_wait(bar(Q_FREE), 0, actx, 103);
          if (!ok) break;
          mbar_expect_tx(bar(Q_FULL), C::kQBytes);
          for (int s = 0; s < KSUB; ++s)
            tma_load_4d(smem + C::kQ + s * BM * 128, &map_q, bar(Q_FULL), s * 64, m0, h, b);
        }
        ok = mbar_wait(bar(K_FREE + st), ph ^ 1, actx, 101);
        if (!ok) break;
        mbar_expect_tx(bar(K_FULL + st), C::kKVBytes);
        for (int s = 0; s < KSUB; ++s)
          tma_load_4d(smem + C::kK + st * C::kKVBytes + s * BN * 128, far ? &map_k2 : &map_k,
                      bar(K_FULL + st), s * 64, n0, hk, b);
        ++issued_k;
        ok = mbar_wait(bar(V_FREE + st), ph ^ 1, actx, 102);
        if (!ok) break;
        mbar_expect_tx(bar(V_FULL + st), C::kKVBytes);
        for (int s = 0; s < KSUB; ++s)
          tma_load_4d(smem + C::kV + st * C::kKVBytes + s * BN * 128, &map_v, bar(V_FULL + st),
                      s * 64, n0, hk, b);
        ++issued_v;
      }
      if (!ok) {
        // let copies already in flight land before the CTA gives its shared memory back
        const long long t0 = clock64();
        for (int i = max(0, issued_k - 2); i < issued_k; ++i)
          while (!mbar_try_wait(bar(K_FULL + (i & 1)), (i >> 1) & 1) && clock64() - t0 < 2000000) {}
        for (int i = max(0, issued_v - 2); i < issued_v; ++i)
          while (!mbar_try_wait(bar(V_FULL + (i & 1)), (i >> 1) & 1) && clock64() - t0 < 2000000) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0 && E > 0) {
      constexpr uint32_t idesc_s = instr_desc_f16(BM, BN, TcElem<T>::kFormat, 0, 0);
      constexpr uint32_t idesc_pv = instr_desc_f16(BM, D, TcElem<T>::kFormat, 0, 1);
      // descriptor low words: the issuing thread only adds a constant per MMA
      const uint32_t q_lo = smem_desc_lo(smem + C::kQ, 0);
      const uint32_t k_lo = smem_desc_lo(smem + C::kK, 0);
      const uint32_t v_lo = smem_desc_lo(smem + C::kV, BN * 128);
      constexpr uint32_t kKV16 = C::kKVBytes >> 4;
      bool ok = mbar_wait(bar(Q_FULL), 0, actx, 201);
      auto issue_pv = [&](int i) -> bool {
        const int st = i & 1, ph = (i >> 1) & 1;
        if (!mbar_wait(bar(V_FULL + st), ph, actx, 203)) return false;
        if (!mbar_wait(bar(P_READY + st), ph, actx, 204)) return false;
        tc_fence_after();
        const uint32_t b_lo = v_lo + st * kKV16;
        const uint32_t a_col = tmem + (st ? C::kColS1 : C::kColS0);
        const uint32_t acc = i > 0 ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_ts_lo(tmem + C::kColO, a_col + kk * 8, b_lo + ((kk * 16 * 128) >> 4), idesc_pv,
                    kk > 0 ? 1u : acc);
        mma_commit(bar(PV_DONE + st));
        mma_commit(bar(V_FREE + st));
        return true;
      };
      for (int e = 0; e < E && ok; ++e) {
        const int st = e & 1, ph = (e >> 1) & 1;
        if (reload_q && e == E2) ok = mbar_wait(bar(Q_FULL), 1, actx, 206);
        if (ok) ok = mbar_wait(bar(K_FULL + st), ph, actx, 202);
        if (!ok) break;
        tc_fence_after();
        const uint32_t b_lo = k_lo + st * kKV16;
        const uint32_t d_col = tmem + (st ? C::kColS1 : C::kColS0);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          mma_ss_lo(d_col, q_lo + (((k / 4) * BM * 128 + (k % 4) * 32) >> 4),
                    b_lo + (((k / 4) * BN * 128 + (k % 4) * 32) >> 4), idesc_s, k > 0 ? 1u : 0u);
        mma_commit(bar(S_FULL + st));
        mma_commit(bar(K_FREE + st));
        if (reload_q && e == E2 - 1) mma_commit(bar(Q_FREE));
        if (e >= 1) ok = issue_pv(e - 1);
      }
      if (ok) ok = issue_pv(E - 1);
      // the last commit's arrive must land before this CTA's shared memory is given back
      if (ok) mbar_wait(bar(V_FREE + ((E - 1) & 1)), ((E - 1) >> 1) & 1, actx, 205);
    }
  } else {
    // ------------------------------ softmax warps -----------------------------
    const int slice = warp & 3;
    const int row_in_tile = slice * 32 + lane;
    const int row = m0 + row_in_tile;
    const uint32_t tlane = tmem + ((uint32_t)(slice * 32) << 16);
    const float qk_scale = p.sm_scale * kLog2e;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;

    for (int e = 0; e < E; ++e) {
      const bool far = PW && e < E2;
      const int j = (PW && e >= E2) ? jf + (e - E2) : e;
      const int st = e & 1, ph = (e >> 1) & 1, n0 = j * BN;
      ok = mbar_wait(bar(S_FULL + st), ph, actx, 301);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t scol = tlane + (st ? C::kColS1 : C::kColS0);
      uint32_t raw[2][32];
      tmem_ld32(scol, raw[0]);
      tmem_ld32(scol + 32, raw[1]);
      tmem_wait_ld();
      float s[BN];
#pragma unroll
      for (int c = 0; c < BN; ++c) s[c] = __uint_as_float(raw[c >> 5][c & 31]);

      // valid columns of this row are [lo, hi)
      bool need_mask = (n0 + BN > p.N) || (p.causal && (n0 + BN - 1 > m0 + p_seq));
      int lo = 0, hi = BN;
      if (need_mask) {
        hi = p.N - n0;
        if (p.causal) hi = min(hi, row + p_seq - n0 + 1);
      }
      if (PW) {
        const int cfar = row + p_seq - p.w - n0;  // columns <= cfar are far pairs of this row
        if (far && j >= jf) hi = min(hi, cfar + 1), need_mask = true;
        if (!far && j < jn) lo = max(lo, cfar + 1), need_mask = true;
      }
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < BN; ++c)
          if (c < lo || c >= hi) s[c] = -INFINITY;
      }
      // four independent chains instead of one 64-deep dependency chain
      // (three-input max: two new elements per instruction)
      float mx4[4] = {fmaxf(s[0], s[1]), fmaxf(s[2], s[3]), fmaxf(s[4], s[5]), fmaxf(s[6], s[7])};
#pragma unroll
      for (int c = 8; c < BN; c += 8) {
        mx4[0] = max3(mx4[0], s[c], s[c + 1]);
        mx4[1] = max3(mx4[1], s[c + 2], s[c + 3]);
        mx4[2] = max3(mx4[2], s[c + 4], s[c + 5]);
        mx4[3] = max3(mx4[3], s[c + 6], s[c + 7]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m_used, mx);
      if (e == 0) {
        m_used = m_new;
      } else {
        const bool need = (m_new - m_used) * qk_scale > 8.f;
        if (__any_sync(0xffffffffu, need)) {
          const int pj = e - 1;
          ok = mbar_wait(bar(PV_DONE + (pj & 1)), (pj >> 1) & 1, actx, 302);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          float alpha = 1.f;
          if (need) {
            alpha = ex2((m_used - m_new) * qk_scale);
            l *= alpha;
            m_used = m_new;
          }
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t ov[32];
            tmem_ld32(tlane + C::kColO + c * 32, ov);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st32(tlane + C::kColO + c * 32, ov);
          }
          tmem_wait_st();
        }
      }
      const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
      const float neg_ms = -m_eff * qk_scale;
      uint32_t pk[BN / 2];
      // packed fp32 pairs: one FMA and one add per two elements
      const uint64_t scale2 = f2_pack(qk_scale, qk_scale), shift2 = f2_pack(neg_ms, neg_ms);
      uint64_t rs2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int c = 0; c < BN; c += 2) {
        float x0, x1;
        f2_unpack(f2_fma(f2_pack(s[c], s[c + 1]), scale2, shift2), x0, x1);
        const float p0 = ex2(x0), p1 = ex2(x1);
        rs2[(c >> 1) & 3] = f2_add(rs2[(c >> 1) & 3], f2_pack(p0, p1));
        pk[c >> 1] = TcElem<T>::pack(p0, p1);
      }
      {
        float a0, a1;
        f2_unpack(f2_add(f2_add(rs2[0], rs2[1]), f2_add(rs2[2], rs2[3])), a0, a1);
        l += a0 + a1;
      }
      tmem_st32(scol, reinterpret_cast<const uint32_t(&)[32]>(pk));
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(P_READY + st));  // one arrival per warp
    }

    // epilogue: O / l -> global, log-normaliser
    if (ok && E > 0) {
      const int lj = E - 1;
      ok = mbar_wait(bar(PV_DONE + (lj & 1)), (lj >> 1) & 1, actx, 303);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T *orow = row_ptr_mut<T>(p.o, p.so, b, h, row);
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t ov[32];
        if (E > 0) {
          tmem_ld32(tlane + C::kColO + c * 32, ov);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = 0u;
        }
        if (row < p.M) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = TcElem<T>::pack(__uint_as_float(ov[8 * i + 0]) * inv, __uint_as_float(ov[8 * i + 1]) * inv);
            v.y = TcElem<T>::pack(__uint_as_float(ov[8 * i + 2]) * inv, __uint_as_float(ov[8 * i + 3]) * inv);
            v.z = TcElem<T>::pack(__uint_as_float(ov[8 * i + 4]) * inv, __uint_as_float(ov[8 * i + 5]) * inv);
            v.w = TcElem<T>::pack(__uint_as_float(ov[8 * i + 6]) * inv, __uint_as_float(ov[8 * i + 7]) * inv);
            *reinterpret_cast<uint4 *>(orow + c * 32 + i * 8) = v;
          }
        }
      }
      if (row < p.M) {
        const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
        p.lse[((int64_t)b * p.H + h) * p.M + row] =
            l > 0.f ? m_eff * p.sm_scale + logf(l) : -INFINITY;
      }
    }
  }

  // ------------------------------ teardown -----------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, C::kTmemCols);
  }
}

}  // namespace tc
}  // namespace fa
