// flash_attention forward on tcgen05, PERSISTENT form of flash_fwd_tc.cuh (head_dim 64 and 128,
// no piecewise branch): the same pipeline — 128 query rows, key tiles of 64, double-buffered
// scores in TMEM, two CTAs per SM — but a CTA does not end with its query tile.  The grid is two
// CTAs per SM; query tiles are handed out heaviest first by a global counter (fetched one item
// ahead by the producer thread and passed on through a four-slot ring in shared memory), and
// barriers, TMEM and the K / V rings keep counting across items: the first score products of the
// next item are issued while the softmax warps still write the previous item's output, and no
// launch, barrier set-up or TMEM allocation stands between two query tiles.  At sequence length
// 512 a one-tile CTA spends two thirds of its life outside the steady state; here that share is
// the reload of Q.
//
//   warp 0      TMA producer: Q per item, K and V tiles through two 2-stage rings
//   warp 1      MMA issuer (one thread): S = Q K^T into S0 | S1, O += P V with P read from TMEM
//   warps 2..5  softmax, one thread per query row (see flash_fwd_tc.cuh)
//
// Issue order:  S(g) | P V(g - 1) | S(g + 1) | P V(g) | ...   over the tiles g of ALL items of the
// CTA; the P V product that closes an item is issued after the first score product of the next
// item if that item's Q has landed by then, before it otherwise.
#pragma once

#include "flash_fwd_tc.cuh"

namespace fa {
namespace tc {

template <int D>
struct FwdPersistCfg {
  static constexpr int BM = 128, BN = 64;
  static constexpr int KSUB = D / 64;
  static constexpr int kQBytes = BM * D * 2;
  static constexpr int kKVBytes = BN * D * 2;
  static constexpr int kQ = 0;
  static constexpr int kK = kQBytes;                  // 2 stages
  static constexpr int kV = kK + 2 * kKVBytes;        // 2 stages
  static constexpr int kBars = kV + 2 * kKVBytes;     // 32 mbarriers
  static constexpr int kMisc = kBars + 32 * 8;        // tmem base, abort flag, ring of work items
  static constexpr int kTotal = kMisc + 32 + 1024;    // + slack to align the base to 1024 bytes
  static constexpr int kTmemCols = 256;               // S0 | S1 | O
  static constexpr int kColS0 = 0, kColS1 = 64, kColO = 128;
  static constexpr int kThreads = 192;
};

enum PersistBar { FP_ITEM_FULL = 0 /* ..3 */, FP_ITEM_FREE = 4 /* ..7 */, FP_Q_FULL = 8, FP_Q_FREE = 9,
                  FP_O_FREE = 10, FP_K_FULL = 12 /* 13 */, FP_K_FREE = 14, FP_V_FULL = 16, FP_V_FREE = 18,
                  FP_S_FULL = 20, FP_P_READY = 22, FP_PV_DONE = 24 /* 25 */ };

struct FwdPersistParams {
  FwdTcParams base;    // num_m_blocks = query tiles per (batch, head)
  unsigned *sched;     // work-item counter: zero at launch, put back to zero by the last fetch
  int num_items;       // query tiles x (batch, head) pairs
};

// One work item: 128 query rows of one (batch, head); E = key tiles of 64 it walks.
struct PersistItem {
  int m0, h, b, hk, E;
};

// The item with list position w (the order of grouped_cta(), heaviest causal tiles first).  Out
// of line on purpose: integer divisions, needed by every warp role, once per item.
static __device__ __noinline__ PersistItem persist_decode(const FwdTcParams &p, int w) {
  constexpr int BM = 128, BN = 64;
  const CtaCoord cta = grouped_cta((unsigned)w, p.num_m_blocks, p.B * p.H, p.group_size);
  PersistItem it;
  it.m0 = (p.num_m_blocks - 1 - cta.blk) * BM;
  it.b = cta.pair / p.H, it.h = cta.pair % p.H, it.hk = it.h / (p.H / p.Hk);
  int n_hi = p.N;
  if (p.causal) n_hi = min(n_hi, p.N - p.M + it.m0 + BM);
  it.E = n_hi > 0 ? (n_hi + BN - 1) / BN : 0;
  return it;
}

template <typename T, int D>
__global__ void __launch_bounds__(FwdPersistCfg<D>::kThreads, 2)
    flash_fwd_persist_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                const __grid_constant__ CUtensorMap map_k,
                                const __grid_constant__ CUtensorMap map_v,
                                const __grid_constant__ FwdPersistParams fp) {
  using C = FwdPersistCfg<D>;
  constexpr int BM = C::BM, BN = C::BN, KSUB = C::KSUB;
  const FwdTcParams &p = fp.base;
  extern __shared__ uint8_t smem_unaligned[];
  const uint32_t smem = (smem_u32(smem_unaligned) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_unaligned + (smem - smem_u32(smem_unaligned));
  auto bar = [&](int i) { return smem + C::kBars + i * 8; };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + C::kMisc);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + C::kMisc + 8);
  volatile int *item_ring = reinterpret_cast<volatile int *>(smem_gen + C::kMisc + 16);   // 4 slots
  const AbortCtx actx{abort_flag, p.status};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int p_seq = p.N - p.M;
  const int total = fp.num_items;
  auto decode = [&](int w) -> PersistItem { return persist_decode(p, w); };
  // the id of this CTA's `ic`-th item, as published by the producer thread (>= total: no more)
  auto ring_item = [&](int ic, int where) -> int {
    if (!mbar_wait(bar(FP_ITEM_FULL + (ic & 3)), (ic >> 2) & 1, actx, where)) return -1;
    return item_ring[ic & 3];
  };

  // a wait that ran out earlier (this launch or a previous one) poisons the device status word:
  // do no work until the host has read and cleared it
  if (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) return;

  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < 4; ++s) {
      mbar_init(bar(FP_ITEM_FULL + s), 1);
      mbar_init(bar(FP_ITEM_FREE + s), 5);   // the MMA thread and four softmax warps
    }
    mbar_init(bar(FP_Q_FULL), 1);
    mbar_init(bar(FP_Q_FREE), 1);
    mbar_init(bar(FP_O_FREE), 4);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(FP_K_FULL + s), 1);
      mbar_init(bar(FP_K_FREE + s), 1);
      mbar_init(bar(FP_V_FULL + s), 1);
      mbar_init(bar(FP_V_FREE + s), 1);
      mbar_init(bar(FP_S_FULL + s), 1);
      mbar_init(bar(FP_P_READY + s), 4);
      mbar_init(bar(FP_PV_DONE + s), 1);
    }
    fence_barrier_init();
    item_ring[0] = (int)blockIdx.x;          // the grid never exceeds the number of items
    mbar_arrive(bar(FP_ITEM_FULL + 0));
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
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
    if (lane == 0) {
      bool ok = true;
      uint32_t g = 0;             // K / V tiles requested so far: ring stage and phase
      uint32_t nk = 0, nv = 0;    // K / V loads requested (for the drain after an abort)
      int cnt = 0;                // items with keys so far: the phase of Q_FULL / Q_FREE
      int w = (int)blockIdx.x;
      for (int ic = 0; w < total && ok; ++ic) {
        // ask for the id of the next item now; it is passed on after this item's first loads
        const unsigned fetched = atomicAdd(fp.sched, 1u);
        const PersistItem it = decode(w);
        auto load_k = [&](int j) -> bool {
          const int st = g & 1, ph = (g >> 1) & 1;
          if (!mbar_wait(bar(FP_K_FREE + st), ph ^ 1, actx, 101)) return false;
          mbar_expect_tx(bar(FP_K_FULL + st), C::kKVBytes);
          for (int s = 0; s < KSUB; ++s)
            tma_load_4d(smem + C::kK + st * C::kKVBytes + s * BN * 128, &map_k, bar(FP_K_FULL + st), s * 64,
                        j * BN, it.hk, it.b);
          ++nk;
          return true;
        };
        auto load_v = [&](int j) -> bool {
          const int st = g & 1, ph = (g >> 1) & 1;
          if (!mbar_wait(bar(FP_V_FREE + st), ph ^ 1, actx, 102)) return false;
          mbar_expect_tx(bar(FP_V_FULL + st), C::kKVBytes);
          for (int s = 0; s < KSUB; ++s)
            tma_load_4d(smem + C::kV + st * C::kKVBytes + s * BN * 128, &map_v, bar(FP_V_FULL + st), s * 64,
                        j * BN, it.hk, it.b);
          ++nv;
          return true;
        };
        if (it.E > 0) {
          // Q: the last score product of the item before has read the tile
          if (cnt > 0) ok = mbar_wait(bar(FP_Q_FREE), (cnt - 1) & 1, actx, 103);
          if (!ok) break;
          mbar_expect_tx(bar(FP_Q_FULL), C::kQBytes);
          for (int s = 0; s < KSUB; ++s)
            tma_load_4d(smem + C::kQ + s * BM * 128, &map_q, bar(FP_Q_FULL), s * 64, it.m0, it.h, it.b);
          ++cnt;
          ok = load_k(0);
          if (ok) ok = load_v(0);
          ++g;
          if (!ok) break;
        }
        // pass the next item's id on, once every reader of the slot's previous content is done
        if (fetched == (unsigned)total - 1u) atomicExch(fp.sched, 0u);
        const int w_next = (int)gridDim.x + (int)fetched;
        if (ic + 1 >= 4)
          ok = mbar_wait(bar(FP_ITEM_FREE + ((ic + 1) & 3)), (((ic + 1) >> 2) - 1) & 1, actx, 104);
        if (!ok) break;
        item_ring[(ic + 1) & 3] = w_next;
        mbar_arrive(bar(FP_ITEM_FULL + ((ic + 1) & 3)));
        for (int j = 1; j < it.E && ok; ++j) {
          ok = load_k(j);
          if (ok) ok = load_v(j);
          ++g;
        }
        w = w_next;
      }
      if (!ok) {
        // let copies already in flight land before the CTA gives its shared memory back
        const long long t0 = clock64();
        if (cnt > 0)
          while (!mbar_try_wait(bar(FP_Q_FULL), (cnt - 1) & 1) && clock64() - t0 < 2000000) {}
        for (uint32_t i = nk > 2u ? nk - 2u : 0u; i < nk; ++i)
          while (!mbar_try_wait(bar(FP_K_FULL + (i & 1)), (i >> 1) & 1) && clock64() - t0 < 2000000) {}
        for (uint32_t i = nv > 2u ? nv - 2u : 0u; i < nv; ++i)
          while (!mbar_try_wait(bar(FP_V_FULL + (i & 1)), (i >> 1) & 1) && clock64() - t0 < 2000000) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = instr_desc_f16(BM, BN, TcElem<T>::kFormat, 0, 0);
      constexpr uint32_t idesc_pv = instr_desc_f16(BM, D, TcElem<T>::kFormat, 0, 1);
      const uint32_t q_lo = smem_desc_lo(smem + C::kQ, 0);
      const uint32_t k_lo = smem_desc_lo(smem + C::kK, 0);
      const uint32_t v_lo = smem_desc_lo(smem + C::kV, BN * 128);
      constexpr uint32_t kKV16 = C::kKVBytes >> 4;
      bool ok = true;
      uint32_t g = 0;              // tiles so far, over all items: buffer and phase of the per-tile barriers
      int cnt = 0;                 // items with keys so far: the phase of Q_FULL / O_FREE
      bool pend = false;           // P V of tile g - 1 is still to be issued
      bool pend_first = false;     // ... and it opens the accumulator of its item,
      int pend_item = 0;           // the pend_item-th with keys
      // O (+)= P(t) V(t), P from TMEM over S(t); `first`: the first product of item number `item`
      auto issue_pv = [&](uint32_t t, bool first, int item) -> bool {
        const int st = t & 1, ph = (t >> 1) & 1;
        if (!mbar_wait(bar(FP_V_FULL + st), ph, actx, 203)) return false;
        // the softmax warps must have read the accumulator of the item before out
        if (first && item > 1 && !mbar_wait(bar(FP_O_FREE), (item - 2) & 1, actx, 207)) return false;
        if (!mbar_wait(bar(FP_P_READY + st), ph, actx, 204)) return false;
        tc_fence_after();
        const uint32_t b_lo = v_lo + st * kKV16;
        const uint32_t a_col = tmem + (st ? C::kColS1 : C::kColS0);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_ts_lo(tmem + C::kColO, a_col + kk * 8, b_lo + ((kk * 16 * 128) >> 4), idesc_pv,
                    (kk > 0 || !first) ? 1u : 0u);
        mma_commit(bar(FP_PV_DONE + st));
        mma_commit(bar(FP_V_FREE + st));
        return true;
      };
      for (int ic = 0; ok; ++ic) {
        const int w = ring_item(ic, 201);
        if (w < 0) {
          ok = false;
          break;
        }
        mbar_arrive(bar(FP_ITEM_FREE + (ic & 3)));
        if (w >= total) break;
        const PersistItem it = decode(w);
        if (it.E == 0) continue;
        // Q of this item: if it has not landed yet, the product that closes the item before goes first
        if (pend && !mbar_try_wait(bar(FP_Q_FULL), cnt & 1)) {
          ok = issue_pv(g - 1, pend_first, pend_item);
          pend = false;
          if (!ok) break;
        }
        ok = mbar_wait(bar(FP_Q_FULL), cnt & 1, actx, 201);
        if (!ok) break;
        ++cnt;
        for (int e = 0; e < it.E && ok; ++e, ++g) {
          const int st = g & 1, ph = (g >> 1) & 1;
          ok = mbar_wait(bar(FP_K_FULL + st), ph, actx, 202);
          if (!ok) break;
          tc_fence_after();
          const uint32_t b_lo = k_lo + st * kKV16;
          const uint32_t d_col = tmem + (st ? C::kColS1 : C::kColS0);
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            mma_ss_lo(d_col, q_lo + (((k / 4) * BM * 128 + (k % 4) * 32) >> 4),
                      b_lo + (((k / 4) * BN * 128 + (k % 4) * 32) >> 4), idesc_s, k > 0 ? 1u : 0u);
          mma_commit(bar(FP_S_FULL + st));
          mma_commit(bar(FP_K_FREE + st));
          if (e == it.E - 1) mma_commit(bar(FP_Q_FREE));
          if (pend) {
            ok = issue_pv(g - 1, pend_first, pend_item);
            if (!ok) break;
          }
          pend = true, pend_first = (e == 0), pend_item = cnt;
        }
      }
      if (ok && pend) ok = issue_pv(g - 1, pend_first, pend_item);
      // the last commit's arrive must land before this CTA's shared memory is given back
      if (ok && g > 0) mbar_wait(bar(FP_V_FREE + ((g - 1) & 1)), ((g - 1) >> 1) & 1, actx, 205);
    }
  } else {
    // ------------------------------ softmax warps -----------------------------
    const int slice = warp & 3;
    const int row_in_tile = slice * 32 + lane;
    const uint32_t tlane = tmem + ((uint32_t)(slice * 32) << 16);
    const float qk_scale = p.sm_scale * kLog2e;
    bool ok = true;
    uint32_t g = 0;   // tiles so far, over all items

    for (int ic = 0; ok; ++ic) {
      const int w = ring_item(ic, 300);
      ok = __all_sync(0xffffffffu, w >= 0);
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(FP_ITEM_FREE + (ic & 3)));
      if (w >= total) break;
      const PersistItem it = decode(w);
      const int m0 = it.m0, row = m0 + row_in_tile;
      float m_used = -INFINITY, l = 0.f;

      for (int e = 0; e < it.E; ++e, ++g) {
        const int st = g & 1, ph = (g >> 1) & 1, n0 = e * BN;
        ok = mbar_wait(bar(FP_S_FULL + st), ph, actx, 301);
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

        // valid columns of this row are [0, hi)
        if ((n0 + BN > p.N) || (p.causal && (n0 + BN - 1 > m0 + p_seq))) {
          int hi = p.N - n0;
          if (p.causal) hi = min(hi, row + p_seq - n0 + 1);
#pragma unroll
          for (int c = 0; c < BN; ++c)
            if (c >= hi) s[c] = -INFINITY;
        }
        // four independent chains (three-input max: two new elements per instruction)
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
          // the accumulator is rescaled only when a row maximum has moved by more than 2^8
          const bool need = (m_new - m_used) * qk_scale > 8.f;
          if (__any_sync(0xffffffffu, need)) {
            const uint32_t pj = g - 1;
            ok = mbar_wait(bar(FP_PV_DONE + (pj & 1)), (pj >> 1) & 1, actx, 302);
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
        if (lane == 0) mbar_arrive(bar(FP_P_READY + st));  // one arrival per warp
      }
      if (!ok) break;

      // write-out: O / l -> global, log-normaliser.  The accumulator is handed back as soon as it
      // is in registers, so that the next item's first P V can start.
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T *orow = row_ptr_mut<T>(p.o, p.so, it.b, it.h, row);
      if (it.E > 0) {
        const uint32_t lj = g - 1;
        ok = mbar_wait(bar(FP_PV_DONE + (lj & 1)), (lj >> 1) & 1, actx, 303);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
      }
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t ov[2][32];
        if (it.E > 0) {
          tmem_ld32(tlane + C::kColO + c * 64, ov[0]);
          tmem_ld32(tlane + C::kColO + c * 64 + 32, ov[1]);
          tmem_wait_ld();
          if (c == D / 64 - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(FP_O_FREE));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[0][i] = ov[1][i] = 0u;
        }
        if (row < p.M) {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = TcElem<T>::pack(__uint_as_float(ov[hh][8 * i + 0]) * inv, __uint_as_float(ov[hh][8 * i + 1]) * inv);
              v.y = TcElem<T>::pack(__uint_as_float(ov[hh][8 * i + 2]) * inv, __uint_as_float(ov[hh][8 * i + 3]) * inv);
              v.z = TcElem<T>::pack(__uint_as_float(ov[hh][8 * i + 4]) * inv, __uint_as_float(ov[hh][8 * i + 5]) * inv);
              v.w = TcElem<T>::pack(__uint_as_float(ov[hh][8 * i + 6]) * inv, __uint_as_float(ov[hh][8 * i + 7]) * inv);
              *reinterpret_cast<uint4 *>(orow + c * 64 + hh * 32 + i * 8) = v;
            }
        }
      }
      if (row < p.M) {
        const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
        p.lse[((int64_t)it.b * p.H + it.h) * p.M + row] =
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
