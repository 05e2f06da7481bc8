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
// TMEM (512 columns):  S^T, then dP^T (128) | dQ (D), P^T over its first 64 columns | dK | dV.
//   The two score products of a tile share one 128-column region: dP^T is issued as soon as the
//   element-wise warps hold S^T in registers, S^T of the next tile as soon as they hold dP^T.
//   P^T goes back to TMEM as packed 16-bit pairs and is the TMEM A operand of dV += P^T dO: no
//   shared-memory store, no async-proxy fence, and P^T never competes with dS^T for a buffer.
//   At head_dim 128 all 512 columns are taken, so P^T(t+1) borrows the first 64 columns of dQ:
//   they are free between the read-out of dQ(t)'s first two quarters and the issue of dQ(t+1)
//   (head_dim 64 has columns to spare and keeps P^T apart).
// Shared memory:       K, V resident | Q ring | dO ring | one 16-bit 128 x 128 tile "PD" | dQ staging.
//   PD holds dS^T of a tile: the K-major A operand of dK += dS^T Q and, under a second descriptor,
//   the MN-major A operand of dQ = dS K.
//
// Issue order (tensor pipe):  dP^T(t) | dV(t) | S^T(t+1) | dQ(t) | dK(t)
// Element-wise order:         phase 1 (t) | phase 2 (t)
//   phase 1: P^T = exp2(S^T * scale - L) -> TMEM     phase 2: dS^T = P^T * (dP^T - delta) -> PD
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
  static constexpr int kMisc = kBars + 32 * 8;         // tmem base, abort flag, ring of work items
  static constexpr int kStats = kMisc + 32;            // -lse*log2e [128] | -delta [128] of a tile
  static constexpr int kTotal = kStats + 2 * 128 * 4 + 1024;
  static constexpr int kTmemCols = 512;
  static constexpr int NH = 1;                         // parts dQ of a tile is produced in
  // head_dim 128: dQ at 128..255 with P^T over 128..191; head_dim 64: P^T at 128..191, dQ at 192..255
  static constexpr bool kPAliasesDQ = (D == 128);
  static constexpr int kColA = 0, kColP = 128, kColQ = (D == 128 ? 128 : 192), kColDK = 256, kColDV = 256 + D;
  static_assert(kPdBytes >= kTile, "dK is staged in the P^T / dS^T tile");
  static_assert(kTotal <= 232448, "shared memory budget");
};

enum FusedBar { FB_KV_FULL = 0, FB_Q_FULL = 1, FB_Q_FREE = 3, FB_DO_FULL = 5, FB_DO_FREE = 7,
                FB_S_FULL = 9, FB_S_LOADED = 10, FB_DP_FULL = 11, FB_DP_LOADED = 12,
                FB_PT_FULL = 13, FB_PT_FREE = 14, FB_DS_FULL = 15, FB_DS_FREE = 16,
                FB_DQ_FULL = 17, FB_DQ_FREE = 18, FB_DONE = 19, FB_LSE_FULL = 20, FB_DLT_FULL = 21,
                FB_V_FULL = 22, FB_DV_STAGED = 23, FB_DK_STAGED = 24, FB_PD_STORED = 25,
                FB_ITEM_FULL = 26 /* .. 29 */, FB_DQ_HALF = 30 };

struct FusedBwdParams {
  BwdTcParams base;   // base.mode: 0 = flash_attention, 3 = piecewise_attention (both branches)
  float *dq_acc;      // (B, H, Mpad / 128, D / 4, 128, 4) fp32, zeroed before the launch
  float *dq_acc2;     // piecewise: the same for dq2 (far branch); dq_acc then holds dq1
  void *dk2;          // piecewise: dk of the far branch (base.dk: near branch), same strides
  int Mpad;           // M rounded up to a multiple of 128
  unsigned *sched;    // work-item counter; zero at launch and at exit (see the kernel)
  int num_items;      // key blocks x (batch, kv head) pairs
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
// it gives its shared memory back)
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

// One work item = one block of 128 keys of one (batch, kv head) pair: its query-tile range.
// Under piecewise_attention a block is walked twice, back to back by the same CTA: first the
// tiles that hold a near pair (mode 1: q1, k1 -> dq1, dk1), then the tiles that hold a far pair
// (mode 2: q2, k2 -> dq2, dk2).  V stays in shared memory and dV keeps accumulating in TMEM
// across the two walks (`first` / `last`: the walk opens / closes the block), so dV is rounded
// once and V and dO of a straddling tile are not fetched by a second launch.
struct FusedItem {
  int n0, hk, b, mt_lo, mt_hi, T_tiles;
  int mode;          // 0 flash, 1 near walk, 2 far walk
  bool first, last;  // of its key block's walks (those with tiles)
};

// PERSISTENT: the grid is one CTA per SM.  A CTA works through items (key block, pair) in the
// order of grouped_cta(): its first item is its block index, every further one comes from a
// global counter (`sched`, zero at launch), fetched one item ahead by the producer thread and
// handed to the other warps through a four-slot ring in shared memory (items whose key block no
// query sees are skipped by the producer: the launcher zero-fills their dk / dv rows).  Barriers, TMEM and the
// operand rings are set up once per CTA and their phases simply keep counting across items, so
// the tail of an item overlaps the head of the next: while the element-wise warps convert dV and
// dK of item i (dV into the shared memory of V, dK into the P^T / dS^T tile, both dead by then)
// and the copy engine stores them, the producer already loads Q, dO, K and V of item i + 1 and the
// tensor pipe computes its first score tile.
template <typename T, int D>
__global__ void __launch_bounds__(kFusedThreads, 1)
    flash_bwd_fused_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                              const __grid_constant__ CUtensorMap map_do,
                              const __grid_constant__ CUtensorMap map_k,
                              const __grid_constant__ CUtensorMap map_v,
                              const __grid_constant__ CUtensorMap map_dk,
                              const __grid_constant__ CUtensorMap map_dv,
                              const __grid_constant__ CUtensorMap map_q2,    // far walk (piecewise); else = map_q ...
                              const __grid_constant__ CUtensorMap map_k2,
                              const __grid_constant__ CUtensorMap map_dk2, const FusedBwdParams fp) {
  using C = FusedBwdCfg<D>;
  constexpr int BM = C::BM, BN = C::BN, KSUB = C::KSUB, NQ = C::NQ, NDO = C::NDO;
  const BwdTcParams &p = fp.base;
  extern __shared__ uint8_t smem_unaligned[];
  const uint32_t smem = (smem_u32(smem_unaligned) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_unaligned + (smem - smem_u32(smem_unaligned));
  auto bar = [&](int i) { return smem + C::kBars + i * 8; };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + C::kMisc);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + C::kMisc + 8);
  volatile int *item_ring = reinterpret_cast<volatile int *>(smem_gen + C::kMisc + 16);   // 4 slots
  const AbortCtx actx{abort_flag, p.status};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.H / p.Hk;
  const int p_seq = p.N - p.M;
  const int num_m_tiles = (p.M + BM - 1) / BM;
  const int total = fp.num_items;

  // query tiles [mt_lo, mt_hi) that the key block starting at n0 walks
  auto tile_range = [&](int n0, int mode, int &mt_lo, int &mt_hi) {
    mt_lo = 0;
    if (p.causal) mt_lo = max(0, n0 - p_seq) / BM;
    mt_hi = num_m_tiles;
    if (mode == 1) {  // query tiles that hold a near pair
      const int lim = p.w - p_seq + n0 + BN - 1;
      mt_hi = min(mt_hi, lim <= 0 ? 0 : (lim + BM - 1) / BM);
    } else if (mode == 2) {  // query tiles that hold a far pair
      const int lim = p.w - p_seq + n0 - (BM - 1);
      mt_lo = max(mt_lo, lim <= 0 ? 0 : (lim + BM - 1) / BM);
    }
  };
  // Walk ids: flash_attention has one walk per key block (id = position of the block in the order
  // of grouped_cta()); piecewise_attention two (id = 2 * position + walk: 0 near, 1 far).
  const bool pw = (p.mode == 3);
  const int end_id = pw ? 2 * total : total;
  auto decode = [&](int id) -> FusedItem {
    const int unit = pw ? (id >> 1) : id;
    const CtaCoord cta = grouped_cta((unsigned)unit, p.num_blocks, p.B * p.Hk, p.group_size);
    FusedItem it;
    it.n0 = cta.blk * BN, it.hk = cta.pair % p.Hk, it.b = cta.pair / p.Hk;
    it.mode = pw ? 1 + (id & 1) : p.mode;
    tile_range(it.n0, it.mode, it.mt_lo, it.mt_hi);
    it.T_tiles = max(0, it.mt_hi - it.mt_lo) * G;
    it.first = it.last = true;
    if (pw) {
      int lo, hi;
      tile_range(it.n0, 3 - it.mode, lo, hi);
      const bool other = hi > lo;            // the block's other walk has tiles too
      if (it.mode == 1) it.last = !other;
      else it.first = !other;
    }
    return it;
  };
  // the id of this CTA's `ic`-th item, as published by the producer thread (>= end_id: no more)
  auto ring_item = [&](int ic, int where) -> int {
    if (!mbar_wait(bar(FB_ITEM_FULL + (ic & 3)), (ic >> 2) & 1, actx, where)) return -1;
    return item_ring[ic & 3];
  };

  if (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) return;

  // First walk with at least one tile of key block `unit` or, if it has none, of the next block
  // handed out: blocks past the end of the list (>= total) end the CTA (returns end_id).  Every id beyond the CTA's first comes from the global counter; whoever makes the
  // last fetch of the launch (every CTA ends on exactly one fetch past the end, so there are `total`
  // in all) puts the counter back to zero for the next launch.
  auto first_walk_of = [&](int unit) -> int {
    while (unit < total) {
      if (!pw) {
        if (decode(unit).T_tiles > 0) return unit;
      } else {
        if (decode(2 * unit).T_tiles > 0) return 2 * unit;
        if (decode(2 * unit + 1).T_tiles > 0) return 2 * unit + 1;
      }
      const unsigned fetched = atomicAdd(fp.sched, 1u);
      if (fetched == (unsigned)total - 1u) atomicExch(fp.sched, 0u);
      unit = (int)gridDim.x + (int)fetched;
    }
    return end_id;
  };
  int w_first = 0;   // producer thread only
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
    mbar_init(bar(FB_DQ_HALF), 4);
    mbar_init(bar(FB_DONE), 1);
    mbar_init(bar(FB_LSE_FULL), 1);
    mbar_init(bar(FB_DLT_FULL), 1);
    mbar_init(bar(FB_DV_STAGED), kEwWarps);
    mbar_init(bar(FB_DK_STAGED), kEwWarps);
    mbar_init(bar(FB_PD_STORED), 1);
    for (int s = 0; s < 4; ++s) mbar_init(bar(FB_ITEM_FULL + s), 1);
    fence_barrier_init();
    w_first = first_walk_of((int)blockIdx.x);   // the grid never exceeds the number of key blocks
    item_ring[0] = w_first;
    mbar_arrive(bar(FB_ITEM_FULL + 0));
    // The loads of the first tile go out right here, before the TMEM allocation and the CTA-wide
    // barrier below, so that their latency (the first bytes of K, V, Q, dO come from HBM) runs
    // under the rest of the set-up.  K and Q first: S^T of the first tile needs only those.
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_v);
    tma_prefetch_desc(&map_do);
    tma_prefetch_desc(&map_dk);
    tma_prefetch_desc(&map_dv);
    if (pw) {
      tma_prefetch_desc(&map_q2);
      tma_prefetch_desc(&map_k2);
      tma_prefetch_desc(&map_dk2);
    }
    if (w_first < end_id) {
      const FusedItem first = decode(w_first);
      const int h0 = first.hk * G, m00 = first.mt_lo * BM;
      const CUtensorMap *mk = first.mode == 2 ? &map_k2 : &map_k, *mq = first.mode == 2 ? &map_q2 : &map_q;
      mbar_expect_tx(bar(FB_KV_FULL), C::kTile);
      for (int s = 0; s < KSUB; ++s)
        tma_load_4d(smem + C::kK + s * BN * 128, mk, bar(FB_KV_FULL), s * 64, first.n0, first.hk, first.b);
      mbar_expect_tx(bar(FB_Q_FULL), C::kTile);
      for (int s = 0; s < KSUB; ++s)
        tma_load_4d(smem + C::kQ0 + s * BM * 128, mq, bar(FB_Q_FULL), s * 64, m00, h0, first.b);
      mbar_expect_tx(bar(FB_V_FULL), C::kTile);
      for (int s = 0; s < KSUB; ++s)
        tma_load_4d(smem + C::kV + s * BN * 128, &map_v, bar(FB_V_FULL), s * 64, first.n0, first.hk, first.b);
      mbar_expect_tx(bar(FB_DO_FULL), C::kTile);
      for (int s = 0; s < KSUB; ++s)
        tma_load_4d(smem + C::kDO0 + s * BM * 128, &map_do, bar(FB_DO_FULL), s * 64, m00, h0, first.b);
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
    if (lane == 0) {
      bool ok = true;
      int sq = 0, phq = 1, sd = 0, phd = 1;   // ring slot and the "free" parity to wait for
      int inflight_q = 0, inflight_do = 0;    // loads requested (for the drain after an abort)
      int real = 0;                           // items with tiles handled so far
      uint32_t gt = 0;                        // tiles of those items
      bool pending = false;                   // dV / dK of the previous such item not stored yet
      int pn0 = 0, phk = 0, pb = 0;           // its coordinates,
      int pmode = 0;                          // its walk
      bool plast = true;                      // and whether it closed its key block (dV final)
      int nvl = 0;                            // V tiles requested so far: the phase of V_FULL
      auto load_q = [&](const FusedItem &it, int h, int mt) {
        mbar_expect_tx(bar(FB_Q_FULL + sq), C::kTile);
        for (int s = 0; s < KSUB; ++s)
          tma_load_4d(smem + C::kQ0 + sq * C::kTile + s * BM * 128, it.mode == 2 ? &map_q2 : &map_q,
                      bar(FB_Q_FULL + sq), s * 64, mt * BM, h, it.b);
        ++inflight_q;
      };
      auto load_do = [&](const FusedItem &it, int h, int mt) {
        mbar_expect_tx(bar(FB_DO_FULL + sd), C::kTile);
        for (int s = 0; s < KSUB; ++s)
          tma_load_4d(smem + C::kDO0 + sd * C::kTile + s * BM * 128, &map_do, bar(FB_DO_FULL + sd),
                      s * 64, mt * BM, h, it.b);
        ++inflight_do;
      };
      // dV then dK of the previous item leave through the copy engine as soon as the element-wise
      // warps have staged them; `between` runs after the dV store has been requested
      auto store_dv = [&]() -> bool {
        if (!mbar_wait(bar(FB_DV_STAGED), (real - 1) & 1, actx, 721)) return false;
        if (plast && !p.dv_accumulate) {   // a near walk that a far walk follows stages nothing
#pragma unroll
          for (int s = 0; s < KSUB; ++s)
            tma_store_4d(&map_dv, smem + C::kV + s * BN * 128, s * 64, pn0, phk, pb);
          bulk_commit();
        }
        return true;
      };
      auto store_dk = [&]() -> bool {
        if (!mbar_wait(bar(FB_DK_STAGED), (real - 1) & 1, actx, 722)) return false;
#pragma unroll
        for (int s = 0; s < KSUB; ++s)
          tma_store_4d(pmode == 2 ? &map_dk2 : &map_dk, smem + C::kPD + s * BN * 128, s * 64, pn0, phk, pb);
        bulk_commit();
        return true;
      };
      int w = w_first, ic = 0;
      if (w < end_id) nvl = 1;   // V of the first walk: see set-up
      while (w < end_id && ok) {
        const FusedItem it = decode(w);
        // Unless the far walk of the same key block follows, ask for the next block now; the answer
        // is looked at after this walk's first loads have gone out, so its latency hides behind them
        const bool more = pw && !it.last;
        const unsigned fetched = more ? 0u : atomicAdd(fp.sched, 1u);
        int w_next = end_id;
        {
          int h = it.hk * G, mt = it.mt_lo;
          const bool preissued = (ic == 0);   // tile 0, K and V of the first item: see set-up
          if (preissued) {
            inflight_q = inflight_do = 1;
          } else {
            ok = mbar_wait(bar(FB_Q_FREE + sq), phq, actx, 711);
            if (!ok) break;
            load_q(it, h, mt);
            ok = mbar_wait(bar(FB_DO_FREE + sd), phd, actx, 712);
            if (!ok) break;
            load_do(it, h, mt);
            if (pending) {
              ok = store_dv();
              // K is free once every product of the previous item has completed (the last one
              // issued reads it).  This thread does not follow the per-tile barriers phase by
              // phase, so it waits on the per-item one.
              if (ok) ok = mbar_wait(bar(FB_DONE), (real - 1) & 1, actx, 723);
              if (!ok) break;
            }
            mbar_expect_tx(bar(FB_KV_FULL), C::kTile);
            for (int s = 0; s < KSUB; ++s)
              tma_load_4d(smem + C::kK + s * BN * 128, it.mode == 2 ? &map_k2 : &map_k, bar(FB_KV_FULL),
                          s * 64, it.n0, it.hk, it.b);
            if (pending) {
              ok = store_dk();
              if (!ok) break;
              bulk_wait_read_1();            // the dV store (if any) has read the shared memory of V
            }
            if (it.first) {                  // a far walk after a near one finds V in place
              mbar_expect_tx(bar(FB_V_FULL), C::kTile);
              for (int s = 0; s < KSUB; ++s)
                tma_load_4d(smem + C::kV + s * BN * 128, &map_v, bar(FB_V_FULL), s * 64, it.n0, it.hk, it.b);
              ++nvl;
            }
            if (pending) {
              bulk_wait_read_all();          // the dK store has read the P^T / dS^T tile
              mbar_arrive(bar(FB_PD_STORED));
            }
          }
          pending = true, pn0 = it.n0, phk = it.hk, pb = it.b, pmode = it.mode, plast = it.last;
          ++real;
          // hand the next walk's id to the other warps
          if (more) {
            w_next = w + 1;
          } else {
            if (fetched == (unsigned)total - 1u) atomicExch(fp.sched, 0u);
            w_next = first_walk_of((int)gridDim.x + (int)fetched);
          }
          item_ring[(ic + 1) & 3] = w_next;
          mbar_arrive(bar(FB_ITEM_FULL + ((ic + 1) & 3)));
          if (++sq == NQ) sq = 0, phq ^= 1;
          if (++sd == NDO) sd = 0, phd ^= 1;
          if (++mt == it.mt_hi) mt = it.mt_lo, ++h;
          for (int t = 1; t < it.T_tiles; ++t) {
            ok = mbar_wait(bar(FB_Q_FREE + sq), phq, actx, 713);
            if (!ok) break;
            load_q(it, h, mt);
            ok = mbar_wait(bar(FB_DO_FREE + sd), phd, actx, 714);
            if (!ok) break;
            load_do(it, h, mt);
            if (++sq == NQ) sq = 0, phq ^= 1;
            if (++sd == NDO) sd = 0, phd ^= 1;
            if (++mt == it.mt_hi) mt = it.mt_lo, ++h;
          }
          if (!ok) break;
          gt += (uint32_t)it.T_tiles;
          // K and V of the next item are read by nobody else: start them towards L2 now, a couple
          // of tiles before this item ends (any earlier and they would be evicted again)
          if (w_next < end_id) {
            const FusedItem nx = decode(w_next);
            for (int s = 0; s < KSUB; ++s) {
              tma_prefetch_l2_4d(nx.mode == 2 ? &map_k2 : &map_k, s * 64, nx.n0, nx.hk, nx.b);
              if (nx.first) tma_prefetch_l2_4d(&map_v, s * 64, nx.n0, nx.hk, nx.b);
            }
          }
        }
        w = w_next, ++ic;
      }
      if (ok && pending) {
        ok = store_dv();
        if (ok) ok = store_dk();
      }
      bulk_wait_read_all();   // shared memory must outlive the copy engine's reads
      if (!ok) {
        // let copies already in flight land before the CTA gives its shared memory back
        const long long t0 = clock64();
        for (int i = max(0, inflight_q - NQ); i < inflight_q; ++i)
          while (!mbar_try_wait(bar(FB_Q_FULL + i % NQ), (i / NQ) & 1) && clock64() - t0 < 2000000) {}
        for (int i = max(0, inflight_do - NDO); i < inflight_do; ++i)
          while (!mbar_try_wait(bar(FB_DO_FULL + i % NDO), (i / NDO) & 1) && clock64() - t0 < 2000000) {}
        if (real > 0)
          while (!mbar_try_wait(bar(FB_KV_FULL), (real - 1) & 1) && clock64() - t0 < 2000000) {}
        if (nvl > 0)
          while (!mbar_try_wait(bar(FB_V_FULL), (nvl - 1) & 1) && clock64() - t0 < 2000000) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = instr_desc_f16(BN, BM, TcElem<T>::kFormat, 0, 0);   // S^T, dP^T
      constexpr uint32_t idesc_acc = instr_desc_f16(BN, D, TcElem<T>::kFormat, 0, 1);  // dV, dK
      constexpr uint32_t idesc_dq = instr_desc_f16(BM, D / C::NH, TcElem<T>::kFormat, 1, 1);  // dQ
      constexpr uint32_t kTile16 = C::kTile >> 4;
      const uint32_t k_lo = smem_desc_lo(smem + C::kK, 0), v_lo = smem_desc_lo(smem + C::kV, 0);
      const uint32_t k_mn_lo = smem_desc_lo(smem + C::kK, BN * 128);     // K as MN-major B of dQ
      const uint32_t q_k_lo = smem_desc_lo(smem + C::kQ0, 0);            // Q as K-major B operand
      const uint32_t q_mn_lo = smem_desc_lo(smem + C::kQ0, BM * 128);     // Q as MN-major B operand
      const uint32_t do_k_lo = smem_desc_lo(smem + C::kDO0, 0);
      const uint32_t do_mn_lo = smem_desc_lo(smem + C::kDO0, BM * 128);
      const uint32_t pd_k_lo = smem_desc_lo(smem + C::kPD, 0);            // P^T / dS^T, K-major A
      const uint32_t pd_mn_lo = smem_desc_lo(smem + C::kPD, BN * 128);    // dS, MN-major A of dQ
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
      bool ok = true;
      int sq = 0, phq = 0, sd = 0, phd = 0;
      int real = 0;            // items with tiles so far
      int nv = 0;              // V tiles so far: the phase of V_FULL (a far walk after a near one loads none)
      uint32_t gt = 0;         // tiles so far, over all items: the phase of every per-tile barrier
      uint32_t gh = 0;         // dQ parts so far: the phase of DQ_FULL / DQ_FREE
      // part `hf` of dQ = dS K into the dQ columns, a fresh accumulator: the read-out of the part
      // before must be over
      auto issue_dq_part = [&](int hf) -> bool {
        if (gh > 0 && !mbar_wait(bar(FB_DQ_FREE), (gh - 1) & 1, actx, 818)) return false;
        tc_fence_after();
        const uint32_t b_lo = k_mn_lo + hf * ((BN * 128) >> 4);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint32_t off16 = (kk * 16 * 128) >> 4;
          mma_ss_lo(tmem + C::kColQ, pd_mn_lo + off16, b_lo + off16, idesc_dq, kk > 0 ? 1u : 0u);
        }
        mma_commit(bar(FB_DQ_FULL));
        ++gh;
        return true;
      };
      for (int ic = 0; ok; ++ic) {
        const int w = ring_item(ic, 801);
        if (w < 0 || w >= end_id) break;
        const FusedItem it = decode(w);
        ok = mbar_wait(bar(FB_KV_FULL), real & 1, actx, 811);
        // the score columns still hold dP^T of the previous item's last tile until the
        // element-wise warps have it in registers
        if (ok && gt > 0) ok = mbar_wait(bar(FB_DP_LOADED), (gt - 1) & 1, actx, 821);
        if (ok) {
          tc_fence_after();
          ok = issue_s(sq, phq);
        }
        for (int t = 0; t < it.T_tiles && ok; ++t, ++gt) {
          int nsq = sq + 1, nphq = phq;
          if (nsq == NQ) nsq = 0, nphq ^= 1;
          const uint32_t acc = t > 0 ? 1u : 0u;                  // dK: fresh per walk
          const uint32_t acc_dv = (t > 0 || !it.first) ? 1u : 0u;   // dV: fresh per key block
          const uint32_t par = gt & 1;
          // dP^T(t) = V dO^T over S^T(t), once every element-wise warp holds S^T(t) in registers
          ok = mbar_wait(bar(FB_S_LOADED), par, actx, 813);
          if (ok && t == 0 && it.first) ok = mbar_wait(bar(FB_V_FULL), (nv++) & 1, actx, 820);
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
          // the second part of dQ of the tile before (head_dim 128): its first part has been read
          // out meanwhile; PD is free once it is through
          if (C::NH == 2 && t > 0) {
            ok = issue_dq_part(1);
            if (!ok) break;
            mma_commit(bar(FB_DS_FREE));
          }
          // dV += P^T(t) dO(t), P^T from TMEM
          ok = mbar_wait(bar(FB_PT_FULL), par, actx, 815);
          if (!ok) break;
          tc_fence_after();
          {
            const uint32_t b_lo = do_mn_lo + sd * kTile16;
#pragma unroll
            for (int kk = 0; kk < BM / 16; ++kk)
              mma_ts_lo(tmem + C::kColDV, tmem + C::kColP + kk * 8, b_lo + ((kk * 16 * 128) >> 4),
                        idesc_acc, kk > 0 ? 1u : acc_dv);
            mma_commit(bar(FB_DO_FREE + sd));
            mma_commit(bar(FB_PT_FREE));
          }
          // S^T(t+1), once every element-wise warp holds dP^T(t) in registers
          if (t + 1 < it.T_tiles) {
            ok = mbar_wait(bar(FB_DP_LOADED), par, actx, 816);
            if (!ok) break;
            tc_fence_after();
            ok = issue_s(nsq, nphq);
            if (!ok) break;
          }
          // the first part of dQ(t) = dS(t) K
          ok = mbar_wait(bar(FB_DS_FULL), par, actx, 817);
          if (ok) ok = issue_dq_part(0);
          if (!ok) break;
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
            if (C::NH == 1) mma_commit(bar(FB_DS_FREE));
          }
          sq = nsq, phq = nphq;
          if (++sd == NDO) sd = 0, phd ^= 1;
        }
        if (!ok) break;
        if (C::NH == 2) {   // the second part of dQ of the item's last tile
          ok = issue_dq_part(1);
          if (!ok) break;
          mma_commit(bar(FB_DS_FREE));
        }
        mma_commit(bar(FB_DONE));
        ++real;
      }
      // the last commit's arrive must land before this CTA's shared memory is given back
      if (ok && real > 0) mbar_wait(bar(FB_DONE), (real - 1) & 1, actx, 819);
    }
  } else if (warp == 2 + kEwWarps + 4) {
    // ------------------------------ statistics warp ----------------------------
    // -lse * log2(e) and -delta of the 128 queries of every tile go through shared memory, where
    // the element-wise threads read them as broadcast vectors (every thread needs the values of
    // all its 32 query columns; fetching them lane by lane and shuffling costs 64 shuffles per
    // thread and tile in a load/store queue that is already the busiest unit).  Queries past M
    // get lse = +inf, which makes their P exactly zero.  One buffer each: lse(t) may be written
    // once phase 1 of the tile before is over, delta(t) once its phase 2 is.
    float4 *lse_s = reinterpret_cast<float4 *>(smem_gen + C::kStats);
    float4 *dlt_s = lse_s + 32;
    bool ok = true;
    uint32_t gt = 0;
    for (int ic = 0; ok; ++ic) {
      const int w = ring_item(ic, 950);
      if (w < 0 || w >= end_id) break;
      const FusedItem it = decode(w);
      int h = it.hk * G, mt = it.mt_lo;
      for (int t = 0; t < it.T_tiles; ++t, ++gt) {
        const int m = mt * BM + lane * 4;
        const int64_t li = ((int64_t)it.b * p.H + h) * p.M + m;
        if (++mt == it.mt_hi) mt = it.mt_lo, ++h;
        float l[4], d[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          l[j] = m + j < p.M ? -p.lse[li + j] * kLog2e : -INFINITY;
          d[j] = m + j < p.M ? -p.delta[li + j] : 0.f;
        }
        if (gt > 0) ok = mbar_wait(bar(FB_PT_FULL), (gt - 1) & 1, actx, 951);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        lse_s[lane] = make_float4(l[0], l[1], l[2], l[3]);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(FB_LSE_FULL));
        if (gt > 0) ok = mbar_wait(bar(FB_DS_FULL), (gt - 1) & 1, actx, 952);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        dlt_s[lane] = make_float4(d[0], d[1], d[2], d[3]);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(FB_DLT_FULL));
      }
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
    int buf = 0;
    bool ok = true;
    uint32_t gt = 0, gh = 0;
    constexpr int QPH = 4 / C::NH;            // quarters per part of dQ
    for (int ic = 0; ok; ++ic) {
      // every wait is bounded, so all four warps reach each vote; they leave together or not at all
      const int w = ring_item(ic, 920);
      if (!red_warps_all(w >= 0)) {
        ok = false;
        break;
      }
      if (w >= end_id) break;
      const FusedItem it = decode(w);
      int h = it.hk * G, mt = it.mt_lo;
      for (int t = 0; t < it.T_tiles; ++t, ++gt) {
        // the tile's block of the workspace: D / 4 runs of (128 queries x 4 columns), contiguous
        float *dst = (it.mode == 2 ? fp.dq_acc2 : fp.dq_acc) +
                     (((int64_t)it.b * p.H + h) * (fp.Mpad / BM) + mt) * (int64_t)(BM * D);
        if (++mt == it.mt_hi) mt = it.mt_lo, ++h;
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
          if (qd % QPH == 0) {   // the next part of dQ
            ok = red_warps_all(mbar_wait(bar(FB_DQ_FULL), gh & 1, actx, 921));
            if (!ok) break;
            ++gh;
            tc_fence_after();
          }
          uint32_t qr[QC];
          if (QC == 32) tmem_ld32(tlane + C::kColQ + (qd % QPH) * QC, *reinterpret_cast<uint32_t(*)[32]>(qr));
          else tmem_ld16(tlane + C::kColQ + (qd % QPH) * QC, qr);
          tmem_wait_ld();
          if (C::kPAliasesDQ && qd == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(FB_DQ_HALF));   // the next P^T may take the first 64 columns
          }
          if (qd % QPH == QPH - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(FB_DQ_FREE));   // the next dQ may overwrite the columns
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
        if (!ok) break;
      }
    }
    if (issuer) bulk_wait_read_all();   // shared memory must outlive the copy engine's reads
  } else {
    // ------------------------------ element-wise warps --------------------------
    const int ew = warp - 2;
    const int slice = warp & 3, cg = ew >> 2;       // TMEM lane slice, 32-column group
    const int row = slice * 32 + lane;              // accumulator row of this thread
    const uint32_t tlane = tmem + ((uint32_t)(slice * 32) << 16);
    const float qk_scale = p.sm_scale * kLog2e;
    // this thread's 64 bytes of a PD row: sub-tile cg / 2, 16-byte chunks (cg & 1) * 4 .. + 3
    uint8_t *pd_row = smem_gen + C::kPD + (cg >> 1) * (128 * 128) + row * 128;
    const int pd_chunk0 = (cg & 1) * 4, pd_xor = row & 7;
    auto store_pd = [&](const uint32_t (&pk)[16]) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4 *>(pd_row + (((pd_chunk0 + j) ^ pd_xor) << 4)) =
            make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
    };
    // -lse * log2(e) / -delta of this thread's 32 query columns, as staged by the statistics warp
    const float4 *lse_s = reinterpret_cast<const float4 *>(smem_gen + C::kStats) + cg * 8;
    const float4 *dlt_s = lse_s + 32;
    // write-out of dV and dK: warp (slice, cg) owns columns cg * D / 4 .. of its 32 rows
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
    // a 128 x D 16-bit tile in the layout of a TMA box (128-byte rows, 128-byte swizzle)
    auto stage = [&](int region, const uint32_t (&ov)[QC], float scale) {
      uint8_t *base = smem_gen + region + (col0 / 64) * (128 * 128) + row * 128;
      const int ch0 = (col0 % 64) / 8;
#pragma unroll
      for (int j = 0; j < QC / 8; ++j)
        *reinterpret_cast<uint4 *>(base + (((ch0 + j) ^ (row & 7)) << 4)) = pack8(ov + 8 * j, scale);
    };
    bool ok = true;
    int real = 0;
    uint32_t gt = 0;

    for (int ic = 0; ok; ++ic) {
      const int w = ring_item(ic, 900);
      ok = __all_sync(0xffffffffu, w >= 0);
      if (!ok || w >= end_id) break;
      const FusedItem it = decode(w);
      const int n0 = it.n0, key = n0 + row;
      const bool key_ok = key < p.N;
      auto direct = [&](void *out, const Strides &so, uint32_t (&ov)[QC], float scale, bool add) {
        if (!key_ok) return;
        T *orow = row_ptr_mut<T>(out, so, it.b, it.hk, key) + col0;
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
      int mt = it.mt_lo;   // query tile of the current tile

      for (int t = 0; t < it.T_tiles; ++t, ++gt) {
        const int m0 = mt * BM;
        if (++mt == it.mt_hi) mt = it.mt_lo;

        // ---- phase 1: P^T = exp2(S^T * scale - lse) -> TMEM ----
        ok = mbar_wait(bar(FB_LSE_FULL), gt & 1, actx, 910);
        if (ok) ok = mbar_wait(bar(FB_S_FULL), gt & 1, actx, 911);
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
        if (it.mode == 1) interior = interior && (m0 + BM - 1 + p_seq - n0 < p.w);
        if (it.mode == 2) interior = interior && (m0 + p_seq - (n0 + BN - 1) >= p.w);
        int cmin = 0, cmax = 32;
        if (p.causal) cmin = max(cmin, key - p_seq - m0 - cg * 32);
        if (it.mode) {
          const int cnear = p.w + key - p_seq - m0 - cg * 32;  // columns below it are near pairs
          if (it.mode == 1) cmax = min(cmax, cnear);
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
          // the P^T columns still hold P^T of the tile before until its dV product has read them
          if (gt > 0) ok = mbar_wait(bar(FB_PT_FREE), (gt - 1) & 1, actx, 912);
          // ... and, where P^T borrows columns of dQ, dQ of the tile before until they are read out
          if (C::kPAliasesDQ && ok && gt > 0) ok = mbar_wait(bar(FB_DQ_HALF), (gt - 1) & 1, actx, 918);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tmem_st16(tlane + C::kColP + cg * 16, pk);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(FB_PT_FULL));
        }
        // ---- phase 2: dS^T = P^T * (dP^T - delta) -> PD ----
        // Its operands are there by now (dP^T(t) was issued as soon as S^T(t) had been read).
        ok = mbar_wait(bar(FB_DLT_FULL), gt & 1, actx, 909);
        if (ok) ok = mbar_wait(bar(FB_DP_FULL), gt & 1, actx, 913);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t sr0[16];
        tmem_ld16(tlane + C::kColA + cg * 32, sr0);
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
            if (lane == 0) mbar_arrive(bar(FB_DP_LOADED));   // the next S^T may overwrite dP^T(t)
            half_ds(1, sr1);
          }
          // PD still holds dS^T of the tile before until its dQ and dK products have read it, and,
          // at the first tile of an item, the staged dK of the item before until it is stored
          if (gt > 0) ok = mbar_wait(bar(FB_DS_FREE), (gt - 1) & 1, actx, 914);
          if (ok && t == 0 && real > 0) ok = mbar_wait(bar(FB_PD_STORED), (real - 1) & 1, actx, 917);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          store_pd(pk);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(FB_DS_FULL));
      }
      if (!ok) break;

      // ---- write-out of dV and dK of this item ----
      // dV is final once its last product has been committed, so it is converted and staged while dQ and dK of the last tile still run on the tensor
      // cores; dK follows after the last commit.  dV is staged in the shared memory of V and dK in
      // the P^T / dS^T tile (both dead by then) in the layout of an operand load, and the producer
      // thread sends them off as bulk tensor stores, which also drop the rows past N.  A dV that is
      // added to (the second launch of a piecewise backward) keeps per-thread global stores.
      {
        uint32_t ov[QC];
        ok = mbar_wait(bar(FB_PT_FREE), (gt - 1) & 1, actx, 915);   // the last dV product
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (it.last) {   // (a near walk that a far walk follows leaves dV in TMEM and V in place)
          load_cols(C::kColDV, ov);
          if (!p.dv_accumulate) {
            stage(C::kV, ov, 1.f);
            fence_proxy_async_smem();
          } else {
            direct(p.dv, p.sdv, ov, 1.f, true);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(FB_DV_STAGED));
        ok = mbar_wait(bar(FB_DONE), real & 1, actx, 916);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        load_cols(C::kColDK, ov);
        stage(C::kPD, ov, p.sm_scale);
        fence_proxy_async_smem();
        // the accumulator columns are free for the next item once every warp has read them
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(FB_DK_STAGED));
      }
      ++real;
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

// Zero-fill of rows [r_begin, r_end) of every (batch, head) of dk / dv: the keys no query sees
// (past the causal triangle, or without a pair of the branch in a piecewise launch), whose blocks
// the kernel above skips.
template <typename T, int D>
__global__ void __launch_bounds__(256)
    zero_rows_kernel(void *out, Strides so, int r_begin, int r_end) {
  const int m = r_begin + blockIdx.x * 16 + (threadIdx.x >> 4);
  if (m >= r_end) return;
  T *orow = row_ptr_mut<T>(out, so, blockIdx.z, blockIdx.y, m);
  for (int c = (threadIdx.x & 15) * 8; c < D; c += 128)
    *reinterpret_cast<uint4 *>(orow + c) = make_uint4(0u, 0u, 0u, 0u);
}

}  // namespace tc
}  // namespace fa
