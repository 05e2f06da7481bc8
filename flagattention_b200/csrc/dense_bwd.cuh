// Shape-generic backward kernels for flash_attention and piecewise_attention:
//   delta kernel      delta = rowsum(O * dO)
//   dK/dV kernel      one CTA per key block, K/V resident, loops over query tiles
//                     (and over the query heads of a GQA group)
//   dQ kernel         one CTA per query block, Q/dO resident, loops over key tiles
// No global atomics anywhere.  P is recomputed from the saved log-normaliser.
// The piecewise variants walk the tiles in two passes (near branch, then far
// branch) so only one dK / dQ accumulator is live at a time.
#pragma once

#include "attn_params.cuh"

namespace fa {

// ---------------------------------------------------------------------------
// delta
// ---------------------------------------------------------------------------
// A thread owns 16 bytes of kDeltaRows rows (all loads are issued before the first use, 128 bytes
// in flight per thread); a block stays inside one (batch, head) pair, so the only divisions are
// one per block and shifts.
constexpr int kDeltaRows = 4;
// `zero` (may be null): a buffer of `zero_granules` 16-byte granules that the same launch fills
// with zeros, every block an equal contiguous share: the workspace of the one-pass backward,
// whose zero-fill is a memory-bound pass over a different buffer and rides with this one.
template <typename T, int D>
__global__ void bwd_delta_kernel(const void *o, Strides so, const void *d_o, Strides sdo,
                                 float *delta, int B, int H, int M, int blocks_per_pair,
                                 uint4 *zero, long long zero_granules) {
  constexpr int LPR = D / 8;  // lanes per row
  if (zero) {
    const long long share = (zero_granules + gridDim.x - 1) / gridDim.x;
    const long long begin = share * blockIdx.x;
    const long long end = begin + share < zero_granules ? begin + share : zero_granules;
    for (long long g = begin + threadIdx.x; g < end; g += blockDim.x) zero[g] = make_uint4(0u, 0u, 0u, 0u);
  }
  const int bh = blockIdx.x / blocks_per_pair;
  const int rows_per_pass = blockDim.x / LPR;
  const int m0 = (blockIdx.x - bh * blocks_per_pair) * (rows_per_pass * kDeltaRows) +
                 threadIdx.x / LPR;
  const int ch = threadIdx.x % LPR;
  const int b = bh / H, h = bh - b * H;
  uint4 ov[kDeltaRows], dv[kDeltaRows];
#pragma unroll
  for (int r = 0; r < kDeltaRows; ++r) {
    const int m = m0 + r * rows_per_pass;
    ov[r] = dv[r] = make_uint4(0u, 0u, 0u, 0u);
    if (m < M) {
      ov[r] = *reinterpret_cast<const uint4 *>(row_ptr<T>(o, so, b, h, m) + ch * 8);
      dv[r] = *reinterpret_cast<const uint4 *>(row_ptr<T>(d_o, sdo, b, h, m) + ch * 8);
    }
  }
#pragma unroll
  for (int r = 0; r < kDeltaRows; ++r) {
    const int m = m0 + r * rows_per_pass;
    const uint32_t *ou = reinterpret_cast<const uint32_t *>(&ov[r]);
    const uint32_t *du = reinterpret_cast<const uint32_t *>(&dv[r]);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 a = Elem<T>::unpack(ou[i]), c = Elem<T>::unpack(du[i]);
      sum += a.x * c.x + a.y * c.y;
    }
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (m < M && ch == 0) delta[(int64_t)bh * M + m] = sum;
  }
}

// 4-byte async copies of `count` floats (zero-filled past `valid`).
__device__ __forceinline__ void load_floats_async(uint32_t dst, const float *src, int count,
                                                  int valid, int tid, int nthreads) {
  for (int i = tid; i < count; i += nthreads) {
    bool ok = i < valid;
    int sz = ok ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst + i * 4),
                 "l"(src + (ok ? i : 0)), "r"(sz));
  }
}

// ---------------------------------------------------------------------------
// dK / dV
// ---------------------------------------------------------------------------
template <int D, int BM, int BN, bool PW>
struct DkdvSmemLayout {
  static constexpr int kKVBytes = BN * D * 2;
  static constexpr int kQBytes = BM * D * 2;
  static constexpr int kK1 = 0;
  static constexpr int kV = kKVBytes;
  static constexpr int kK2 = 2 * kKVBytes;
  static constexpr int kStage0 = (PW ? 3 : 2) * kKVBytes;
  // stage: Q1, dO, (Q2), lse[BM], delta[BM]
  static constexpr int kStQ1 = 0;
  static constexpr int kStDO = kQBytes;
  static constexpr int kStQ2 = 2 * kQBytes;
  static constexpr int kStLse = (PW ? 3 : 2) * kQBytes;
  static constexpr int kStDelta = kStLse + BM * 4;
  static constexpr int kStageBytes = kStDelta + BM * 4;
  static constexpr int kTotal = kStage0 + 2 * kStageBytes;
};

template <typename T, int D, int BM, int BN, bool PW>
__global__ void __launch_bounds__(BN / 16 * 32) dense_bwd_dkdv_kernel(const BwdParams p) {
  constexpr int NW = BN / 16, NT = NW * 32;
  using L = DkdvSmemLayout<D, BM, BN, PW>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const uint32_t smem = smem_u32(smem_raw);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int nb = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = p.H / p.Hk;
  const int n0 = nb * BN;
  const int p_seq = p.N - p.M;
  const float qk_scale = p.sm_scale * kLog2e;
  const int kr0 = warp * 16;
  const int key_g[2] = {n0 + kr0 + g, n0 + kr0 + g + 8};

  // resident K, V (and K2)
  load_tile_async<T, D, BN, NT>(smem + L::kK1, row_ptr<T>(p.k, p.sk, b, hk, n0), p.sk.l,
                                p.N - n0, tid);
  load_tile_async<T, D, BN, NT>(smem + L::kV, row_ptr<T>(p.v, p.sv, b, hk, n0), p.sv.l, p.N - n0,
                                tid);
  if (PW)
    load_tile_async<T, D, BN, NT>(smem + L::kK2, row_ptr<T>(p.k2, p.sk2, b, hk, n0), p.sk2.l,
                                  p.N - n0, tid);
  cp_async_commit();

  // query-tile range seen by this key block
  const int num_m_tiles = (p.M + BM - 1) / BM;
  int mt_lo = 0;
  if (p.causal) mt_lo = max(0, n0 - p_seq) / BM;  // first tile with a row m, m + p_seq >= n0

  float dv[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) dv[j][0] = dv[j][1] = dv[j][2] = dv[j][3] = 0.f;

  constexpr int NPASS = PW ? 2 : 1;
#pragma unroll 1
  for (int pass = 0; pass < NPASS; ++pass) {
    // tile window of this pass
    int mt_begin = mt_lo, mt_end = num_m_tiles;
    if (PW) {
      if (pass == 0) {
        // tiles with a near element: m0 + p_seq - (n0 + BN - 1) < w
        int lim = p.w - p_seq + n0 + BN - 1;  // m0 < lim
        int e = lim <= 0 ? 0 : (lim + BM - 1) / BM;
        mt_end = min(num_m_tiles, e);
      } else {
        // tiles with a far element: m0 + BM - 1 + p_seq - n0 >= w
        int lim = p.w - p_seq + n0 - BM + 1;  // m0 >= lim
        int s = lim <= 0 ? 0 : (lim + BM - 1) / BM;
        mt_begin = max(mt_lo, s);
      }
    }
    const int tiles = max(0, mt_end - mt_begin);
    const int iters = tiles * G;

    float dk[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) dk[j][0] = dk[j][1] = dk[j][2] = dk[j][3] = 0.f;

    auto issue = [&](int it) {
      const int gi = it / tiles, mt = mt_begin + it % tiles;
      const int h = hk * G + gi, m0 = mt * BM;
      const uint32_t st = smem + L::kStage0 + (it & 1) * L::kStageBytes;
      PwClass c{true, false};
      if (PW) c = pw_classify(m0, BM, n0, BN, p_seq, p.w);
      if (c.need1)
        load_tile_async<T, D, BM, NT>(st + L::kStQ1, row_ptr<T>(p.q, p.sq, b, h, m0), p.sq.l,
                                      p.M - m0, tid);
      if (PW && c.need2)
        load_tile_async<T, D, BM, NT>(st + L::kStQ2, row_ptr<T>(p.q2, p.sq2, b, h, m0), p.sq2.l,
                                      p.M - m0, tid);
      load_tile_async<T, D, BM, NT>(st + L::kStDO, row_ptr<T>(p.d_o, p.sdo, b, h, m0), p.sdo.l,
                                    p.M - m0, tid);
      const int64_t lbase = ((int64_t)b * p.H + h) * p.M + m0;
      load_floats_async(st + L::kStLse, p.lse + lbase, BM, p.M - m0, tid, NT);
      load_floats_async(st + L::kStDelta, p.delta + lbase, BM, p.M - m0, tid, NT);
    };

    if (iters > 0) issue(0);
    cp_async_commit();

#pragma unroll 1
    for (int it = 0; it < iters; ++it) {
      if (it + 1 < iters) {
        issue(it + 1);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();

      const int mt = mt_begin + it % tiles;
      const int m0 = mt * BM;
      const uint32_t st = smem + L::kStage0 + (it & 1) * L::kStageBytes;
      const uint8_t *st_raw = smem_raw + L::kStage0 + (it & 1) * L::kStageBytes;
      const float *lse_s = reinterpret_cast<const float *>(st_raw + L::kStLse);
      const float *delta_s = reinterpret_cast<const float *>(st_raw + L::kStDelta);
      PwClass c{true, false};
      if (PW) c = pw_classify(m0, BM, n0, BN, p_seq, p.w);

      // S^T = K Q^T  (16 keys x BM queries per warp)
      float s[BM / 8][4];
#pragma unroll
      for (int j = 0; j < BM / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      if (c.need1) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          uint32_t a[4];
          load_A<D>(a, smem + L::kK1, kr0, kk, lane);
#pragma unroll
          for (int mj = 0; mj < BM / 16; ++mj) {
            uint32_t bb[4];
            load_B_nk<D>(bb, st + L::kStQ1, mj * 16, kk, lane);
            Elem<T>::mma(s[2 * mj], a, bb[0], bb[1]);
            Elem<T>::mma(s[2 * mj + 1], a, bb[2], bb[3]);
          }
        }
      }
      if (PW && c.need2) {
        float s2[BM / 8][4];
#pragma unroll
        for (int j = 0; j < BM / 8; ++j) s2[j][0] = s2[j][1] = s2[j][2] = s2[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          uint32_t a[4];
          load_A<D>(a, smem + L::kK2, kr0, kk, lane);
#pragma unroll
          for (int mj = 0; mj < BM / 16; ++mj) {
            uint32_t bb[4];
            load_B_nk<D>(bb, st + L::kStQ2, mj * 16, kk, lane);
            Elem<T>::mma(s2[2 * mj], a, bb[0], bb[1]);
            Elem<T>::mma(s2[2 * mj + 1], a, bb[2], bb[3]);
          }
        }
#pragma unroll
        for (int j = 0; j < BM / 8; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            int key = key_g[e >> 1], qm = m0 + j * 8 + 2 * t4 + (e & 1);
            if (!c.need1 || qm + p_seq - key >= p.w) s[j][e] = s2[j][e];
          }
      }

      // P^T = exp2(S^T * qk_scale - lse * log2e), masked after the exponential
#pragma unroll
      for (int j = 0; j < BM / 8; ++j) {
        const float2 l2 = *reinterpret_cast<const float2 *>(lse_s + j * 8 + 2 * t4);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key_g[e >> 1], qm = m0 + j * 8 + 2 * t4 + (e & 1);
          const float lv = (e & 1) ? l2.y : l2.x;
          const bool ok = qm < p.M && key < p.N && (!p.causal || qm + p_seq >= key);
          const float pv = fast_exp2(s[j][e] * qk_scale - lv * kLog2e);
          s[j][e] = ok ? pv : 0.f;
        }
      }

      // dropout: keep[j][e] * 1/(1-p) multiplies P on its way into dV and dP on its way into dS
      const bool dropout = !PW && p.dropout_p > 0.f;
      const float rp = dropout ? 1.f / (1.f - p.dropout_p) : 1.f;
      uint32_t keep_bits = 0xffffffffu;  // bit j*4+e
      if (dropout) {
        const int hq = hk * G + it / tiles;
        keep_bits = 0;
#pragma unroll
        for (int j = 0; j < BM / 8; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = key_g[e >> 1], qm = m0 + j * 8 + 2 * t4 + (e & 1);
            const uint64_t idx = (((uint64_t)b * p.H + hq) * p.M + qm) * p.N + key;
            if (dropout_keep(p.seed, p.offset, idx, p.dropout_p)) keep_bits |= 1u << (j * 4 + e);
          }
      }
      auto kept = [&](int j, int e, float v) { return (keep_bits >> (j * 4 + e)) & 1u ? v * rp : 0.f; };

      // dV += P^T dO   (in the far pass, straddling tiles were already counted)
      const bool do_dv = !PW || pass == 0 || !c.need1;
      if (do_dv) {
#pragma unroll
        for (int kj = 0; kj < BM / 16; ++kj) {
          uint32_t a[4];
          a[0] = Elem<T>::pack(kept(2 * kj, 0, s[2 * kj][0]), kept(2 * kj, 1, s[2 * kj][1]));
          a[1] = Elem<T>::pack(kept(2 * kj, 2, s[2 * kj][2]), kept(2 * kj, 3, s[2 * kj][3]));
          a[2] = Elem<T>::pack(kept(2 * kj + 1, 0, s[2 * kj + 1][0]), kept(2 * kj + 1, 1, s[2 * kj + 1][1]));
          a[3] = Elem<T>::pack(kept(2 * kj + 1, 2, s[2 * kj + 1][2]), kept(2 * kj + 1, 3, s[2 * kj + 1][3]));
#pragma unroll
          for (int dj = 0; dj < D / 16; ++dj) {
            uint32_t bb[4];
            load_B_kn<D>(bb, st + L::kStDO, kj * 16, dj * 2, lane);
            Elem<T>::mma(dv[2 * dj], a, bb[0], bb[1]);
            Elem<T>::mma(dv[2 * dj + 1], a, bb[2], bb[3]);
          }
        }
      }

      // dP^T = V dO^T
      float dp[BM / 8][4];
#pragma unroll
      for (int j = 0; j < BM / 8; ++j) dp[j][0] = dp[j][1] = dp[j][2] = dp[j][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        load_A<D>(a, smem + L::kV, kr0, kk, lane);
#pragma unroll
        for (int mj = 0; mj < BM / 16; ++mj) {
          uint32_t bb[4];
          load_B_nk<D>(bb, st + L::kStDO, mj * 16, kk, lane);
          Elem<T>::mma(dp[2 * mj], a, bb[0], bb[1]);
          Elem<T>::mma(dp[2 * mj + 1], a, bb[2], bb[3]);
        }
      }

      // dS^T = P^T * (dP^T - delta), routed to the branch of this pass
#pragma unroll
      for (int j = 0; j < BM / 8; ++j) {
        const float2 d2 = *reinterpret_cast<const float2 *>(delta_s + j * 8 + 2 * t4);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float dl = (e & 1) ? d2.y : d2.x;
          float ds = s[j][e] * (kept(j, e, dp[j][e]) - dl);
          if (PW) {
            const int key = key_g[e >> 1], qm = m0 + j * 8 + 2 * t4 + (e & 1);
            const bool far = qm + p_seq - key >= p.w;
            if (far != (pass == 1)) ds = 0.f;
          }
          s[j][e] = ds;
        }
      }

      // dK += dS^T Q (the Q of this pass's branch)
      const uint32_t qt = st + ((PW && pass == 1) ? L::kStQ2 : L::kStQ1);
#pragma unroll
      for (int kj = 0; kj < BM / 16; ++kj) {
        uint32_t a[4];
        a[0] = Elem<T>::pack(s[2 * kj][0], s[2 * kj][1]);
        a[1] = Elem<T>::pack(s[2 * kj][2], s[2 * kj][3]);
        a[2] = Elem<T>::pack(s[2 * kj + 1][0], s[2 * kj + 1][1]);
        a[3] = Elem<T>::pack(s[2 * kj + 1][2], s[2 * kj + 1][3]);
#pragma unroll
        for (int dj = 0; dj < D / 16; ++dj) {
          uint32_t bb[4];
          load_B_kn<D>(bb, qt, kj * 16, dj * 2, lane);
          Elem<T>::mma(dk[2 * dj], a, bb[0], bb[1]);
          Elem<T>::mma(dk[2 * dj + 1], a, bb[2], bb[3]);
        }
      }
      __syncthreads();
    }
    cp_async_wait<0>();

    // store dK of this pass (scaled), through the stage-0 Q1 buffer
    {
      void *dst = (PW && pass == 1) ? p.dk2 : p.dk;
      const Strides sd = (PW && pass == 1) ? p.sdk2 : p.sdk;
      uint8_t *buf = smem_raw + L::kStage0;  // >= 16 rows x D per warp needs BM*D >= BN*D? no:
      // each warp stages its 16 key rows in its own 16-row slice of a BN-row
      // scratch that spans both stages (2 * kStageBytes >= BN * D * 2 bytes).
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = kr0 + g + 8 * i;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
          uint32_t v = Elem<T>::pack(dk[j][2 * i] * p.sm_scale, dk[j][2 * i + 1] * p.sm_scale);
          *reinterpret_cast<uint32_t *>(buf + Tile<D>::offset(r, j) + t4 * 4) = v;
        }
      }
      __syncwarp();
      constexpr int CPR = D / 8;
#pragma unroll
      for (int i = 0; i < 16 * CPR / 32; ++i) {
        const int idx = lane + i * 32;
        const int r = idx / CPR, ch = idx % CPR;
        const int key = n0 + kr0 + r;
        if (key < p.N) {
          uint4 v = *reinterpret_cast<const uint4 *>(buf + Tile<D>::offset(kr0 + r, ch));
          *reinterpret_cast<uint4 *>(row_ptr_mut<T>(dst, sd, b, hk, key) + ch * 8) = v;
        }
      }
      __syncthreads();  // scratch is reused by the next pass's loads
    }
  }

  // store dV
  {
    uint8_t *buf = smem_raw + L::kStage0;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = kr0 + g + 8 * i;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        uint32_t v = Elem<T>::pack(dv[j][2 * i], dv[j][2 * i + 1]);
        *reinterpret_cast<uint32_t *>(buf + Tile<D>::offset(r, j) + t4 * 4) = v;
      }
    }
    __syncwarp();
    constexpr int CPR = D / 8;
#pragma unroll
    for (int i = 0; i < 16 * CPR / 32; ++i) {
      const int idx = lane + i * 32;
      const int r = idx / CPR, ch = idx % CPR;
      const int key = n0 + kr0 + r;
      if (key < p.N) {
        uint4 v = *reinterpret_cast<const uint4 *>(buf + Tile<D>::offset(kr0 + r, ch));
        *reinterpret_cast<uint4 *>(row_ptr_mut<T>(p.dv, p.sdv, b, hk, key) + ch * 8) = v;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// dQ
// ---------------------------------------------------------------------------
template <int D, int BM, int BN, bool PW>
struct DqSmemLayout {
  static constexpr int kQBytes = BM * D * 2;
  static constexpr int kKVBytes = BN * D * 2;
  static constexpr int kQ1 = 0;
  static constexpr int kDO = kQBytes;
  static constexpr int kQ2 = 2 * kQBytes;
  static constexpr int kStage0 = (PW ? 3 : 2) * kQBytes;
  static constexpr int kStK1 = 0;
  static constexpr int kStV = kKVBytes;
  static constexpr int kStK2 = 2 * kKVBytes;
  static constexpr int kStageBytes = (PW ? 3 : 2) * kKVBytes;
  static constexpr int kTotal = kStage0 + 2 * kStageBytes;
};

template <typename T, int D, int BM, int BN, bool PW>
__global__ void __launch_bounds__(BM / 16 * 32) dense_bwd_dq_kernel(const BwdParams p) {
  constexpr int NW = BM / 16, NT = NW * 32;
  using L = DqSmemLayout<D, BM, BN, PW>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const uint32_t smem = smem_u32(smem_raw);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int mb = gridDim.x - 1 - blockIdx.x;
  const int b = blockIdx.y / p.H, h = blockIdx.y % p.H;
  const int hk = h / (p.H / p.Hk);
  const int m0 = mb * BM;
  const int p_seq = p.N - p.M;
  const float qk_scale = p.sm_scale * kLog2e;
  const int r0 = warp * 16;
  const int row_g[2] = {m0 + r0 + g, m0 + r0 + g + 8};

  load_tile_async<T, D, BM, NT>(smem + L::kQ1, row_ptr<T>(p.q, p.sq, b, h, m0), p.sq.l, p.M - m0,
                                tid);
  load_tile_async<T, D, BM, NT>(smem + L::kDO, row_ptr<T>(p.d_o, p.sdo, b, h, m0), p.sdo.l,
                                p.M - m0, tid);
  if (PW)
    load_tile_async<T, D, BM, NT>(smem + L::kQ2, row_ptr<T>(p.q2, p.sq2, b, h, m0), p.sq2.l,
                                  p.M - m0, tid);
  cp_async_commit();

  float lse_r[2], delta_r[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const bool ok = row_g[i] < p.M;
    const int64_t li = ((int64_t)b * p.H + h) * p.M + row_g[i];
    lse_r[i] = ok ? p.lse[li] * kLog2e : 0.f;
    delta_r[i] = ok ? p.delta[li] : 0.f;
  }

  int n_hi = p.N;
  if (p.causal) n_hi = max(0, min(p.N, p_seq + m0 + BM));
  const int num_n_tiles = (n_hi + BN - 1) / BN;

  constexpr int NPASS = PW ? 2 : 1;
#pragma unroll 1
  for (int pass = 0; pass < NPASS; ++pass) {
    int nt_begin = 0, nt_end = num_n_tiles;
    if (PW) {
      if (pass == 0) {
        // tiles with a near element: n0 > m0 + p_seq - w - BN + 1
        int lim = m0 + p_seq - p.w - BN + 2;  // n0 >= lim
        nt_begin = lim <= 0 ? 0 : (lim + BN - 1) / BN;
      } else {
        // tiles with a far element: n0 <= m0 + BM - 1 + p_seq - w
        int lim = m0 + BM - 1 + p_seq - p.w;  // n0 <= lim
        nt_end = lim < 0 ? 0 : min(num_n_tiles, lim / BN + 1);
      }
    }
    const int iters = max(0, nt_end - nt_begin);

    float dq[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) dq[j][0] = dq[j][1] = dq[j][2] = dq[j][3] = 0.f;

    auto issue = [&](int it) {
      const int n0 = (nt_begin + it) * BN;
      const uint32_t st = smem + L::kStage0 + (it & 1) * L::kStageBytes;
      PwClass c{true, false};
      if (PW) c = pw_classify(m0, BM, n0, BN, p_seq, p.w);
      if (c.need1)
        load_tile_async<T, D, BN, NT>(st + L::kStK1, row_ptr<T>(p.k, p.sk, b, hk, n0), p.sk.l,
                                      p.N - n0, tid);
      if (PW && c.need2)
        load_tile_async<T, D, BN, NT>(st + L::kStK2, row_ptr<T>(p.k2, p.sk2, b, hk, n0), p.sk2.l,
                                      p.N - n0, tid);
      load_tile_async<T, D, BN, NT>(st + L::kStV, row_ptr<T>(p.v, p.sv, b, hk, n0), p.sv.l,
                                    p.N - n0, tid);
    };
    if (iters > 0) issue(0);
    cp_async_commit();

#pragma unroll 1
    for (int it = 0; it < iters; ++it) {
      if (it + 1 < iters) {
        issue(it + 1);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();

      const int n0 = (nt_begin + it) * BN;
      const uint32_t st = smem + L::kStage0 + (it & 1) * L::kStageBytes;
      PwClass c{true, false};
      if (PW) c = pw_classify(m0, BM, n0, BN, p_seq, p.w);

      float s[BN / 8][4];
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      if (c.need1) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          uint32_t a[4];
          load_A<D>(a, smem + L::kQ1, r0, kk, lane);
#pragma unroll
          for (int nj = 0; nj < BN / 16; ++nj) {
            uint32_t bb[4];
            load_B_nk<D>(bb, st + L::kStK1, nj * 16, kk, lane);
            Elem<T>::mma(s[2 * nj], a, bb[0], bb[1]);
            Elem<T>::mma(s[2 * nj + 1], a, bb[2], bb[3]);
          }
        }
      }
      if (PW && c.need2) {
        float s2[BN / 8][4];
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) s2[j][0] = s2[j][1] = s2[j][2] = s2[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          uint32_t a[4];
          load_A<D>(a, smem + L::kQ2, r0, kk, lane);
#pragma unroll
          for (int nj = 0; nj < BN / 16; ++nj) {
            uint32_t bb[4];
            load_B_nk<D>(bb, st + L::kStK2, nj * 16, kk, lane);
            Elem<T>::mma(s2[2 * nj], a, bb[0], bb[1]);
            Elem<T>::mma(s2[2 * nj + 1], a, bb[2], bb[3]);
          }
        }
#pragma unroll
        for (int j = 0; j < BN / 8; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            int row = row_g[e >> 1], col = n0 + j * 8 + 2 * t4 + (e & 1);
            if (!c.need1 || row + p_seq - col >= p.w) s[j][e] = s2[j][e];
          }
      }

      // P
#pragma unroll
      for (int j = 0; j < BN / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = row_g[e >> 1], col = n0 + j * 8 + 2 * t4 + (e & 1);
          const bool ok = row < p.M && col < p.N && (!p.causal || row + p_seq >= col);
          const float pv = fast_exp2(s[j][e] * qk_scale - lse_r[e >> 1]);
          s[j][e] = ok ? pv : 0.f;
        }

      // dP = dO V^T
      float dp[BN / 8][4];
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) dp[j][0] = dp[j][1] = dp[j][2] = dp[j][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        load_A<D>(a, smem + L::kDO, r0, kk, lane);
#pragma unroll
        for (int nj = 0; nj < BN / 16; ++nj) {
          uint32_t bb[4];
          load_B_nk<D>(bb, st + L::kStV, nj * 16, kk, lane);
          Elem<T>::mma(dp[2 * nj], a, bb[0], bb[1]);
          Elem<T>::mma(dp[2 * nj + 1], a, bb[2], bb[3]);
        }
      }

      // dropout: dP is masked and scaled like the probabilities were in the forward pass
      if (!PW && p.dropout_p > 0.f) {
        const float rp = 1.f / (1.f - p.dropout_p);
#pragma unroll
        for (int j = 0; j < BN / 8; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int row = row_g[e >> 1], col = n0 + j * 8 + 2 * t4 + (e & 1);
            const uint64_t idx = (((uint64_t)b * p.H + h) * p.M + row) * p.N + col;
            dp[j][e] = dropout_keep(p.seed, p.offset, idx, p.dropout_p) ? dp[j][e] * rp : 0.f;
          }
      }

      // dS, routed to this pass's branch
#pragma unroll
      for (int j = 0; j < BN / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float ds = s[j][e] * (dp[j][e] - delta_r[e >> 1]);
          if (PW) {
            const int row = row_g[e >> 1], col = n0 + j * 8 + 2 * t4 + (e & 1);
            const bool far = row + p_seq - col >= p.w;
            if (far != (pass == 1)) ds = 0.f;
          }
          s[j][e] = ds;
        }

      // dQ += dS K
      const uint32_t kt = st + ((PW && pass == 1) ? L::kStK2 : L::kStK1);
#pragma unroll
      for (int kj = 0; kj < BN / 16; ++kj) {
        uint32_t a[4];
        a[0] = Elem<T>::pack(s[2 * kj][0], s[2 * kj][1]);
        a[1] = Elem<T>::pack(s[2 * kj][2], s[2 * kj][3]);
        a[2] = Elem<T>::pack(s[2 * kj + 1][0], s[2 * kj + 1][1]);
        a[3] = Elem<T>::pack(s[2 * kj + 1][2], s[2 * kj + 1][3]);
#pragma unroll
        for (int dj = 0; dj < D / 16; ++dj) {
          uint32_t bb[4];
          load_B_kn<D>(bb, kt, kj * 16, dj * 2, lane);
          Elem<T>::mma(dq[2 * dj], a, bb[0], bb[1]);
          Elem<T>::mma(dq[2 * dj + 1], a, bb[2], bb[3]);
        }
      }
      __syncthreads();
    }
    cp_async_wait<0>();

    // store dQ of this pass through this warp's rows of stage memory
    {
      void *dst = (PW && pass == 1) ? p.dq2 : p.dq;
      const Strides sd = (PW && pass == 1) ? p.sdq2 : p.sdq;
      uint8_t *buf = smem_raw + L::kStage0;  // 2 stages >= BM rows x D
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = r0 + g + 8 * i;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
          uint32_t v = Elem<T>::pack(dq[j][2 * i] * p.sm_scale, dq[j][2 * i + 1] * p.sm_scale);
          *reinterpret_cast<uint32_t *>(buf + Tile<D>::offset(r, j) + t4 * 4) = v;
        }
      }
      __syncwarp();
      constexpr int CPR = D / 8;
#pragma unroll
      for (int i = 0; i < 16 * CPR / 32; ++i) {
        const int idx = lane + i * 32;
        const int r = idx / CPR, ch = idx % CPR;
        const int row = m0 + r0 + r;
        if (row < p.M) {
          uint4 v = *reinterpret_cast<const uint4 *>(buf + Tile<D>::offset(r0 + r, ch));
          *reinterpret_cast<uint4 *>(row_ptr_mut<T>(dst, sd, b, h, row) + ch * 8) = v;
        }
      }
      __syncthreads();
    }
  }
}

// ---------------------------------------------------------------------------
// total attention: tot[b,h,n] = sum_m P[m,n]
// ---------------------------------------------------------------------------
template <int D, int BM, int BN>
struct TotSmemLayout {
  static constexpr int kK = 0;
  static constexpr int kStage0 = BN * D * 2;
  static constexpr int kStLse = BM * D * 2;
  static constexpr int kStageBytes = kStLse + BM * 4;
  static constexpr int kTotal = kStage0 + 2 * kStageBytes;
};

template <typename T, int D, int BM, int BN>
__global__ void __launch_bounds__(BN / 16 * 32)
    total_attention_kernel(const void *q, Strides sq, const void *k, Strides sk, const float *lse,
                           float *total, int B, int H, int Hk, int M, int N, int causal,
                           float sm_scale) {
  constexpr int NW = BN / 16, NT = NW * 32;
  using L = TotSmemLayout<D, BM, BN>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const uint32_t smem = smem_u32(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int n0 = blockIdx.x * BN;
  const int b = blockIdx.y / H, h = blockIdx.y % H;
  const int hk = h / (H / Hk);
  const int p_seq = N - M;
  const float qk_scale = sm_scale * kLog2e;
  const int kr0 = warp * 16;
  const int key_g[2] = {n0 + kr0 + g, n0 + kr0 + g + 8};

  load_tile_async<T, D, BN, NT>(smem + L::kK, row_ptr<T>(k, sk, b, hk, n0), sk.l, N - n0, tid);
  cp_async_commit();

  const int num_m_tiles = (M + BM - 1) / BM;
  int mt_lo = 0;
  if (causal) mt_lo = max(0, n0 - p_seq) / BM;
  const int iters = max(0, num_m_tiles - mt_lo);

  auto issue = [&](int it) {
    const int m0 = (mt_lo + it) * BM;
    const uint32_t st = smem + L::kStage0 + (it & 1) * L::kStageBytes;
    load_tile_async<T, D, BM, NT>(st, row_ptr<T>(q, sq, b, h, m0), sq.l, M - m0, tid);
    load_floats_async(st + L::kStLse, lse + ((int64_t)b * H + h) * M + m0, BM, M - m0, tid, NT);
  };
  if (iters > 0) issue(0);
  cp_async_commit();

  float tot[2] = {0.f, 0.f};
#pragma unroll 1
  for (int it = 0; it < iters; ++it) {
    if (it + 1 < iters) {
      issue(it + 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int m0 = (mt_lo + it) * BM;
    const uint32_t st = smem + L::kStage0 + (it & 1) * L::kStageBytes;
    const float *lse_s = reinterpret_cast<const float *>(smem_raw + L::kStage0 +
                                                         (it & 1) * L::kStageBytes + L::kStLse);
    float s[BM / 8][4];
#pragma unroll
    for (int j = 0; j < BM / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a[4];
      load_A<D>(a, smem + L::kK, kr0, kk, lane);
#pragma unroll
      for (int mj = 0; mj < BM / 16; ++mj) {
        uint32_t bb[4];
        load_B_nk<D>(bb, st, mj * 16, kk, lane);
        Elem<T>::mma(s[2 * mj], a, bb[0], bb[1]);
        Elem<T>::mma(s[2 * mj + 1], a, bb[2], bb[3]);
      }
    }
#pragma unroll
    for (int j = 0; j < BM / 8; ++j) {
      const float2 l2 = *reinterpret_cast<const float2 *>(lse_s + j * 8 + 2 * t4);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key_g[e >> 1], qm = m0 + j * 8 + 2 * t4 + (e & 1);
        const float lv = (e & 1) ? l2.y : l2.x;
        const bool ok = qm < M && key < N && (!causal || qm + p_seq >= key);
        const float pv = fast_exp2(s[j][e] * qk_scale - lv * kLog2e);
        if (ok) tot[e >> 1] += pv;
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float v = quad_sum(tot[i]);
    if (t4 == 0 && key_g[i] < N) total[((int64_t)b * H + h) * N + key_g[i]] = v;
  }
}

}  // namespace fa
