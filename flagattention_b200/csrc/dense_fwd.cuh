// Shape-generic forward kernel for flash_attention, piecewise_attention and
// the split-KV stage 1: FA2-style online softmax on m16n8k16 tensor-core MMAs,
// K/V tiles double-buffered through swizzled shared memory with cp.async.
// It covers every head_dim, ragged M/N, arbitrary strides and empty causal
// rows; the tcgen05 kernels take over the large aligned shapes.
#pragma once

#include "attn_params.cuh"

namespace fa {

template <int D, int BM, int BN, bool PW>
struct FwdSmemLayout {
  static constexpr int kQBytes = BM * D * 2;
  static constexpr int kKVBytes = BN * D * 2;
  static constexpr int kStageTiles = PW ? 3 : 2;  // K1,(K2),V
  static constexpr int kStageBytes = kStageTiles * kKVBytes;
  static constexpr int kQ1 = 0;
  static constexpr int kQ2 = kQBytes;
  static constexpr int kStage0 = (PW ? 2 : 1) * kQBytes;
  static constexpr int kTotal = kStage0 + 2 * kStageBytes;
};

template <typename T, int D, int BM, int BN, bool PW, bool SPLIT>
__global__ void __launch_bounds__(BM / 16 * 32) dense_fwd_kernel(const FwdParams p) {
  constexpr int NW = BM / 16, NT = NW * 32;
  using L = FwdSmemLayout<D, BM, BN, PW>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const uint32_t smem = smem_u32(smem_raw);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;

  const int mb = gridDim.x - 1 - blockIdx.x;  // heaviest causal tiles first
  const int b = blockIdx.y / p.H, h = blockIdx.y % p.H;
  const int hk = h / (p.H / p.Hk);
  const int split = SPLIT ? blockIdx.z : 0;
  const int m0 = mb * BM;
  const int p_seq = p.N - p.M;

  int n_lo = SPLIT ? split * p.n_split_size : 0;
  int n_end = SPLIT ? min(p.N, n_lo + p.n_split_size) : p.N;  // end before causal clamp
  int n_hi = n_end;
  if (p.causal) n_hi = min(n_hi, p_seq + m0 + BM);
  const int num_tiles = n_hi > n_lo ? (n_hi - n_lo + BN - 1) / BN : 0;

  const float qk_scale = p.sm_scale * kLog2e;

  // ---- async loads -------------------------------------------------------
  const T *qg = row_ptr<T>(p.q, p.sq, b, h, m0);
  load_tile_async<T, D, BM, NT>(smem + L::kQ1, qg, p.sq.l, p.M - m0, tid);
  if (PW) {
    const T *q2g = row_ptr<T>(p.q2, p.sq2, b, h, m0);
    load_tile_async<T, D, BM, NT>(smem + L::kQ2, q2g, p.sq2.l, p.M - m0, tid);
  }
  auto issue_tile = [&](int t) {
    const int n0 = n_lo + t * BN;
    const uint32_t st = smem + L::kStage0 + (t & 1) * L::kStageBytes;
    PwClass c{true, false};
    if (PW) c = pw_classify(m0, BM, n0, BN, p_seq, p.w);
    if (c.need1)
      load_tile_async<T, D, BN, NT>(st, row_ptr<T>(p.k, p.sk, b, hk, n0), p.sk.l, p.N - n0, tid);
    if (PW && c.need2)
      load_tile_async<T, D, BN, NT>(st + 2 * L::kKVBytes, row_ptr<T>(p.k2, p.sk2, b, hk, n0),
                                    p.sk2.l, p.N - n0, tid);
    load_tile_async<T, D, BN, NT>(st + L::kKVBytes, row_ptr<T>(p.v, p.sv, b, hk, n0), p.sv.l,
                                  p.N - n0, tid);
  };
  if (num_tiles > 0) issue_tile(0);
  cp_async_commit();

  // ---- running state -----------------------------------------------------
  float acc[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  float m_i[2] = {-INFINITY, -INFINITY};
  float l_i[2] = {0.f, 0.f};  // per-thread partial row sums (quad-reduced at the end)
  const int r0 = warp * 16;
  const int row_g[2] = {m0 + r0 + g, m0 + r0 + g + 8};

  for (int t = 0; t < num_tiles; ++t) {
    if (t + 1 < num_tiles) {
      issue_tile(t + 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    const int n0 = n_lo + t * BN;
    const uint32_t st = smem + L::kStage0 + (t & 1) * L::kStageBytes;
    const uint32_t kt = st, vt = st + L::kKVBytes, k2t = st + 2 * L::kKVBytes;
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
          load_B_nk<D>(bb, kt, nj * 16, kk, lane);
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
          load_B_nk<D>(bb, k2t, nj * 16, kk, lane);
          Elem<T>::mma(s2[2 * nj], a, bb[0], bb[1]);
          Elem<T>::mma(s2[2 * nj + 1], a, bb[2], bb[3]);
        }
      }
      if (!c.need1) {
#pragma unroll
        for (int j = 0; j < BN / 8; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) s[j][e] = s2[j][e];
      } else {
#pragma unroll
        for (int j = 0; j < BN / 8; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            int row = row_g[e >> 1], col = n0 + j * 8 + 2 * t4 + (e & 1);
            if (row + p_seq - col >= p.w) s[j][e] = s2[j][e];
          }
      }
    }

    // scale into the base-2 domain, then mask
    const bool need_mask = (n0 + BN > n_end) || (p.causal && (n0 + BN - 1 > m0 + p_seq));
#pragma unroll
    for (int j = 0; j < BN / 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] *= qk_scale;
    if (need_mask) {
#pragma unroll
      for (int j = 0; j < BN / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int row = row_g[e >> 1], col = n0 + j * 8 + 2 * t4 + (e & 1);
          bool ok = col < n_end && (!p.causal || row + p_seq >= col);
          if (!ok) s[j][e] = -INFINITY;
        }
    }

    // online softmax
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) mx = fmaxf(mx, fmaxf(s[j][2 * i], s[j][2 * i + 1]));
      mx = quad_max(mx);
      const float m_new = fmaxf(m_i[i], mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = fast_exp2(m_i[i] - m_use);
      float rs = 0.f;
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) {
        float p0 = fast_exp2(s[j][2 * i] - m_use);
        float p1 = fast_exp2(s[j][2 * i + 1] - m_use);
        s[j][2 * i] = p0;
        s[j][2 * i + 1] = p1;
        rs += p0 + p1;
      }
      l_i[i] = l_i[i] * alpha + rs;
      m_i[i] = m_new;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        acc[j][2 * i] *= alpha;
        acc[j][2 * i + 1] *= alpha;
      }
    }

    // dropout acts on the probabilities that enter P V; the row sums above stay undropped
    if (!SPLIT && p.dropout_p > 0.f) {
#pragma unroll
      for (int j = 0; j < BN / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = row_g[e >> 1], col = n0 + j * 8 + 2 * t4 + (e & 1);
          const uint64_t idx = (((uint64_t)b * p.H + h) * p.M + row) * p.N + col;
          if (!dropout_keep(p.seed, p.offset, idx, p.dropout_p)) s[j][e] = 0.f;
        }
    }

    // O += P V
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
        load_B_kn<D>(bb, vt, kj * 16, dj * 2, lane);
        Elem<T>::mma(acc[2 * dj], a, bb[0], bb[1]);
        Elem<T>::mma(acc[2 * dj + 1], a, bb[2], bb[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  // The epilogue stages O in the Q tile.  With no key tile to visit the loop above never ran its
  // barrier, and another thread's asynchronous copy of Q could still land in this warp's rows
  // after the staged O: wait for everybody's copies first.
  if (num_tiles == 0) __syncthreads();

  // ---- epilogue ------------------------------------------------------------
  float inv[2], lse[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float l = quad_sum(l_i[i]);
    inv[i] = l > 0.f ? 1.f / l : 0.f;
    if (!SPLIT && p.dropout_p > 0.f) inv[i] *= 1.f / (1.f - p.dropout_p);
    lse[i] = l > 0.f ? m_i[i] * kLn2 + logf(l) : -INFINITY;
  }

  if (SPLIT) {
    // fp32 partials, (B,H,S,M,D) and (B,H,S,M)
    const int64_t base = (((int64_t)b * p.H + h) * p.num_splits + split) * p.M;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = row_g[i];
      if (row < p.M) {
        float *orow = p.o_partial + (base + row) * D;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
          float2 val = make_float2(acc[j][2 * i] * inv[i], acc[j][2 * i + 1] * inv[i]);
          *reinterpret_cast<float2 *>(orow + j * 8 + 2 * t4) = val;
        }
        if (t4 == 0) p.lse_partial[base + row] = lse[i];
      }
    }
    return;
  }

  // stage O through this warp's rows of the Q tile for 16-byte coalesced stores
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = r0 + g + 8 * i;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      uint32_t v = Elem<T>::pack(acc[j][2 * i] * inv[i], acc[j][2 * i + 1] * inv[i]);
      *reinterpret_cast<uint32_t *>(smem_raw + L::kQ1 + Tile<D>::offset(r, j) + t4 * 4) = v;
    }
    if (t4 == 0 && row_g[i] < p.M)
      p.lse[((int64_t)b * p.H + h) * p.M + row_g[i]] = lse[i];
  }
  __syncwarp();
  constexpr int CPR = D / 8;
#pragma unroll
  for (int i = 0; i < 16 * CPR / 32; ++i) {
    const int idx = lane + i * 32;
    const int r = idx / CPR, ch = idx % CPR;
    const int row = m0 + r0 + r;
    if (row < p.M) {
      uint4 v = *reinterpret_cast<const uint4 *>(smem_raw + L::kQ1 + Tile<D>::offset(r0 + r, ch));
      *reinterpret_cast<uint4 *>(row_ptr_mut<T>(p.o, p.so, b, h, row) + ch * 8) = v;
    }
  }
}

// Stage 2 of split-KV: one thread per (row, 4 columns).
template <typename T>
__global__ void splitkv_combine_kernel(const float *__restrict__ o_partial,
                                       const float *__restrict__ lse_partial, void *o, Strides so,
                                       float *lse, int B, int H, int M, int D, int S) {
  const int vec_per_row = D / 4;
  const int64_t total = (int64_t)B * H * M * vec_per_row;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(idx % vec_per_row);
    const int64_t rowid = idx / vec_per_row;  // (b*H + h)*M + m
    const int m = (int)(rowid % M);
    const int64_t bh = rowid / M;
    const float *lp = lse_partial + bh * S * M + m;
    float mx = -INFINITY;
    for (int s = 0; s < S; ++s) mx = fmaxf(mx, lp[(int64_t)s * M]);
    float den = 0.f;
    float4 accv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (mx != -INFINITY) {
      for (int s = 0; s < S; ++s) {
        const float wgt = __expf(lp[(int64_t)s * M] - mx);
        den += wgt;
        const float4 v = *reinterpret_cast<const float4 *>(
            o_partial + ((bh * S + s) * M + m) * (int64_t)D + c * 4);
        accv.x += wgt * v.x;
        accv.y += wgt * v.y;
        accv.z += wgt * v.z;
        accv.w += wgt * v.w;
      }
      const float r = 1.f / den;
      accv.x *= r, accv.y *= r, accv.z *= r, accv.w *= r;
    }
    const int b = (int)(bh / H), h = (int)(bh % H);
    T *orow = row_ptr_mut<T>(o, so, b, h, m) + c * 4;
    uint2 packed;
    packed.x = Elem<T>::pack(accv.x, accv.y);
    packed.y = Elem<T>::pack(accv.z, accv.w);
    *reinterpret_cast<uint2 *>(orow) = packed;
    if (c == 0) lse[rowid] = (mx == -INFINITY) ? -INFINITY : mx + logf(den);
  }
}

}  // namespace fa
