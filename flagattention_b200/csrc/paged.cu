// paged_attention decode: block-table-indexed gather of the KV cache with
// online softmax, optional split-KV partitions and the partition reducer.
//
// HBM-bound by design: every warp of a CTA streams its own 16-token groups of
// K and V through a private multi-stage cp.async ring (16-byte coalesced
// gathers, swizzled shared memory), so nothing in the main loop needs a
// CTA-wide barrier.  The tiny GEMMs (query group padded to 16 rows) run on
// m16n8k16 tensor-core MMAs so that arithmetic never limits the stream.
#include "common.cuh"

namespace fa {

template <typename IdxT>
__device__ __forceinline__ int64_t phys_block(const void *block_tables, int64_t bt_stride_s,
                                              int seq, int logical_block) {
  return (int64_t) reinterpret_cast<const IdxT *>(block_tables)[(int64_t)seq * bt_stride_s +
                                                                logical_block];
}

template <int D>
struct PagedCfg {
  static constexpr int kWarps = D <= 128 ? 4 : 2;
  static constexpr int kStages = D <= 64 ? 4 : 3;
  static constexpr int kGroupBytes = 16 * D * 2;             // one 16-token K or V group
  static constexpr int kStageBytes = 2 * kGroupBytes;        // K + V
  static constexpr int kWarpBytes = kStages * kStageBytes;
  static constexpr int kQBytes = 16 * D * 2;
  static constexpr int kStatBytes = 2 * kWarps * 16 * 4;     // m, l per warp per row
  static constexpr int kRing = kQBytes + kStatBytes;
  static constexpr int kRingBytes = kWarps * kWarpBytes;
  static constexpr int kMergeBytes = kWarps * 16 * D * 4;    // fp32 partial outputs, aliases ring
  static constexpr int kTotal = kRing + (kRingBytes > kMergeBytes ? kRingBytes : kMergeBytes);
};

template <typename T, int D, typename IdxT>
__global__ void __launch_bounds__(PagedCfg<D>::kWarps * 32) paged_decode_kernel(
    const fa_paged_args a) {
  using C = PagedCfg<D>;
  constexpr int NW = C::kWarps, NS = C::kStages, CPR = D / 8;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const uint32_t smem = smem_u32(smem_raw);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int seq = blockIdx.x;
  const int G = a.num_q_heads / a.num_kv_heads;
  const int q_tiles = (G + 15) / 16;
  const int hk = blockIdx.y / q_tiles, qt = blockIdx.y % q_tiles;
  const int part = blockIdx.z;
  const int rows = min(16, G - qt * 16);          // valid query rows of this CTA
  const int qh0 = hk * G + qt * 16;               // first query head

  const int ctx = a.context_lens[seq];
  const int t_begin = a.partition_size > 0 ? part * a.partition_size : 0;
  if (a.partition_size > 0 && t_begin >= ctx) return;
  const int t_end = a.partition_size > 0 ? min(ctx, t_begin + a.partition_size) : ctx;
  const int BS = a.block_size;
  const bool group_in_block = (BS % 16 == 0) && (t_begin % 16 == 0);
  // Several queries per head (a.causal_rows = Mq > 0): query head index = head * Mq + m, and query
  // m of a head is the (Mq - 1 - m)-th from the end of the sequence, so it sees the tokens below
  // ctx - (Mq - 1 - m).  This thread's two accumulator rows are g and g + 8 of the tile.
  int row_end[2] = {t_end, t_end};
  if (a.causal_rows > 0) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int m = (qt * 16 + g + 8 * r) % a.causal_rows;
      row_end[r] = min(t_end, ctx - (a.causal_rows - 1 - m));
    }
  }

  // ---- query group -> shared (rows >= `rows` are zero) ---------------------
  {
    const T *qg = reinterpret_cast<const T *>(a.query) + (int64_t)seq * a.q_stride_s;
    for (int idx = tid; idx < 16 * CPR; idx += NW * 32) {
      const int r = idx / CPR, ch = idx % CPR;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < rows)
        v = *reinterpret_cast<const uint4 *>(qg + (int64_t)(qh0 + r) * a.q_stride_h + ch * 8);
      *reinterpret_cast<uint4 *>(smem_raw + Tile<D>::offset(r, ch)) = v;
    }
  }
  __syncthreads();

  constexpr bool kQInRegs = D <= 128;
  uint32_t qf[kQInRegs ? D / 16 : 1][4];
  if (kQInRegs) {
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) load_A<D>(qf[kk], smem, 0, kk, lane);
  }

  // ---- this warp's token groups ---------------------------------------------
  const int n_groups = (t_end - t_begin + 15) / 16;           // groups of the CTA
  const int my_groups = n_groups > warp ? (n_groups - warp + NW - 1) / NW : 0;
  const uint32_t ring = smem + C::kRing + warp * C::kWarpBytes;
  const T *kc = reinterpret_cast<const T *>(a.key_cache) + (int64_t)hk * a.kv_stride_h;
  const T *vc = reinterpret_cast<const T *>(a.value_cache) + (int64_t)hk * a.kv_stride_h;

  // Per-lane constants of the gather.  In every 16-token group this lane copies the 16-byte
  // chunk `ch` of rows c * RPC + lane_r (c = 0..NC-1), for K and for V, so the shared-memory
  // offsets are fixed and the global address only advances by RPC rows per step.
  constexpr int NC = 16 * CPR / 32;  // copy steps per lane per group
  constexpr int RPC = 16 / NC;       // rows covered per step
  const int lane_r = lane / CPR, ch = lane % CPR;
  uint32_t dst_off[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) dst_off[c] = Tile<D>::offset(c * RPC + lane_r, ch);
  const int64_t lane_src = (int64_t)lane_r * a.kv_stride_t + ch * 8;
  const int64_t c_step = (int64_t)RPC * a.kv_stride_t;
  const int64_t v_minus_k = vc - kc;
  const int bs_shift = (BS & (BS - 1)) == 0 ? 31 - __clz(BS) : -1;

  auto issue = [&](int i) {  // i-th group of this warp -> stage i % NS
    const int tok0 = t_begin + (warp + i * NW) * 16;
    const uint32_t st = ring + (i % NS) * C::kStageBytes;
    if (group_in_block) {
      // the whole group lies in one physical block: one table lookup, then pointer increments
      const int lb = bs_shift >= 0 ? tok0 >> bs_shift : tok0 / BS;
      const int in_blk = tok0 - lb * BS;
      const int64_t pb = phys_block<IdxT>(a.block_tables, a.bt_stride_s, seq, lb);
      const T *src = kc + pb * a.kv_stride_b + (int64_t)in_blk * a.kv_stride_t + lane_src;
      const int rows_left = t_end - tok0 - lane_r;  // row c*RPC + lane_r exists iff c*RPC < rows_left
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const bool ok = c * RPC < rows_left;
        const T *sk = ok ? src : kc;
        cp_async16(st + dst_off[c], sk, ok);
        cp_async16(st + C::kGroupBytes + dst_off[c], sk + v_minus_k, ok);
        src += c_step;
      }
    } else {
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int tok = tok0 + c * RPC + lane_r;
        const bool ok = tok < t_end;
        int64_t off = 0;
        if (ok) {
          const int64_t pb = phys_block<IdxT>(a.block_tables, a.bt_stride_s, seq, tok / BS);
          off = pb * a.kv_stride_b + (int64_t)(tok % BS) * a.kv_stride_t + ch * 8;
        }
        cp_async16(st + dst_off[c], kc + off, ok);
        cp_async16(st + C::kGroupBytes + dst_off[c], vc + off, ok);
      }
    }
  };

#pragma unroll
  for (int i = 0; i < NS - 1; ++i) {
    if (i < my_groups) issue(i);
    cp_async_commit();
  }

  float acc[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  float m_i[2] = {-INFINITY, -INFINITY};
  float l_i[2] = {0.f, 0.f};
  const float qk_scale = a.attn_scale * kLog2e;

#pragma unroll 1
  for (int i = 0; i < my_groups; ++i) {
    if (i + NS - 1 < my_groups) issue(i + NS - 1);
    cp_async_commit();
    cp_async_wait<NS - 1>();
    __syncwarp();

    const int tok0 = t_begin + (warp + i * NW) * 16;
    const uint32_t st = ring + (i % NS) * C::kStageBytes;

    float s[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t bb[4];
      load_B_nk<D>(bb, st, 0, kk, lane);
      if (kQInRegs) {
        Elem<T>::mma(s[0], qf[kk], bb[0], bb[1]);
        Elem<T>::mma(s[1], qf[kk], bb[2], bb[3]);
      } else {
        uint32_t qa[4];
        load_A<D>(qa, smem, 0, kk, lane);
        Elem<T>::mma(s[0], qa, bb[0], bb[1]);
        Elem<T>::mma(s[1], qa, bb[2], bb[3]);
      }
    }
    const bool tail = tok0 + 16 > min(row_end[0], row_end[1]);
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = tok0 + j * 8 + 2 * t4 + (e & 1);
        s[j][e] = (tail && tok >= row_end[e >> 1]) ? -INFINITY : s[j][e] * qk_scale;
      }
    // Running maximum with lazy rescaling: the accumulators are only rescaled when some row's
    // maximum grew by more than 2^8 (scores are already in the base-2 domain); otherwise the
    // stale maximum stays the reference point and P simply ranges up to 2^8.
    float m_new[2];
    bool need = false;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = fmaxf(fmaxf(s[0][2 * r], s[0][2 * r + 1]), fmaxf(s[1][2 * r], s[1][2 * r + 1]));
      mx = quad_max(mx);
      m_new[r] = fmaxf(m_i[r], mx);  // -inf only while a row has not seen a token it may see
      need = need || (m_new[r] - m_i[r] > 8.f);
    }
    if (__any_sync(0xffffffffu, need)) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float alpha = (m_new[r] == -INFINITY) ? 1.f : fast_exp2(m_i[r] - m_new[r]);
        l_i[r] *= alpha;
        m_i[r] = m_new[r];
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
          acc[j][2 * r] *= alpha;
          acc[j][2 * r + 1] *= alpha;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float rs = 0.f;
      const float m_ref = (m_i[r] == -INFINITY) ? 0.f : m_i[r];   // all scores -inf: P = 0
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        s[j][2 * r] = fast_exp2(s[j][2 * r] - m_ref);
        s[j][2 * r + 1] = fast_exp2(s[j][2 * r + 1] - m_ref);
        rs += s[j][2 * r] + s[j][2 * r + 1];
      }
      l_i[r] += rs;
    }
    uint32_t pa[4];
    pa[0] = Elem<T>::pack(s[0][0], s[0][1]);
    pa[1] = Elem<T>::pack(s[0][2], s[0][3]);
    pa[2] = Elem<T>::pack(s[1][0], s[1][1]);
    pa[3] = Elem<T>::pack(s[1][2], s[1][3]);
#pragma unroll
    for (int dj = 0; dj < D / 16; ++dj) {
      uint32_t bb[4];
      load_B_kn<D>(bb, st + C::kGroupBytes, 0, dj * 2, lane);
      Elem<T>::mma(acc[2 * dj], pa, bb[0], bb[1]);
      Elem<T>::mma(acc[2 * dj + 1], pa, bb[2], bb[3]);
    }
    __syncwarp();  // stage may be refilled by the next iteration's issue
  }
  cp_async_wait<0>();

  // ---- merge the warps' partial states --------------------------------------
  float *stat_m = reinterpret_cast<float *>(smem_raw + C::kQBytes);
  float *stat_l = stat_m + NW * 16;
  float *merge = reinterpret_cast<float *>(smem_raw + C::kRing);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const float l = quad_sum(l_i[r]);
    if (t4 == 0) {
      stat_m[warp * 16 + g + 8 * r] = m_i[r];
      stat_l[warp * 16 + g + 8 * r] = l;
    }
  }
  __syncthreads();  // stats visible; every warp has drained its ring
  float m_all[2], scale_w[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = g + 8 * r;
    float mm = -INFINITY;
#pragma unroll
    for (int w2 = 0; w2 < NW; ++w2) mm = fmaxf(mm, stat_m[w2 * 16 + row]);
    m_all[r] = mm;
    scale_w[r] = (m_i[r] == -INFINITY) ? 0.f : fast_exp2(m_i[r] - mm);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = g + 8 * r;
    if (row < rows) {
      float *dst = merge + ((int64_t)warp * 16 + row) * D;
#pragma unroll
      for (int j = 0; j < D / 8; ++j)
        *reinterpret_cast<float2 *>(dst + j * 8 + 2 * t4) =
            make_float2(acc[j][2 * r] * scale_w[r], acc[j][2 * r + 1] * scale_w[r]);
    }
  }
  __syncthreads();

  for (int idx = tid; idx < rows * (D / 4); idx += NW * 32) {
    const int row = idx / (D / 4), c4 = idx % (D / 4);
    float mm = -INFINITY;
#pragma unroll
    for (int w2 = 0; w2 < NW; ++w2) mm = fmaxf(mm, stat_m[w2 * 16 + row]);
    float l = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w2 = 0; w2 < NW; ++w2) {
      const float mw = stat_m[w2 * 16 + row];
      if (mw != -INFINITY) l += stat_l[w2 * 16 + row] * fast_exp2(mw - mm);
      const float4 v = *reinterpret_cast<const float4 *>(merge + ((int64_t)w2 * 16 + row) * D + c4 * 4);
      o.x += v.x, o.y += v.y, o.z += v.z, o.w += v.w;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    o.x *= inv, o.y *= inv, o.z *= inv, o.w *= inv;
    const int qh = qh0 + row;
    if (a.partition_size > 0) {
      const int P = (a.max_context_len + a.partition_size - 1) / a.partition_size;
      const int64_t pi = ((int64_t)seq * a.num_q_heads + qh) * P + part;
      *reinterpret_cast<float4 *>(a.part_out + pi * D + c4 * 4) = o;
      if (c4 == 0) {
        a.part_max[pi] = mm;
        a.part_sum[pi] = l;
      }
    } else {
      T *dst = reinterpret_cast<T *>(a.out) + (int64_t)seq * a.o_stride_s +
               (int64_t)qh * a.o_stride_h + c4 * 4;
      uint2 pk;
      pk.x = Elem<T>::pack(o.x, o.y);
      pk.y = Elem<T>::pack(o.z, o.w);
      *reinterpret_cast<uint2 *>(dst) = pk;
    }
  }
  (void)m_all;
}

// One CTA per (seq, query head); thread d4 owns 4 output columns.
template <typename T>
__global__ void paged_reduce_kernel(const fa_paged_args a) {
  const int seq = blockIdx.x, qh = blockIdx.y;
  const int D = a.head_size;
  const int P = (a.max_context_len + a.partition_size - 1) / a.partition_size;
  const int ctx = a.context_lens[seq];
  const int np = min(P, (ctx + a.partition_size - 1) / a.partition_size);
  const int64_t base = ((int64_t)seq * a.num_q_heads + qh) * P;
  float mm = -INFINITY;
  for (int p = 0; p < np; ++p) mm = fmaxf(mm, a.part_max[base + p]);
  for (int c4 = threadIdx.x; c4 < D / 4; c4 += blockDim.x) {
    float den = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < np; ++p) {
      const float wgt = a.part_sum[base + p] * fast_exp2(a.part_max[base + p] - mm);
      den += wgt;
      const float4 v = *reinterpret_cast<const float4 *>(a.part_out + (base + p) * D + c4 * 4);
      o.x += wgt * v.x, o.y += wgt * v.y, o.z += wgt * v.z, o.w += wgt * v.w;
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    T *dst = reinterpret_cast<T *>(a.out) + (int64_t)seq * a.o_stride_s +
             (int64_t)qh * a.o_stride_h + c4 * 4;
    uint2 pk;
    pk.x = Elem<T>::pack(o.x * inv, o.y * inv);
    pk.y = Elem<T>::pack(o.z * inv, o.w * inv);
    *reinterpret_cast<uint2 *>(dst) = pk;
  }
}

template <typename IdxT>
__global__ void paged_trace_kernel(const fa_paged_args a, int64_t *visited, int max_blocks) {
  const int seq = blockIdx.x;
  const int ctx = a.context_lens[seq];
  const int used = (ctx + a.block_size - 1) / a.block_size;
  for (int blk = threadIdx.x; blk < max_blocks; blk += blockDim.x)
    visited[(int64_t)seq * max_blocks + blk] =
        blk < used ? phys_block<IdxT>(a.block_tables, a.bt_stride_s, seq, blk) : -1;
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static int validate_paged(const fa_paged_args *a, bool need_ws) {
  if (!a || !a->query || !a->key_cache || !a->value_cache || !a->context_lens ||
      !a->block_tables || !a->out)
    return FA_ERR_BAD_ARG;
  if (a->dtype != FA_F16 && a->dtype != FA_BF16) return FA_ERR_BAD_ARG;
  if (a->num_seqs <= 0 || a->num_q_heads <= 0 || a->num_kv_heads <= 0 || a->block_size <= 0 ||
      a->max_context_len <= 0 || a->partition_size < 0)
    return FA_ERR_BAD_ARG;
  if (a->num_q_heads % a->num_kv_heads != 0) return FA_ERR_BAD_ARG;
  if (a->partition_size % 16 != 0) return FA_ERR_BAD_ARG;
  if (a->causal_rows < 0 || (a->causal_rows > 0 && (a->num_q_heads / a->num_kv_heads) % a->causal_rows != 0))
    return FA_ERR_BAD_ARG;
  const int D = a->head_size;
  if (!(D == 16 || D == 32 || D == 64 || D == 128 || D == 256)) return FA_ERR_UNSUPPORTED;
  if (!aligned16(a->query) || !aligned16(a->key_cache) || !aligned16(a->value_cache) ||
      !aligned16(a->out))
    return FA_ERR_ALIGNMENT;
  if (a->q_stride_s % 8 || a->q_stride_h % 8 || a->kv_stride_b % 8 || a->kv_stride_h % 8 ||
      a->kv_stride_t % 8 || a->o_stride_s % 4 || a->o_stride_h % 4)
    return FA_ERR_ALIGNMENT;
  if (need_ws && a->partition_size > 0 && (!a->part_out || !a->part_max || !a->part_sum))
    return FA_ERR_WORKSPACE;
  return FA_OK;
}

template <typename T, int D, typename IdxT>
static int launch_paged(const fa_paged_args *a, cudaStream_t stream) {
  using C = PagedCfg<D>;
  auto kern = paged_decode_kernel<T, D, IdxT>;
  static unsigned long long attr_done = 0;  // per instantiation, one bit per device
  if (int st = ensure_dyn_smem(kern, C::kTotal, &attr_done)) return st;
  const int G = a->num_q_heads / a->num_kv_heads;
  const int q_tiles = (G + 15) / 16;
  const int P = a->partition_size > 0
                    ? (a->max_context_len + a->partition_size - 1) / a->partition_size
                    : 1;
  dim3 grid(a->num_seqs, a->num_kv_heads * q_tiles, P);
  kern<<<grid, C::kWarps * 32, C::kTotal, stream>>>(*a);
  FA_CHECK_LAUNCH();
  return FA_OK;
}

template <typename T, typename IdxT>
static int dispatch_paged_d(const fa_paged_args *a, cudaStream_t stream) {
  switch (a->head_size) {
    case 16: return launch_paged<T, 16, IdxT>(a, stream);
    case 32: return launch_paged<T, 32, IdxT>(a, stream);
    case 64: return launch_paged<T, 64, IdxT>(a, stream);
    case 128: return launch_paged<T, 128, IdxT>(a, stream);
    case 256: return launch_paged<T, 256, IdxT>(a, stream);
  }
  return FA_ERR_UNSUPPORTED;
}

}  // namespace fa

using namespace fa;

extern "C" int fa_paged_decode(const fa_paged_args *a, void *stream) {
  int st = validate_paged(a, true);
  if (st != FA_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a->dtype == FA_F16)
    return a->block_table_is_i64 ? dispatch_paged_d<__half, int64_t>(a, s)
                                 : dispatch_paged_d<__half, int32_t>(a, s);
  return a->block_table_is_i64 ? dispatch_paged_d<__nv_bfloat16, int64_t>(a, s)
                               : dispatch_paged_d<__nv_bfloat16, int32_t>(a, s);
}

extern "C" int fa_paged_reduce(const fa_paged_args *a, void *stream) {
  int st = validate_paged(a, true);
  if (st != FA_OK) return st;
  if (a->partition_size <= 0) return FA_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(a->num_seqs, a->num_q_heads);
  const int threads = a->head_size / 4 < 32 ? 32 : a->head_size / 4;
  if (a->dtype == FA_F16)
    paged_reduce_kernel<__half><<<grid, threads, 0, s>>>(*a);
  else
    paged_reduce_kernel<__nv_bfloat16><<<grid, threads, 0, s>>>(*a);
  FA_CHECK_LAUNCH();
  return FA_OK;
}

extern "C" int64_t fa_paged_workspace_bytes(const fa_paged_args *a) {
  if (!a || a->partition_size <= 0) return 0;
  const int64_t P = (a->max_context_len + a->partition_size - 1) / a->partition_size;
  const int64_t rows = (int64_t)a->num_seqs * a->num_q_heads * P;
  return rows * a->head_size * 4 + 2 * rows * 4;
}

extern "C" int fa_paged_trace_blocks(const fa_paged_args *a, int64_t *visited, int32_t max_blocks,
                                     void *stream) {
  int st = validate_paged(a, false);
  if (st != FA_OK) return st;
  if (!visited || max_blocks <= 0) return FA_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a->block_table_is_i64)
    paged_trace_kernel<int64_t><<<a->num_seqs, 256, 0, s>>>(*a, visited, max_blocks);
  else
    paged_trace_kernel<int32_t><<<a->num_seqs, 256, 0, s>>>(*a, visited, max_blocks);
  FA_CHECK_LAUNCH();
  return FA_OK;
}

// ---------------------------------------------------------------------------
// Partitioned decode for callers that have no memory to hand us.
//
// Some hosts of this library cannot supply the split-KV workspace: a serving
// process that gave every spare byte of HBM to its KV-cache pool at start-up
// has nothing left to carve a workspace from, and a decode loop that is
// forbidden from entering the CUDA allocator (it would stall on the allocator
// lock or break its latency budget) cannot create one per call either.  For
// them the partial outputs and softmax statistics live in the fixed array
// below, which is part of the library image: every GPU that loads the library
// carries these FA_PAGED_NOALLOC_SCRATCH_BYTES until the process exits.
//
// `g_paged_scratch` names a device object.  Host code must not treat that name
// as a pointer: it is only a handle from which the real device address is
// looked up, once per device, with cudaGetSymbolAddress while that device is
// current; the address is then what the kernels receive.
// ---------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_paged_scratch[FA_PAGED_NOALLOC_SCRATCH_BYTES];

namespace fa {

static constexpr int kMaxDevices = 64;
static unsigned char *g_paged_scratch_addr[kMaxDevices];  // resolved device addresses, per device

// Looks up (first call on a device) or returns (later calls) the device address of the scratch
// array for the current device.  No allocation happens here or anywhere below.
static int paged_scratch_base(unsigned char **base) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return FA_ERR_LAUNCH;
  if (dev < 0 || dev >= kMaxDevices) return FA_ERR_TOO_LARGE;
  if (!g_paged_scratch_addr[dev]) {
    unsigned char *ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_paged_scratch) != cudaSuccess ||
        !ptr)
      return FA_ERR_LAUNCH;
    g_paged_scratch_addr[dev] = ptr;
  }
  *base = g_paged_scratch_addr[dev];
  return FA_OK;
}

}  // namespace fa

extern "C" int fa_paged_attention_noalloc(const fa_paged_args *a, void *stream) {
  if (!a) return FA_ERR_BAD_ARG;
  if (a->partition_size <= 0) return FA_ERR_BAD_ARG;  // the one-pass mode needs no scratch at all
  fa_paged_args local = *a;
  local.part_out = nullptr, local.part_max = nullptr, local.part_sum = nullptr;
  int st = validate_paged(&local, false);
  if (st != FA_OK) return st;
  const int64_t need = fa_paged_workspace_bytes(&local);
  if (need > (int64_t)FA_PAGED_NOALLOC_SCRATCH_BYTES) return FA_ERR_TOO_LARGE;

  unsigned char *base = nullptr;
  st = paged_scratch_base(&base);
  if (st != FA_OK) return st;
  const int64_t P = (local.max_context_len + local.partition_size - 1) / local.partition_size;
  const int64_t rows = (int64_t)local.num_seqs * local.num_q_heads * P;
  // layout inside the array: partial outputs, then running maxima, then running sums.  Nothing
  // has to be zeroed: the decode kernel writes every (row, partition) slot the reducer later reads.
  local.part_out = reinterpret_cast<float *>(base);
  local.part_max = local.part_out + rows * local.head_size;
  local.part_sum = local.part_max + rows;
  st = fa_paged_decode(&local, stream);
  if (st != FA_OK) return st;
  return fa_paged_reduce(&local, stream);
}
