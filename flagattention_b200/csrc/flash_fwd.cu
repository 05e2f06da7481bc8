// C ABI entry points of the flash_attention forward: the one-pass kernel, the
// split-KV two-stage path for decode-shaped M, and the split-count heuristic.
#include <cmath>

#include "dense_fwd.cuh"
#include "dense_host.cuh"

namespace fa {

template <int D>
struct FwdTile {
  static constexpr int BM = 128;
  static constexpr int BN = 64;
};
struct SplitTile {
  static constexpr int BM = 64;
  static constexpr int BN = 64;
};

struct FwdLaunch {
  FwdParams p;
  cudaStream_t stream;
  template <typename T, int D>
  int operator()() const {
    constexpr int BM = FwdTile<D>::BM, BN = FwdTile<D>::BN;
    using L = FwdSmemLayout<D, BM, BN, false>;
    auto kern = dense_fwd_kernel<T, D, BM, BN, false, false>;
    static unsigned long long done = 0;
    if (int st = ensure_dyn_smem(kern, L::kTotal, &done)) return st;
    dim3 grid((p.M + BM - 1) / BM, p.B * p.H, 1);
    kern<<<grid, BM / 16 * 32, L::kTotal, stream>>>(p);
    FA_CHECK_LAUNCH();
    return FA_OK;
  }
};

struct SplitLaunch {
  FwdParams p;
  cudaStream_t stream;
  template <typename T, int D>
  int operator()() const {
    constexpr int BM = SplitTile::BM, BN = SplitTile::BN;
    using L = FwdSmemLayout<D, BM, BN, false>;
    auto kern = dense_fwd_kernel<T, D, BM, BN, false, true>;
    static unsigned long long done = 0;
    if (int st = ensure_dyn_smem(kern, L::kTotal, &done)) return st;
    dim3 grid((p.M + BM - 1) / BM, p.B * p.H, p.num_splits);
    kern<<<grid, BM / 16 * 32, L::kTotal, stream>>>(p);
    FA_CHECK_LAUNCH();
    return FA_OK;
  }
};

static FwdParams make_fwd_params(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                                 const fa_tensor4 *v) {
  FwdParams p{};
  p.q = q->ptr, p.k = k->ptr, p.v = v->ptr;
  p.sq = strides_of(q), p.sk = strides_of(k), p.sv = strides_of(v);
  p.B = s->B, p.H = s->H, p.Hk = s->Hk, p.M = s->M, p.N = s->N;
  p.causal = s->causal, p.sm_scale = s->sm_scale;
  p.dropout_p = s->dropout_p, p.seed = s->philox_seed, p.offset = s->philox_offset;
  p.num_splits = 1;
  return p;
}

namespace tc {
int flash_fwd_tc(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                 const fa_tensor4 *v, const fa_tensor4 *o, float *lse, cudaStream_t stream);
}

}  // namespace fa

using namespace fa;

extern "C" int fa_flash_fwd(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                            const fa_tensor4 *v, const fa_tensor4 *o, float *lse, void *stream) {
  if (int st = validate_shape(s)) return st;
  if (int st = validate_tensors({q, k, v, o})) return st;
  if (!lse) return FA_ERR_BAD_ARG;
  // head_dim 64 / 128 run on tcgen05; everything else on the shape-generic kernel
  const int tc_status = tc::flash_fwd_tc(s, q, k, v, o, lse, static_cast<cudaStream_t>(stream));
  if (tc_status <= 0) return tc_status;
  FwdParams p = make_fwd_params(s, q, k, v);
  p.o = o->ptr, p.so = strides_of(o), p.lse = lse;
  return dispatch_dtype_d(s->dtype, s->D, FwdLaunch{p, static_cast<cudaStream_t>(stream)});
}

extern "C" int fa_splitkv_fwd(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                              const fa_tensor4 *v, int32_t num_splits, int32_t n_split_size,
                              float *o_partial, float *lse_partial, void *stream) {
  if (int st = validate_shape(s)) return st;
  if (int st = validate_tensors({q, k, v})) return st;
  if (!o_partial || !lse_partial) return FA_ERR_WORKSPACE;
  if (s->dropout_p > 0.f) return FA_ERR_UNSUPPORTED;  // no dropout on the split-KV path
  if (num_splits < 1 || num_splits > 65535 || n_split_size <= 0 ||
      n_split_size % SplitTile::BN != 0)
    return FA_ERR_BAD_ARG;
  if ((int64_t)num_splits * n_split_size < s->N) return FA_ERR_BAD_ARG;
  FwdParams p = make_fwd_params(s, q, k, v);
  p.num_splits = num_splits, p.n_split_size = n_split_size;
  p.o_partial = o_partial, p.lse_partial = lse_partial;
  return dispatch_dtype_d(s->dtype, s->D, SplitLaunch{p, static_cast<cudaStream_t>(stream)});
}

extern "C" int fa_splitkv_combine(const fa_flash_shape *s, int32_t num_splits,
                                  const float *o_partial, const float *lse_partial,
                                  const fa_tensor4 *o, float *lse, void *stream) {
  if (int st = validate_shape(s)) return st;
  if (int st = validate_tensors({o})) return st;
  if (!o_partial || !lse_partial) return FA_ERR_WORKSPACE;
  if (!lse || num_splits < 1) return FA_ERR_BAD_ARG;
  const int64_t total = (int64_t)s->B * s->H * s->M * (s->D / 4);
  const int threads = 256;
  const int blocks = (int)std::min<int64_t>((total + threads - 1) / threads, 148 * 16);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (s->dtype == FA_F16)
    splitkv_combine_kernel<__half><<<blocks, threads, 0, st>>>(
        o_partial, lse_partial, o->ptr, strides_of(o), lse, s->B, s->H, s->M, s->D, num_splits);
  else
    splitkv_combine_kernel<__nv_bfloat16><<<blocks, threads, 0, st>>>(
        o_partial, lse_partial, o->ptr, strides_of(o), lse, s->B, s->H, s->M, s->D, num_splits);
  FA_CHECK_LAUNCH();
  return FA_OK;
}

extern "C" int64_t fa_splitkv_workspace_bytes(const fa_flash_shape *s, int32_t num_splits) {
  if (!s || num_splits < 1) return 0;
  const int64_t rows = (int64_t)s->B * s->H * num_splits * s->M;
  return rows * s->D * 4 + rows * 4;
}

// Restates src/flag_attn/split_kv.py:234-262: no split when the unsplit grid
// already fills 80% of the SMs; otherwise the smallest split count whose wave
// efficiency is within 85% of the best one, among counts that leave no split
// empty.
extern "C" int32_t fa_num_splits_heuristic(int32_t B, int32_t H, int32_t M, int32_t N,
                                           int32_t block_m, int32_t block_n, int32_t num_sms,
                                           int32_t max_splits) {
  const int64_t blocks = (int64_t)B * H * ((M + block_m - 1) / block_m);
  if ((double)blocks >= 0.8 * num_sms) return 1;
  const int n_blocks = (N + block_n - 1) / block_n;
  max_splits = std::min(std::min(num_sms, n_blocks), max_splits);
  auto available = [&](int sp) {
    const int per = (n_blocks + sp - 1) / sp;
    return sp == 1 || (per * sp - n_blocks < per);
  };
  auto efficiency = [&](int sp) {
    const double waves = (double)(blocks * sp) / num_sms;
    return waves / std::ceil(waves);
  };
  double best = 0.0;
  for (int sp = 1; sp <= max_splits; ++sp)
    if (available(sp)) best = std::max(best, efficiency(sp));
  for (int sp = 1; sp <= max_splits; ++sp)
    if (available(sp) && efficiency(sp) >= 0.85 * best) return sp;
  return 1;
}
