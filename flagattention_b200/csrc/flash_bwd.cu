// C ABI entry points of the flash_attention backward (delta, dK/dV, dQ) and of
// the total-attention auxiliary output.
#include "dense_bwd.cuh"
#include "dense_host.cuh"

namespace fa {

struct DeltaLaunch {
  const fa_flash_shape *s;
  const fa_tensor4 *o, *d_o;
  float *delta;
  cudaStream_t stream;
  void *zero = nullptr;        // optional buffer to fill with zeros in the same launch
  int64_t zero_bytes = 0;
  template <typename T, int D>
  int operator()() const {
    const int threads = 256;
    const int rows_per_block = threads / (D / 8) * kDeltaRows;
    const int64_t blocks_per_pair = (s->M + rows_per_block - 1) / rows_per_block;
    const int64_t blocks = blocks_per_pair * s->B * s->H;
    if (blocks > 0x7fffffff) return FA_ERR_TOO_LARGE;
    if (blocks == 0)
      return (zero && cudaMemsetAsync(zero, 0, (size_t)zero_bytes, stream) != cudaSuccess) ? FA_ERR_LAUNCH : FA_OK;
    bwd_delta_kernel<T, D><<<(unsigned)blocks, threads, 0, stream>>>(
        o->ptr, strides_of(o), d_o->ptr, strides_of(d_o), delta, s->B, s->H, s->M,
        (int)blocks_per_pair, static_cast<uint4 *>(zero), (long long)(zero_bytes / 16));
    FA_CHECK_LAUNCH();
    return FA_OK;
  }
};

template <bool PW>
struct DkdvLaunch {
  BwdParams p;
  cudaStream_t stream;
  template <typename T, int D>
  int operator()() const {
    constexpr int BM = 64, BN = 128;
    using L = DkdvSmemLayout<D, BM, BN, PW>;
    static_assert(4 * BM >= BN, "store scratch must fit in the two stages");
    auto kern = dense_bwd_dkdv_kernel<T, D, BM, BN, PW>;
    static unsigned long long done = 0;
    if (int st = ensure_dyn_smem(kern, L::kTotal, &done)) return st;
    dim3 grid((p.N + BN - 1) / BN, p.Hk, p.B);
    kern<<<grid, BN / 16 * 32, L::kTotal, stream>>>(p);
    FA_CHECK_LAUNCH();
    return FA_OK;
  }
};

template <bool PW>
struct DqLaunch {
  BwdParams p;
  cudaStream_t stream;
  template <typename T, int D>
  int operator()() const {
    constexpr int BM = 128, BN = 64;
    using L = DqSmemLayout<D, BM, BN, PW>;
    static_assert(4 * BN >= BM, "store scratch must fit in the two stages");
    auto kern = dense_bwd_dq_kernel<T, D, BM, BN, PW>;
    static unsigned long long done = 0;
    if (int st = ensure_dyn_smem(kern, L::kTotal, &done)) return st;
    dim3 grid((p.M + BM - 1) / BM, p.B * p.H, 1);
    kern<<<grid, BM / 16 * 32, L::kTotal, stream>>>(p);
    FA_CHECK_LAUNCH();
    return FA_OK;
  }
};

struct TotalLaunch {
  const fa_flash_shape *s;
  const fa_tensor4 *q, *k;
  const float *lse;
  float *total;
  cudaStream_t stream;
  template <typename T, int D>
  int operator()() const {
    constexpr int BM = 64, BN = 128;
    using L = TotSmemLayout<D, BM, BN>;
    auto kern = total_attention_kernel<T, D, BM, BN>;
    static unsigned long long done = 0;
    if (int st = ensure_dyn_smem(kern, L::kTotal, &done)) return st;
    dim3 grid((s->N + BN - 1) / BN, s->B * s->H, 1);
    kern<<<grid, BN / 16 * 32, L::kTotal, stream>>>(q->ptr, strides_of(q), k->ptr, strides_of(k),
                                                    lse, total, s->B, s->H, s->Hk, s->M, s->N,
                                                    s->causal, s->sm_scale);
    FA_CHECK_LAUNCH();
    return FA_OK;
  }
};

namespace tc {
int total_attention_tc(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                       const float *lse, float *total, cudaStream_t stream);
int flash_bwd_dq_tc(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                    const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                    const float *delta, const fa_tensor4 *dq, cudaStream_t stream);
int flash_bwd_dkdv_tc(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                      const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                      const float *delta, const fa_tensor4 *dk, const fa_tensor4 *dv,
                      cudaStream_t stream);
int piecewise_bwd_dq_tc(const fa_flash_shape *s, int w, const fa_tensor4 *q1, const fa_tensor4 *k1,
                        const fa_tensor4 *q2, const fa_tensor4 *k2, const fa_tensor4 *v,
                        const fa_tensor4 *d_o, const float *lse, const float *delta,
                        const fa_tensor4 *dq1, const fa_tensor4 *dq2, cudaStream_t stream);
int piecewise_bwd_dkdv_tc(const fa_flash_shape *s, int w, const fa_tensor4 *q1,
                          const fa_tensor4 *k1, const fa_tensor4 *q2, const fa_tensor4 *k2,
                          const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                          const float *delta, const fa_tensor4 *dk1, const fa_tensor4 *dk2,
                          const fa_tensor4 *dv, cudaStream_t stream);
}  // namespace tc

}  // namespace fa

using namespace fa;

extern "C" int fa_flash_bwd_delta(const fa_flash_shape *s, const fa_tensor4 *o,
                                  const fa_tensor4 *d_o, float *delta, void *stream) {
  if (int st = validate_shape(s)) return st;
  if (int st = validate_tensors({o, d_o})) return st;
  if (!delta) return FA_ERR_BAD_ARG;
  return dispatch_dtype_d(s->dtype, s->D,
                          DeltaLaunch{s, o, d_o, delta, static_cast<cudaStream_t>(stream)});
}

extern "C" int fa_flash_bwd_delta_zero(const fa_flash_shape *s, const fa_tensor4 *o,
                                       const fa_tensor4 *d_o, float *delta, void *zero,
                                       int64_t zero_bytes, void *stream) {
  if (int st = validate_shape(s)) return st;
  if (int st = validate_tensors({o, d_o})) return st;
  if (!delta || !zero || zero_bytes <= 0 || zero_bytes % 16 || (reinterpret_cast<uintptr_t>(zero) & 15))
    return FA_ERR_BAD_ARG;
  DeltaLaunch l{s, o, d_o, delta, static_cast<cudaStream_t>(stream)};
  l.zero = zero, l.zero_bytes = zero_bytes;
  return dispatch_dtype_d(s->dtype, s->D, l);
}

static BwdParams make_bwd(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                          const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                          const float *delta) {
  BwdParams p{};
  p.q = q->ptr, p.k = k->ptr, p.v = v->ptr, p.d_o = d_o->ptr;
  p.sq = strides_of(q), p.sk = strides_of(k), p.sv = strides_of(v), p.sdo = strides_of(d_o);
  p.lse = lse, p.delta = delta;
  p.B = s->B, p.H = s->H, p.Hk = s->Hk, p.M = s->M, p.N = s->N;
  p.causal = s->causal, p.sm_scale = s->sm_scale;
  p.dropout_p = s->dropout_p, p.seed = s->philox_seed, p.offset = s->philox_offset;
  return p;
}

extern "C" int fa_flash_bwd_dkdv(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                                 const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                                 const float *delta, const fa_tensor4 *dk, const fa_tensor4 *dv,
                                 void *stream) {
  if (int st = validate_shape(s)) return st;
  if (int st = validate_tensors({q, k, v, d_o, dk, dv})) return st;
  if (!lse || !delta) return FA_ERR_BAD_ARG;
  // head_dim 64 / 128 run on tcgen05; everything else on the shape-generic kernel
  const int tc_status = tc::flash_bwd_dkdv_tc(s, q, k, v, d_o, lse, delta, dk, dv,
                                              static_cast<cudaStream_t>(stream));
  if (tc_status <= 0) return tc_status;
  BwdParams p = make_bwd(s, q, k, v, d_o, lse, delta);
  p.dk = dk->ptr, p.dv = dv->ptr, p.sdk = strides_of(dk), p.sdv = strides_of(dv);
  return dispatch_dtype_d(s->dtype, s->D, DkdvLaunch<false>{p, static_cast<cudaStream_t>(stream)});
}

extern "C" int fa_flash_bwd_dq(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                               const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                               const float *delta, const fa_tensor4 *dq, void *stream) {
  if (int st = validate_shape(s)) return st;
  if (int st = validate_tensors({q, k, v, d_o, dq})) return st;
  if (!lse || !delta) return FA_ERR_BAD_ARG;
  const int tc_status =
      tc::flash_bwd_dq_tc(s, q, k, v, d_o, lse, delta, dq, static_cast<cudaStream_t>(stream));
  if (tc_status <= 0) return tc_status;
  BwdParams p = make_bwd(s, q, k, v, d_o, lse, delta);
  p.dq = dq->ptr, p.sdq = strides_of(dq);
  return dispatch_dtype_d(s->dtype, s->D, DqLaunch<false>{p, static_cast<cudaStream_t>(stream)});
}

extern "C" int fa_total_attention(const fa_flash_shape *s, const fa_tensor4 *q,
                                  const fa_tensor4 *k, const float *lse, float *total,
                                  void *stream) {
  if (int st = validate_shape(s)) return st;
  if (int st = validate_tensors({q, k})) return st;
  if (!lse || !total) return FA_ERR_BAD_ARG;
  // head_dim 64 / 128 run on tcgen05; everything else on the shape-generic kernel
  const int tc_status = tc::total_attention_tc(s, q, k, lse, total, static_cast<cudaStream_t>(stream));
  if (tc_status <= 0) return tc_status;
  return dispatch_dtype_d(s->dtype, s->D,
                          TotalLaunch{s, q, k, lse, total, static_cast<cudaStream_t>(stream)});
}

// ---- piecewise backward ------------------------------------------------------

extern "C" int fa_piecewise_bwd_dkdv(const fa_flash_shape *s, int32_t dist_threshold,
                                     const fa_tensor4 *q1, const fa_tensor4 *k1,
                                     const fa_tensor4 *q2, const fa_tensor4 *k2,
                                     const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                                     const float *delta, const fa_tensor4 *dk1,
                                     const fa_tensor4 *dk2, const fa_tensor4 *dv, void *stream) {
  if (int st = validate_shape(s)) return st;
  if (s->H != s->Hk) return FA_ERR_BAD_ARG;
  if (int st = validate_tensors({q1, k1, q2, k2, v, d_o, dk1, dk2, dv})) return st;
  if (!lse || !delta) return FA_ERR_BAD_ARG;
  const int tc_status =
      tc::piecewise_bwd_dkdv_tc(s, dist_threshold, q1, k1, q2, k2, v, d_o, lse, delta, dk1, dk2, dv,
                                static_cast<cudaStream_t>(stream));
  if (tc_status <= 0) return tc_status;
  BwdParams p = make_bwd(s, q1, k1, v, d_o, lse, delta);
  p.q2 = q2->ptr, p.k2 = k2->ptr, p.sq2 = strides_of(q2), p.sk2 = strides_of(k2);
  p.w = dist_threshold;
  p.dk = dk1->ptr, p.dk2 = dk2->ptr, p.dv = dv->ptr;
  p.sdk = strides_of(dk1), p.sdk2 = strides_of(dk2), p.sdv = strides_of(dv);
  return dispatch_dtype_d(s->dtype, s->D, DkdvLaunch<true>{p, static_cast<cudaStream_t>(stream)});
}

extern "C" int fa_piecewise_bwd_dq(const fa_flash_shape *s, int32_t dist_threshold,
                                   const fa_tensor4 *q1, const fa_tensor4 *k1,
                                   const fa_tensor4 *q2, const fa_tensor4 *k2, const fa_tensor4 *v,
                                   const fa_tensor4 *d_o, const float *lse, const float *delta,
                                   const fa_tensor4 *dq1, const fa_tensor4 *dq2, void *stream) {
  if (int st = validate_shape(s)) return st;
  if (s->H != s->Hk) return FA_ERR_BAD_ARG;
  if (int st = validate_tensors({q1, k1, q2, k2, v, d_o, dq1, dq2})) return st;
  if (!lse || !delta) return FA_ERR_BAD_ARG;
  const int tc_status =
      tc::piecewise_bwd_dq_tc(s, dist_threshold, q1, k1, q2, k2, v, d_o, lse, delta, dq1, dq2,
                              static_cast<cudaStream_t>(stream));
  if (tc_status <= 0) return tc_status;
  BwdParams p = make_bwd(s, q1, k1, v, d_o, lse, delta);
  p.q2 = q2->ptr, p.k2 = k2->ptr, p.sq2 = strides_of(q2), p.sk2 = strides_of(k2);
  p.w = dist_threshold;
  p.dq = dq1->ptr, p.dq2 = dq2->ptr, p.sdq = strides_of(dq1), p.sdq2 = strides_of(dq2);
  return dispatch_dtype_d(s->dtype, s->D, DqLaunch<true>{p, static_cast<cudaStream_t>(stream)});
}
