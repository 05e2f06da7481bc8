// C ABI entry point of the piecewise_attention forward.
#include "dense_fwd.cuh"
#include "dense_host.cuh"

namespace fa {

struct PwFwdLaunch {
  FwdParams p;
  cudaStream_t stream;
  template <typename T, int D>
  int operator()() const {
    constexpr int BM = 128, BN = 64;
    using L = FwdSmemLayout<D, BM, BN, true>;
    auto kern = dense_fwd_kernel<T, D, BM, BN, true, false>;
    static unsigned long long done = 0;
    if (int st = ensure_dyn_smem(kern, L::kTotal, &done)) return st;
    dim3 grid((p.M + BM - 1) / BM, p.B * p.H, 1);
    kern<<<grid, BM / 16 * 32, L::kTotal, stream>>>(p);
    FA_CHECK_LAUNCH();
    return FA_OK;
  }
};

namespace tc {
int piecewise_fwd_tc(const fa_flash_shape *s, int w, const fa_tensor4 *q1, const fa_tensor4 *k1,
                     const fa_tensor4 *q2, const fa_tensor4 *k2, const fa_tensor4 *v,
                     const fa_tensor4 *o, float *lse, cudaStream_t stream);
}

}  // namespace fa

using namespace fa;

extern "C" int fa_piecewise_fwd(const fa_flash_shape *s, int32_t dist_threshold,
                                const fa_tensor4 *q1, const fa_tensor4 *k1, const fa_tensor4 *q2,
                                const fa_tensor4 *k2, const fa_tensor4 *v, const fa_tensor4 *o,
                                float *lse, void *stream) {
  if (int st = validate_shape(s)) return st;
  if (s->H != s->Hk) return FA_ERR_BAD_ARG;
  if (int st = validate_tensors({q1, k1, q2, k2, v, o})) return st;
  if (!lse) return FA_ERR_BAD_ARG;
  // head_dim 64 / 128 run on tcgen05; everything else on the shape-generic kernel
  const int tc_status = tc::piecewise_fwd_tc(s, dist_threshold, q1, k1, q2, k2, v, o, lse,
                                             static_cast<cudaStream_t>(stream));
  if (tc_status <= 0) return tc_status;
  FwdParams p{};
  p.q = q1->ptr, p.k = k1->ptr, p.q2 = q2->ptr, p.k2 = k2->ptr, p.v = v->ptr;
  p.sq = strides_of(q1), p.sk = strides_of(k1), p.sq2 = strides_of(q2), p.sk2 = strides_of(k2);
  p.sv = strides_of(v);
  p.o = o->ptr, p.so = strides_of(o), p.lse = lse;
  p.B = s->B, p.H = s->H, p.Hk = s->Hk, p.M = s->M, p.N = s->N;
  p.causal = s->causal, p.sm_scale = s->sm_scale, p.w = dist_threshold;
  p.num_splits = 1;
  return dispatch_dtype_d(s->dtype, s->D, PwFwdLaunch{p, static_cast<cudaStream_t>(stream)});
}
