// Launchers of the tcgen05 flash_attention backward kernels.
#include "flash_bwd_tc.cuh"
#include "tma_host.cuh"
#include "../common.cuh"

namespace fa {
int *device_status_word();

namespace tc {

bool generic_forced();

struct BwdMaps {
  CUtensorMap q, d_o, k, v;
};

static BwdTcParams make_params(const fa_flash_shape *s, const float *lse, const float *delta) {
  BwdTcParams p{};
  p.lse = lse, p.delta = delta;
  p.B = s->B, p.H = s->H, p.Hk = s->Hk, p.M = s->M, p.N = s->N;
  p.causal = s->causal, p.sm_scale = s->sm_scale;
  p.status = device_status_word();
  return p;
}

template <typename T, int D>
static int launch_dq(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                     const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                     const float *delta, const fa_tensor4 *dq, cudaStream_t stream) {
  using C = DqTcCfg<D>;
  BwdMaps m;
  if (!make_map_bhld(&m.q, q, s->dtype, s->B, s->H, s->M, D, C::BM) ||
      !make_map_bhld(&m.d_o, d_o, s->dtype, s->B, s->H, s->M, D, C::BM) ||
      !make_map_bhld(&m.k, k, s->dtype, s->B, s->Hk, s->N, D, C::BN) ||
      !make_map_bhld(&m.v, v, s->dtype, s->B, s->Hk, s->N, D, C::BN))
    return 1;
  auto kern = flash_bwd_dq_tc_kernel<T, D>;
  static unsigned long long done = 0;
  if (int st = ensure_dyn_smem(kern, C::kTotal, &done)) return st;
  BwdTcParams p = make_params(s, lse, delta);
  p.dq = dq->ptr, p.sdq = strides_of(dq);
  dim3 grid((s->M + C::BM - 1) / C::BM, s->B * s->H, 1);
  kern<<<grid, kBwdThreads, C::kTotal, stream>>>(m.q, m.d_o, m.k, m.v, p);
  FA_CHECK_LAUNCH();
  return FA_OK;
}

template <typename T, int D>
static int launch_dkdv(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                       const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                       const float *delta, const fa_tensor4 *dk, const fa_tensor4 *dv,
                       cudaStream_t stream) {
  using C = DkdvTcCfg<D>;
  BwdMaps m;
  if (!make_map_bhld(&m.q, q, s->dtype, s->B, s->H, s->M, D, C::BM) ||
      !make_map_bhld(&m.d_o, d_o, s->dtype, s->B, s->H, s->M, D, C::BM) ||
      !make_map_bhld(&m.k, k, s->dtype, s->B, s->Hk, s->N, D, C::BN) ||
      !make_map_bhld(&m.v, v, s->dtype, s->B, s->Hk, s->N, D, C::BN))
    return 1;
  auto kern = flash_bwd_dkdv_tc_kernel<T, D>;
  static unsigned long long done = 0;
  if (int st = ensure_dyn_smem(kern, C::kTotal, &done)) return st;
  BwdTcParams p = make_params(s, lse, delta);
  p.dk = dk->ptr, p.dv = dv->ptr, p.sdk = strides_of(dk), p.sdv = strides_of(dv);
  dim3 grid((s->N + C::BN - 1) / C::BN, s->Hk, s->B);
  kern<<<grid, kBwdThreads, C::kTotal, stream>>>(m.q, m.d_o, m.k, m.v, p);
  FA_CHECK_LAUNCH();
  return FA_OK;
}

static bool covered(const fa_flash_shape *s) {
  return !generic_forced() && s->sm_scale > 0.f && (s->D == 64 || s->D == 128);
}

// Return FA_OK / a negative status, or 1 when the tensor-core path does not cover the call.
int flash_bwd_dq_tc(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                    const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                    const float *delta, const fa_tensor4 *dq, cudaStream_t stream) {
  if (!covered(s)) return 1;
  if (s->dtype == FA_F16)
    return s->D == 128 ? launch_dq<__half, 128>(s, q, k, v, d_o, lse, delta, dq, stream)
                       : launch_dq<__half, 64>(s, q, k, v, d_o, lse, delta, dq, stream);
  return s->D == 128 ? launch_dq<__nv_bfloat16, 128>(s, q, k, v, d_o, lse, delta, dq, stream)
                     : launch_dq<__nv_bfloat16, 64>(s, q, k, v, d_o, lse, delta, dq, stream);
}

int flash_bwd_dkdv_tc(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                      const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                      const float *delta, const fa_tensor4 *dk, const fa_tensor4 *dv,
                      cudaStream_t stream) {
  if (!covered(s)) return 1;
  if (s->dtype == FA_F16)
    return s->D == 128 ? launch_dkdv<__half, 128>(s, q, k, v, d_o, lse, delta, dk, dv, stream)
                       : launch_dkdv<__half, 64>(s, q, k, v, d_o, lse, delta, dk, dv, stream);
  return s->D == 128
             ? launch_dkdv<__nv_bfloat16, 128>(s, q, k, v, d_o, lse, delta, dk, dv, stream)
             : launch_dkdv<__nv_bfloat16, 64>(s, q, k, v, d_o, lse, delta, dk, dv, stream);
}

}  // namespace tc
}  // namespace fa
