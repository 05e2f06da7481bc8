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

static BwdTcParams make_params(const fa_flash_shape *s, const float *lse, const float *delta,
                               int mode, int w) {
  BwdTcParams p{};
  p.lse = lse, p.delta = delta;
  p.B = s->B, p.H = s->H, p.Hk = s->Hk, p.M = s->M, p.N = s->N;
  p.causal = s->causal, p.sm_scale = s->sm_scale;
  p.mode = mode, p.w = w;
  p.status = device_status_word();
  return p;
}

template <typename T, int D>
static int launch_dq(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                     const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                     const float *delta, const fa_tensor4 *dq, cudaStream_t stream, int mode = 0,
                     int w = 0) {
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
  BwdTcParams p = make_params(s, lse, delta, mode, w);
  p.dq = dq->ptr, p.sdq = strides_of(dq);
  // the CTAs of a (batch, head) pair share its K and V
  p.num_blocks = (s->M + C::BM - 1) / C::BM;
  p.group_size = cta_group_size((int64_t)s->N * D * 4, s->B * s->H);
  dim3 grid((unsigned)((int64_t)p.num_blocks * s->B * s->H), 1, 1);
  kern<<<grid, kBwdThreads, C::kTotal, stream>>>(m.q, m.d_o, m.k, m.v, p);
  FA_CHECK_LAUNCH();
  return FA_OK;
}

template <typename T, int D>
static int launch_dkdv(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                       const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                       const float *delta, const fa_tensor4 *dk, const fa_tensor4 *dv,
                       cudaStream_t stream, int mode = 0, int w = 0, int dv_accumulate = 0) {
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
  BwdTcParams p = make_params(s, lse, delta, mode, w);
  p.dv_accumulate = dv_accumulate;
  p.dk = dk->ptr, p.dv = dv->ptr, p.sdk = strides_of(dk), p.sdv = strides_of(dv);
  // the CTAs of a (batch, kv head) pair share its Q and dO
  p.num_blocks = (s->N + C::BN - 1) / C::BN;
  p.group_size = cta_group_size((int64_t)(s->H / s->Hk) * s->M * D * 4, s->B * s->Hk);
  dim3 grid((unsigned)((int64_t)p.num_blocks * s->Hk * s->B), 1, 1);
  kern<<<grid, kDkdvThreads, C::kTotal, stream>>>(m.q, m.d_o, m.k, m.v, p);
  FA_CHECK_LAUNCH();
  return FA_OK;
}

static bool covered(const fa_flash_shape *s) {
  return !generic_forced() && s->sm_scale > 0.f && (s->D == 64 || s->D == 128) &&
         s->dropout_p == 0.f;  // dropout runs on the shape-generic kernels
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

// piecewise_attention backward: each kernel runs once per branch.  The near launch scores with
// (q1, k1) and visits the tiles that hold a near pair, the far launch with (q2, k2); dV is written
// by the near launch and added to by the far one.
template <typename T, int D>
static int launch_pw_dq(const fa_flash_shape *s, int w, const fa_tensor4 *q1, const fa_tensor4 *k1,
                        const fa_tensor4 *q2, const fa_tensor4 *k2, const fa_tensor4 *v,
                        const fa_tensor4 *d_o, const float *lse, const float *delta,
                        const fa_tensor4 *dq1, const fa_tensor4 *dq2, cudaStream_t stream) {
  int st = launch_dq<T, D>(s, q1, k1, v, d_o, lse, delta, dq1, stream, 1, w);
  if (st != FA_OK) return st;
  return launch_dq<T, D>(s, q2, k2, v, d_o, lse, delta, dq2, stream, 2, w);
}

template <typename T, int D>
static int launch_pw_dkdv(const fa_flash_shape *s, int w, const fa_tensor4 *q1,
                          const fa_tensor4 *k1, const fa_tensor4 *q2, const fa_tensor4 *k2,
                          const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                          const float *delta, const fa_tensor4 *dk1, const fa_tensor4 *dk2,
                          const fa_tensor4 *dv, cudaStream_t stream) {
  int st = launch_dkdv<T, D>(s, q1, k1, v, d_o, lse, delta, dk1, dv, stream, 1, w, 0);
  if (st != FA_OK) return st;
  return launch_dkdv<T, D>(s, q2, k2, v, d_o, lse, delta, dk2, dv, stream, 2, w, 1);
}

static bool pw_covered(const fa_flash_shape *s, int w) {
  return covered(s) && w <= (1 << 29) && w >= -(1 << 29);
}

int piecewise_bwd_dq_tc(const fa_flash_shape *s, int w, const fa_tensor4 *q1, const fa_tensor4 *k1,
                        const fa_tensor4 *q2, const fa_tensor4 *k2, const fa_tensor4 *v,
                        const fa_tensor4 *d_o, const float *lse, const float *delta,
                        const fa_tensor4 *dq1, const fa_tensor4 *dq2, cudaStream_t stream) {
  if (!pw_covered(s, w)) return 1;
#define FA_PW_ARGS s, w, q1, k1, q2, k2, v, d_o, lse, delta, dq1, dq2, stream
  if (s->dtype == FA_F16)
    return s->D == 128 ? launch_pw_dq<__half, 128>(FA_PW_ARGS) : launch_pw_dq<__half, 64>(FA_PW_ARGS);
  return s->D == 128 ? launch_pw_dq<__nv_bfloat16, 128>(FA_PW_ARGS)
                     : launch_pw_dq<__nv_bfloat16, 64>(FA_PW_ARGS);
#undef FA_PW_ARGS
}

int piecewise_bwd_dkdv_tc(const fa_flash_shape *s, int w, const fa_tensor4 *q1,
                          const fa_tensor4 *k1, const fa_tensor4 *q2, const fa_tensor4 *k2,
                          const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                          const float *delta, const fa_tensor4 *dk1, const fa_tensor4 *dk2,
                          const fa_tensor4 *dv, cudaStream_t stream) {
  if (!pw_covered(s, w)) return 1;
#define FA_PW_ARGS s, w, q1, k1, q2, k2, v, d_o, lse, delta, dk1, dk2, dv, stream
  if (s->dtype == FA_F16)
    return s->D == 128 ? launch_pw_dkdv<__half, 128>(FA_PW_ARGS)
                       : launch_pw_dkdv<__half, 64>(FA_PW_ARGS);
  return s->D == 128 ? launch_pw_dkdv<__nv_bfloat16, 128>(FA_PW_ARGS)
                     : launch_pw_dkdv<__nv_bfloat16, 64>(FA_PW_ARGS);
#undef FA_PW_ARGS
}

}  // namespace tc
}  // namespace fa
