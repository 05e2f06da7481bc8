// Launcher of the tcgen05 total_attention kernel.
#include "total_attn_tc.cuh"
#include "tma_host.cuh"
#include "../common.cuh"

namespace fa {
int *device_status_word();

namespace tc {

bool generic_forced();

template <typename T, int D>
static int launch_total_tc(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                           const float *lse, float *total, cudaStream_t stream) {
  using C = TotalTcCfg<D>;
  CUtensorMap mq, mk;
  if (!make_map_bhld(&mq, q, s->dtype, s->B, s->H, s->M, D, C::BM) ||
      !make_map_bhld(&mk, k, s->dtype, s->B, s->Hk, s->N, D, C::BN))
    return 1;   // layout not expressible as a tensor map: the caller uses the generic kernel
  auto kern = total_attention_tc_kernel<T, D>;
  static unsigned long long done = 0;
  if (int st = ensure_dyn_smem(kern, C::kTotal, &done)) return st;
  TotalTcParams p{};
  p.lse = lse, p.total = total;
  p.B = s->B, p.H = s->H, p.Hk = s->Hk, p.M = s->M, p.N = s->N;
  p.causal = s->causal, p.sm_scale = s->sm_scale;
  p.status = device_status_word();
  dim3 grid((s->N + C::BN - 1) / C::BN, s->B * s->H, 1);
  kern<<<grid, C::kThreads, C::kTotal, stream>>>(mq, mk, p);
  FA_CHECK_LAUNCH();
  return FA_OK;
}

// Returns FA_OK / a negative status, or 1 when this path does not cover the call.
int total_attention_tc(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                       const float *lse, float *total, cudaStream_t stream) {
  if (generic_forced() || !(s->sm_scale > 0.f) || (s->D != 64 && s->D != 128)) return 1;
  if (s->dtype == FA_F16)
    return s->D == 128 ? launch_total_tc<__half, 128>(s, q, k, lse, total, stream)
                       : launch_total_tc<__half, 64>(s, q, k, lse, total, stream);
  return s->D == 128 ? launch_total_tc<__nv_bfloat16, 128>(s, q, k, lse, total, stream)
                     : launch_total_tc<__nv_bfloat16, 64>(s, q, k, lse, total, stream);
}

}  // namespace tc
}  // namespace fa
