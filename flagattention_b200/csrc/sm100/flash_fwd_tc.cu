// Launcher of the tcgen05 flash_attention forward.
#include <atomic>
#include <cstdlib>

#include "flash_fwd_tc.cuh"
#include "tma_host.cuh"
#include "../common.cuh"

namespace fa {
int *device_status_word();

namespace tc {

// Kernel family switch (fa_set_kernel_family): 0 = tcgen05 kernels wherever they cover the call,
// 1 = shape-generic kernels only.  The environment variable FLAGATTN_B200_GENERIC=1 only sets the
// value the process starts with.
static std::atomic<int> g_kernel_family{[] {
  const char *e = std::getenv("FLAGATTN_B200_GENERIC");
  return (e && e[0] == '1') ? 1 : 0;
}()};
bool generic_forced() { return g_kernel_family.load(std::memory_order_relaxed) == 1; }
int set_kernel_family(int family) { return g_kernel_family.exchange(family == 1 ? 1 : 0); }

template <typename T, int D, bool PW>
static int launch_fwd_tc(const fa_flash_shape *s, int w, const fa_tensor4 *q, const fa_tensor4 *k,
                         const fa_tensor4 *q2, const fa_tensor4 *k2, const fa_tensor4 *v,
                         const fa_tensor4 *o, float *lse, cudaStream_t stream) {
  using C = FwdTcCfg<D>;
  CUtensorMap mq, mk, mv, mq2, mk2;
  if (!make_map_bhld(&mq, q, s->dtype, s->B, s->H, s->M, D, C::BM) ||
      !make_map_bhld(&mk, k, s->dtype, s->B, s->Hk, s->N, D, C::BN) ||
      !make_map_bhld(&mv, v, s->dtype, s->B, s->Hk, s->N, D, C::BN) ||
      !make_map_bhld(&mq2, q2, s->dtype, s->B, s->H, s->M, D, C::BM) ||
      !make_map_bhld(&mk2, k2, s->dtype, s->B, s->Hk, s->N, D, C::BN))
    return 1;  // layout not expressible as a tensor map: caller falls back to the generic kernel
  auto kern = flash_fwd_tc_kernel<T, D, PW>;
  static unsigned long long done = 0;
  if (int st = ensure_dyn_smem(kern, C::kTotal, &done)) return st;
  FwdTcParams p{};
  p.o = o->ptr, p.lse = lse, p.so = strides_of(o);
  p.B = s->B, p.H = s->H, p.Hk = s->Hk, p.M = s->M, p.N = s->N;
  p.causal = s->causal, p.sm_scale = s->sm_scale, p.w = w;
  p.status = device_status_word();
  // the CTAs of a (batch, head) pair share its K and V (and K2 under piecewise)
  p.num_m_blocks = (s->M + C::BM - 1) / C::BM;
  p.group_size = cta_group_size((int64_t)s->N * D * 2 * (PW ? 3 : 2), s->B * s->H);
  dim3 grid((unsigned)((int64_t)p.num_m_blocks * s->B * s->H), 1, 1);
  kern<<<grid, C::kThreads, C::kTotal, stream>>>(mq, mk, mv, mq2, mk2, p);
  FA_CHECK_LAUNCH();
  return FA_OK;
}

static bool covered(const fa_flash_shape *s) {
  return !generic_forced() && s->sm_scale > 0.f && (s->D == 64 || s->D == 128) &&
         s->dropout_p == 0.f;  // dropout runs on the shape-generic kernels
}

// Return FA_OK / a negative status, or 1 when this path does not cover the call.
int flash_fwd_tc(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                 const fa_tensor4 *v, const fa_tensor4 *o, float *lse, cudaStream_t stream) {
  if (!covered(s)) return 1;
  if (s->dtype == FA_F16)
    return s->D == 128 ? launch_fwd_tc<__half, 128, false>(s, 0, q, k, q, k, v, o, lse, stream)
                       : launch_fwd_tc<__half, 64, false>(s, 0, q, k, q, k, v, o, lse, stream);
  return s->D == 128 ? launch_fwd_tc<__nv_bfloat16, 128, false>(s, 0, q, k, q, k, v, o, lse, stream)
                     : launch_fwd_tc<__nv_bfloat16, 64, false>(s, 0, q, k, q, k, v, o, lse, stream);
}

int piecewise_fwd_tc(const fa_flash_shape *s, int w, const fa_tensor4 *q1, const fa_tensor4 *k1,
                     const fa_tensor4 *q2, const fa_tensor4 *k2, const fa_tensor4 *v,
                     const fa_tensor4 *o, float *lse, cudaStream_t stream) {
  if (!covered(s) || w > (1 << 29) || w < -(1 << 29)) return 1;
  if (s->dtype == FA_F16)
    return s->D == 128 ? launch_fwd_tc<__half, 128, true>(s, w, q1, k1, q2, k2, v, o, lse, stream)
                       : launch_fwd_tc<__half, 64, true>(s, w, q1, k1, q2, k2, v, o, lse, stream);
  return s->D == 128
             ? launch_fwd_tc<__nv_bfloat16, 128, true>(s, w, q1, k1, q2, k2, v, o, lse, stream)
             : launch_fwd_tc<__nv_bfloat16, 64, true>(s, w, q1, k1, q2, k2, v, o, lse, stream);
}

}  // namespace tc
}  // namespace fa

extern "C" int32_t fa_set_kernel_family(int32_t family) { return fa::tc::set_kernel_family(family); }
