// Launcher of the tcgen05 flash_attention forward.
#include <atomic>
#include <cstdlib>

#include "flash_fwd_tc.cuh"
#include "flash_fwd_persist_tc.cuh"
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
// family 2 (test suites, A/B timing): tcgen05 kernels, but the forward with one CTA per query tile
static bool one_cta_per_tile_forced() { return g_kernel_family.load(std::memory_order_relaxed) == 2; }
int set_kernel_family(int family) {
  return g_kernel_family.exchange(family == 1 ? 1 : (family == 2 ? 2 : 0));
}

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

// Work-item counters of the persistent forward.  The forward entry points take no workspace, so
// the counters live in the library: a table of 64 words per device, one word per launch, taken
// round-robin, zeroed by a four-byte stream-ordered memset in front of the launch (a launch also
// puts its word back to zero with its last fetch, but relying on that alone let one cut-short
// launch spoil a later one: seen in the test suite).  A word is only touched while its kernel
// runs, so two launches collide only if 64 later launches start while the first still runs.
static __device__ unsigned g_fwd_sched[64];
static unsigned *fwd_sched_table() {
  static std::atomic<unsigned *> base[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  unsigned *b = base[dev].load(std::memory_order_acquire);
  if (!b) {
    void *ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_fwd_sched) != cudaSuccess) return nullptr;
    b = static_cast<unsigned *>(ptr);
    base[dev].store(b, std::memory_order_release);
  }
  return b;
}
static unsigned *fwd_sched_slot() {
  static std::atomic<unsigned> next{0};
  unsigned *b = fwd_sched_table();
  return b ? b + (next.fetch_add(1u, std::memory_order_relaxed) & 63u) : nullptr;
}
int reset_fwd_sched() {
  unsigned *b = fwd_sched_table();
  if (!b) return FA_ERR_LAUNCH;
  return cudaMemset(b, 0, 64 * sizeof(unsigned)) == cudaSuccess ? FA_OK : FA_ERR_LAUNCH;
}

static int sm_count_fwd() {
  static std::atomic<int> n[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  int v = n[dev].load(std::memory_order_relaxed);
  if (!v) {
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    n[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}

// The persistent form (flash_fwd_persist_tc.cuh): two CTAs per SM that work through the query tiles.
template <typename T, int D>
static int launch_fwd_persist(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                              const fa_tensor4 *v, const fa_tensor4 *o, float *lse, cudaStream_t stream) {
  using C = FwdPersistCfg<D>;
  CUtensorMap mq, mk, mv;
  if (!make_map_bhld(&mq, q, s->dtype, s->B, s->H, s->M, D, C::BM) ||
      !make_map_bhld(&mk, k, s->dtype, s->B, s->Hk, s->N, D, C::BN) ||
      !make_map_bhld(&mv, v, s->dtype, s->B, s->Hk, s->N, D, C::BN))
    return 1;
  auto kern = flash_fwd_persist_tc_kernel<T, D>;
  static unsigned long long done = 0;
  if (int st = ensure_dyn_smem(kern, C::kTotal, &done)) return st;
  FwdPersistParams fp{};
  FwdTcParams &p = fp.base;
  p.o = o->ptr, p.lse = lse, p.so = strides_of(o);
  p.B = s->B, p.H = s->H, p.Hk = s->Hk, p.M = s->M, p.N = s->N;
  p.causal = s->causal, p.sm_scale = s->sm_scale, p.w = 0;
  p.status = device_status_word();
  p.num_m_blocks = (s->M + C::BM - 1) / C::BM;
  p.group_size = cta_group_size((int64_t)s->N * D * 2 * 2, s->B * s->H);
  const int64_t items = (int64_t)p.num_m_blocks * s->B * s->H;
  const int sms = sm_count_fwd();
  fp.sched = fwd_sched_slot();
  if (items <= 0 || items > (1ll << 30) || sms <= 0 || !fp.sched) return 1;
  fp.num_items = (int)items;
  dim3 grid((unsigned)(items < 2 * sms ? items : 2 * sms), 1, 1);
  if (cudaMemsetAsync(fp.sched, 0, sizeof(unsigned), stream) != cudaSuccess) return FA_ERR_LAUNCH;
  kern<<<grid, C::kThreads, C::kTotal, stream>>>(mq, mk, mv, fp);
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
  // More query tiles than CTA slots and short walks (or head_dim 64): the persistent kernel.  It
  // measured +3..5 % at N <= 1024 and at head_dim 64, but -10 % at head_dim 128 and N = 4096, -17 %
  // at 16384: its steady tile period is 1750-1840 clocks against 1534 of the one-CTA-per-tile
  // kernel (why is not known: starting the second CTA of every SM a fraction of a tile period late,
  // in case the two walked in step, changed nothing).
  const bool short_walks = s->D == 64 || s->N <= 1536;
  if (!one_cta_per_tile_forced() && short_walks &&
      (int64_t)((s->M + 127) / 128) * s->B * s->H > 2 * (int64_t)sm_count_fwd()) {
    int st;
    if (s->dtype == FA_F16)
      st = s->D == 128 ? launch_fwd_persist<__half, 128>(s, q, k, v, o, lse, stream)
                       : launch_fwd_persist<__half, 64>(s, q, k, v, o, lse, stream);
    else
      st = s->D == 128 ? launch_fwd_persist<__nv_bfloat16, 128>(s, q, k, v, o, lse, stream)
                       : launch_fwd_persist<__nv_bfloat16, 64>(s, q, k, v, o, lse, stream);
    if (st != 1) return st;
  }
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
