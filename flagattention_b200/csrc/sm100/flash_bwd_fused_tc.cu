// Launcher and C entry points of the one-pass tcgen05 flash_attention backward.
#include <cstdlib>
#include <utility>
#include <vector>

#include "flash_bwd_fused_tc.cuh"
#include "tma_host.cuh"
#include "../common.cuh"
#include "../dense_host.cuh"

namespace fa {
int *device_status_word();

namespace tc {

bool generic_forced();

static bool fused_covered(const fa_flash_shape *s) {
  return !generic_forced() && s->sm_scale > 0.f &&
         (s->D == 64 || s->D == 128) && s->dropout_p == 0.f;
}

// Workspace: fp32 dq accumulator (B, H, Mpad, D) | 16 bytes that hold the kernel's work-item
// counter.
static int64_t fused_dq_acc_bytes(const fa_flash_shape *s) {
  const int64_t mpad = ((int64_t)s->M + 127) / 128 * 128;
  return (int64_t)s->B * s->H * mpad * s->D * 4;
}
static int64_t fused_workspace_bytes(const fa_flash_shape *s, int accumulators = 1) {
  return accumulators * fused_dq_acc_bytes(s) + 16;
}

// one persistent CTA per SM
static int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
    return 0;
  return n;
}

// diff[i] holds +1 / -1 where coverage of unit i starts / ends; returns the maximal runs of
// uncovered units as row ranges (unit = `rows_per_unit` rows, clipped to `rows`).
static std::vector<std::pair<int, int>> zero_runs(const std::vector<int> &diff, int units,
                                                  int rows_per_unit, int rows) {
  std::vector<std::pair<int, int>> runs;
  int seen = 0, run_begin = -1;
  for (int u = 0; u <= units; ++u) {
    if (u < units) seen += diff[u];
    const bool uncovered = u < units && seen == 0;
    if (uncovered && run_begin < 0) run_begin = u;
    if (!uncovered && run_begin >= 0) {
      const int end = u * rows_per_unit < rows ? u * rows_per_unit : rows;
      runs.emplace_back(run_begin * rows_per_unit, end);
      run_begin = -1;
    }
  }
  return runs;
}

// Row ranges [begin, end) of dk / dv whose key block no query tile sees (keys past the causal
// triangle when N > M + ..., keys without a pair of the branch in a piecewise launch): the kernel
// skips those blocks.
static std::vector<std::pair<int, int>> unvisited_key_rows(const fa_flash_shape *s, int mode, int w) {
  const int BM = 128, BN = 128;
  const int p_seq = s->N - s->M, num_m_tiles = (s->M + BM - 1) / BM;
  const int num_blocks = (s->N + BN - 1) / BN;
  std::vector<int> diff(num_blocks + 1, 0);
  for (int nb = 0; nb < num_blocks; ++nb) {
    const int n0 = nb * BN;
    int lo = 0, hi = num_m_tiles;
    if (s->causal) lo = (n0 - p_seq > 0 ? n0 - p_seq : 0) / BM;
    if (mode == 1) {
      const int lim = w - p_seq + n0 + BN - 1;
      const int cap = lim <= 0 ? 0 : (lim + BM - 1) / BM;
      hi = cap < hi ? cap : hi;
    } else if (mode == 2) {
      const int lim = w - p_seq + n0 - (BM - 1);
      const int flo = lim <= 0 ? 0 : (lim + BM - 1) / BM;
      lo = flo > lo ? flo : lo;
    }
    if (lo < hi) ++diff[nb], --diff[nb + 1];
  }
  return zero_runs(diff, num_blocks, BN, s->N);
}

// Piecewise operands of the far branch; null for flash_attention.
struct FarBranch {
  const fa_tensor4 *q2, *k2, *dq2, *dk2;
  int w;
};

// flash_attention (far == nullptr) or piecewise_attention (both branches in ONE launch: every
// key block is walked twice by the same CTA, near pairs with (q, k) -> (dq, dk), far pairs with
// (q2, k2) -> (dq2, dk2); dV accumulates across the two walks and is rounded once).
// Workspace: dq accumulator [| dq2 accumulator] | 16 bytes of work-item counter.
template <typename T, int D>
static int launch_fused(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                        const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                        const float *delta, const fa_tensor4 *dq, const fa_tensor4 *dk,
                        const fa_tensor4 *dv, float *workspace, cudaStream_t stream,
                        const FarBranch *far = nullptr, int stages = 7) {
  using C = FusedBwdCfg<D>;
  const fa_tensor4 *q2 = far ? far->q2 : q, *k2 = far ? far->k2 : k, *dk2 = far ? far->dk2 : dk;
  CUtensorMap mq, mdo, mk, mv, mdk, mdv, mq2, mk2, mdk2;
  if (!make_map_bhld(&mq, q, s->dtype, s->B, s->H, s->M, D, C::BM) ||
      !make_map_bhld(&mdo, d_o, s->dtype, s->B, s->H, s->M, D, C::BM) ||
      !make_map_bhld(&mk, k, s->dtype, s->B, s->Hk, s->N, D, C::BN) ||
      !make_map_bhld(&mv, v, s->dtype, s->B, s->Hk, s->N, D, C::BN) ||
      !make_map_bhld(&mdk, dk, s->dtype, s->B, s->Hk, s->N, D, C::BN) ||
      !make_map_bhld(&mdv, dv, s->dtype, s->B, s->Hk, s->N, D, C::BN) ||
      !make_map_bhld(&mq2, q2, s->dtype, s->B, s->H, s->M, D, C::BM) ||
      !make_map_bhld(&mk2, k2, s->dtype, s->B, s->Hk, s->N, D, C::BN) ||
      !make_map_bhld(&mdk2, dk2, s->dtype, s->B, s->Hk, s->N, D, C::BN))
    return FA_ERR_UNSUPPORTED;
  auto kern = flash_bwd_fused_tc_kernel<T, D>;
  static unsigned long long done = 0;
  if (int st = ensure_dyn_smem(kern, C::kTotal, &done)) return st;
  FusedBwdParams fp{};
  BwdTcParams &p = fp.base;
  p.lse = lse, p.delta = delta;
  p.B = s->B, p.H = s->H, p.Hk = s->Hk, p.M = s->M, p.N = s->N;
  p.causal = s->causal, p.sm_scale = s->sm_scale;
  p.status = device_status_word();
  p.mode = far ? 3 : 0, p.w = far ? far->w : 0, p.dv_accumulate = 0;
  p.dk = dk->ptr, p.dv = dv->ptr, p.sdk = strides_of(dk), p.sdv = strides_of(dv);
  p.dq = dq->ptr, p.sdq = strides_of(dq);
  const int64_t acc_bytes = fused_dq_acc_bytes(s);
  const int n_acc = far ? 2 : 1;
  fp.dq_acc = workspace;
  fp.dq_acc2 = far ? reinterpret_cast<float *>(reinterpret_cast<char *>(workspace) + acc_bytes) : workspace;
  fp.dk2 = dk2->ptr;
  fp.Mpad = (s->M + 127) / 128 * 128;
  fp.sched = reinterpret_cast<unsigned *>(reinterpret_cast<char *>(workspace) + n_acc * acc_bytes);
  // stages: 1 = zero-fill of the workspace, 2 = the kernel, 4 = scale + convert the workspace to dq
  if ((stages & 1) &&
      cudaMemsetAsync(workspace, 0, (size_t)(n_acc * acc_bytes + 16), stream) != cudaSuccess)
    return FA_ERR_LAUNCH;
  if (stages & 2) {
    // the CTAs of a (batch, kv head) pair share its Q and dO tiles and its slice of the dq workspace
    p.num_blocks = (s->N + C::BN - 1) / C::BN;
    p.group_size = cta_group_size((int64_t)(s->H / s->Hk) * s->M * D * 8 * n_acc, s->B * s->Hk);
    const int64_t items = (int64_t)p.num_blocks * s->Hk * s->B;
    const int sms = sm_count();
    if (items > 0x3fffffff) return FA_ERR_TOO_LARGE;
    if (sms <= 0) return FA_ERR_LAUNCH;
    fp.num_items = (int)items;
    // dk / dv rows of key blocks that walk no query tile (which the kernel skips) get their zeros
    // here: dk of a branch where the block holds no pair of that branch, dv where it holds none at all
    auto zero_rows = [&](const fa_tensor4 *t, int mode) -> int {
      for (const auto &r : unvisited_key_rows(s, mode, p.w)) {
        if (r.first >= r.second) continue;
        dim3 zgrid((r.second - r.first + 15) / 16, s->Hk, s->B);
        zero_rows_kernel<T, D><<<zgrid, 256, 0, stream>>>(t->ptr, strides_of(t), r.first, r.second);
        FA_CHECK_LAUNCH();
      }
      return FA_OK;
    };
    if (int st = zero_rows(dv, 0)) return st;
    if (int st = zero_rows(dk, far ? 1 : 0)) return st;
    if (far)
      if (int st = zero_rows(dk2, 2)) return st;
    // persistent: a CTA takes key block `blockIdx.x`, then blocks handed out by the counter
    dim3 grid((unsigned)(items < sms ? items : sms), 1, 1);
    kern<<<grid, kFusedThreads, C::kTotal, stream>>>(mq, mdo, mk, mv, mdk, mdv, mq2, mk2, mdk2, fp);
    FA_CHECK_LAUNCH();
  }
  if (stages & 4) {
    dim3 cgrid((s->M + 31) / 32, s->H, s->B);
    dq_convert_kernel<T, D><<<cgrid, 256, 0, stream>>>(fp.dq_acc, dq->ptr, strides_of(dq), s->H,
                                                       s->M, fp.Mpad, s->sm_scale);
    FA_CHECK_LAUNCH();
    if (far) {
      dq_convert_kernel<T, D><<<cgrid, 256, 0, stream>>>(fp.dq_acc2, far->dq2->ptr, strides_of(far->dq2),
                                                         s->H, s->M, fp.Mpad, s->sm_scale);
      FA_CHECK_LAUNCH();
    }
  }
  return FA_OK;
}

template <typename T, int D>
static int launch_pw_fused(const fa_flash_shape *s, int w, const fa_tensor4 *q1, const fa_tensor4 *k1,
                           const fa_tensor4 *q2, const fa_tensor4 *k2, const fa_tensor4 *v,
                           const fa_tensor4 *d_o, const float *lse, const float *delta,
                           const fa_tensor4 *dq1, const fa_tensor4 *dq2, const fa_tensor4 *dk1,
                           const fa_tensor4 *dk2, const fa_tensor4 *dv, float *workspace,
                           cudaStream_t stream) {
  const FarBranch far{q2, k2, dq2, dk2, w};
  return launch_fused<T, D>(s, q1, k1, v, d_o, lse, delta, dq1, dk1, dv, workspace, stream, &far);
}

}  // namespace tc
}  // namespace fa

using namespace fa;

extern "C" int fa_piecewise_bwd_fused(const fa_flash_shape *s, int32_t dist_threshold,
                                      const fa_tensor4 *q1, const fa_tensor4 *k1,
                                      const fa_tensor4 *q2, const fa_tensor4 *k2,
                                      const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                                      const float *delta, const fa_tensor4 *dq1,
                                      const fa_tensor4 *dq2, const fa_tensor4 *dk1,
                                      const fa_tensor4 *dk2, const fa_tensor4 *dv, void *workspace,
                                      int64_t workspace_bytes, void *stream) {
  if (int st = validate_shape(s)) return st;
  if (s->H != s->Hk) return FA_ERR_BAD_ARG;
  if (int st = validate_tensors({q1, k1, q2, k2, v, d_o, dq1, dq2, dk1, dk2, dv})) return st;
  if (!lse || !delta) return FA_ERR_BAD_ARG;
  if (!tc::fused_covered(s) || dist_threshold > (1 << 29) || dist_threshold < -(1 << 29))
    return FA_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < tc::fused_workspace_bytes(s, 2) ||
      (reinterpret_cast<uintptr_t>(workspace) & 15))
    return FA_ERR_WORKSPACE;
  float *ws = static_cast<float *>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define FA_PWF_ARGS s, dist_threshold, q1, k1, q2, k2, v, d_o, lse, delta, dq1, dq2, dk1, dk2, dv, ws, st
  if (s->dtype == FA_F16)
    return s->D == 128 ? tc::launch_pw_fused<__half, 128>(FA_PWF_ARGS)
                       : tc::launch_pw_fused<__half, 64>(FA_PWF_ARGS);
  return s->D == 128 ? tc::launch_pw_fused<__nv_bfloat16, 128>(FA_PWF_ARGS)
                     : tc::launch_pw_fused<__nv_bfloat16, 64>(FA_PWF_ARGS);
#undef FA_PWF_ARGS
}

extern "C" int64_t fa_flash_bwd_fused_workspace_bytes(const fa_flash_shape *s) {
  if (!s || validate_shape(s) != FA_OK || !tc::fused_covered(s)) return 0;
  return tc::fused_workspace_bytes(s);
}

extern "C" int64_t fa_piecewise_bwd_fused_workspace_bytes(const fa_flash_shape *s) {
  if (!s || validate_shape(s) != FA_OK || !tc::fused_covered(s) || s->H != s->Hk) return 0;
  return tc::fused_workspace_bytes(s, 2);
}

extern "C" int fa_flash_bwd_fused_stages(const fa_flash_shape *s, const fa_tensor4 *q,
                                         const fa_tensor4 *k, const fa_tensor4 *v,
                                         const fa_tensor4 *d_o, const float *lse, const float *delta,
                                         const fa_tensor4 *dq, const fa_tensor4 *dk,
                                         const fa_tensor4 *dv, void *workspace,
                                         int64_t workspace_bytes, int32_t stages, void *stream);

extern "C" int fa_flash_bwd_fused(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                                  const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                                  const float *delta, const fa_tensor4 *dq, const fa_tensor4 *dk,
                                  const fa_tensor4 *dv, void *workspace, int64_t workspace_bytes,
                                  void *stream) {
  return fa_flash_bwd_fused_stages(s, q, k, v, d_o, lse, delta, dq, dk, dv, workspace,
                                   workspace_bytes, 7, stream);
}

extern "C" int fa_flash_bwd_fused_stages(const fa_flash_shape *s, const fa_tensor4 *q,
                                         const fa_tensor4 *k, const fa_tensor4 *v,
                                         const fa_tensor4 *d_o, const float *lse, const float *delta,
                                         const fa_tensor4 *dq, const fa_tensor4 *dk,
                                         const fa_tensor4 *dv, void *workspace,
                                         int64_t workspace_bytes, int32_t stages, void *stream) {
  if (stages < 1 || stages > 7) return FA_ERR_BAD_ARG;
  if (int st = validate_shape(s)) return st;
  if (int st = validate_tensors({q, k, v, d_o, dq, dk, dv})) return st;
  if (!lse || !delta) return FA_ERR_BAD_ARG;
  if (!tc::fused_covered(s)) return FA_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < tc::fused_workspace_bytes(s) ||
      (reinterpret_cast<uintptr_t>(workspace) & 15))
    return FA_ERR_WORKSPACE;
  float *ws = static_cast<float *>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define FA_FUSED_ARGS s, q, k, v, d_o, lse, delta, dq, dk, dv, ws, st, nullptr, stages
  if (s->dtype == FA_F16)
    return s->D == 128 ? tc::launch_fused<__half, 128>(FA_FUSED_ARGS)
                       : tc::launch_fused<__half, 64>(FA_FUSED_ARGS);
  return s->D == 128 ? tc::launch_fused<__nv_bfloat16, 128>(FA_FUSED_ARGS)
                     : tc::launch_fused<__nv_bfloat16, 64>(FA_FUSED_ARGS);
#undef FA_FUSED_ARGS
}
