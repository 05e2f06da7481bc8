// Host-side glue for the dense kernels: argument validation and dispatch over
// (dtype, head_dim).
#pragma once

#include "attn_params.cuh"

namespace fa {

inline int validate_shape(const fa_flash_shape *s) {
  if (!s) return FA_ERR_BAD_ARG;
  if (s->dtype != FA_F16 && s->dtype != FA_BF16) return FA_ERR_BAD_ARG;
  if (s->B <= 0 || s->H <= 0 || s->Hk <= 0 || s->M <= 0 || s->N <= 0) return FA_ERR_BAD_ARG;
  if (s->H % s->Hk != 0) return FA_ERR_BAD_ARG;
  if (!(s->D == 16 || s->D == 32 || s->D == 64 || s->D == 128)) return FA_ERR_UNSUPPORTED;
  if ((int64_t)s->B * s->H > 65535) return FA_ERR_TOO_LARGE;  // grid.y / grid.z limit
  if (!(s->dropout_p >= 0.f && s->dropout_p < 1.f)) return FA_ERR_BAD_ARG;
  return FA_OK;
}

inline int validate_tensors(std::initializer_list<const fa_tensor4 *> ts) {
  for (const fa_tensor4 *t : ts)
    if (!tensor_ok(t)) return FA_ERR_BAD_ARG;
  for (const fa_tensor4 *t : ts)
    if (!tensor_aligned(t)) return FA_ERR_ALIGNMENT;
  return FA_OK;
}

// Calls f.template operator()<T, D>() for the runtime (dtype, D).
template <typename F>
inline int dispatch_dtype_d(int dtype, int D, F &&f) {
#define FA_CASE_D(TT)                                    \
  switch (D) {                                           \
    case 16: return f.template operator()<TT, 16>();     \
    case 32: return f.template operator()<TT, 32>();     \
    case 64: return f.template operator()<TT, 64>();     \
    case 128: return f.template operator()<TT, 128>();   \
    default: return FA_ERR_UNSUPPORTED;                  \
  }
  if (dtype == FA_F16) {
    FA_CASE_D(__half)
  } else {
    FA_CASE_D(__nv_bfloat16)
  }
#undef FA_CASE_D
}

}  // namespace fa
