// Kernel parameter blocks shared by the dense (flash / piecewise) kernels and
// the host-side glue that fills them from the C ABI structs.
#pragma once

#include "common.cuh"

namespace fa {

struct Strides {
  int64_t b, h, l;
};

__host__ __device__ inline Strides strides_of(const fa_tensor4 *t) {
  return Strides{t->stride_b, t->stride_h, t->stride_l};
}

// Forward (flash, piecewise and split-KV stage 1).
struct FwdParams {
  const void *q, *k, *v, *q2, *k2;
  void *o;
  float *lse;
  Strides sq, sk, sv, sq2, sk2, so;
  int B, H, Hk, M, N;
  int causal;
  int w;  // piecewise distance threshold
  float sm_scale;
  // split-KV
  int num_splits, n_split_size;
  float *o_partial;    // (B,H,S,M,D)
  float *lse_partial;  // (B,H,S,M)
};

// Backward (flash and piecewise).  In the flash kernels q2/k2/dq2/dk2 are unused.
struct BwdParams {
  const void *q, *k, *v, *q2, *k2, *d_o;
  const float *lse, *delta;
  void *dq, *dq2, *dk, *dk2, *dv;
  Strides sq, sk, sv, sq2, sk2, sdo, sdq, sdq2, sdk, sdk2, sdv;
  int B, H, Hk, M, N;
  int causal;
  int w;
  float sm_scale;
};

template <typename T>
__device__ __forceinline__ const T *row_ptr(const void *base, const Strides &s, int b, int h,
                                            int l) {
  return reinterpret_cast<const T *>(base) + (int64_t)b * s.b + (int64_t)h * s.h +
         (int64_t)l * s.l;
}
template <typename T>
__device__ __forceinline__ T *row_ptr_mut(void *base, const Strides &s, int b, int h, int l) {
  return reinterpret_cast<T *>(base) + (int64_t)b * s.b + (int64_t)h * s.h + (int64_t)l * s.l;
}

// Which score branch a (BM x BN) tile needs under the piecewise rule
// "branch 2 iff (m + P_SEQ) - n >= w".
struct PwClass {
  bool need1, need2;
};
__device__ __forceinline__ PwClass pw_classify(int m0, int rows, int n0, int cols, int p_seq,
                                               int w) {
  int dmin = m0 + p_seq - (n0 + cols - 1);
  int dmax = m0 + rows - 1 + p_seq - n0;
  PwClass c;
  c.need2 = dmax >= w;  // some element is far
  c.need1 = dmin < w;   // some element is near
  return c;
}

}  // namespace fa
