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
  // dropout (flash forward only): keep iff uniform(seed, offset + linear index) > dropout_p
  float dropout_p;
  uint64_t seed, offset;
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
  float dropout_p;
  uint64_t seed, offset;
};

// First output word of Philox-4x32 with 6 rounds, counter (c0, c1, 0, 0), key (k0, k1).
__host__ __device__ __forceinline__ uint32_t philox4x32_6(uint32_t k0, uint32_t k1, uint32_t c0,
                                                          uint32_t c1) {
  uint32_t c2 = 0, c3 = 0;
#pragma unroll
  for (int r = 0; r < 6; ++r) {
    const uint32_t a0 = c0, a2 = c2;
    const uint64_t pb = (uint64_t)0xCD9E8D57u * a2, pa = (uint64_t)0xD2511F53u * a0;
    c0 = (uint32_t)(pb >> 32) ^ c1 ^ k0;
    c2 = (uint32_t)(pa >> 32) ^ c3 ^ k1;
    c1 = (uint32_t)pb;
    c3 = (uint32_t)pa;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}
// Dropout decision of attention element `idx` (= ((b*H + h)*M + m)*N + n): true = keep.
__host__ __device__ __forceinline__ bool dropout_keep(uint64_t seed, uint64_t offset, uint64_t idx,
                                                      float dropout_p) {
  const uint64_t ctr = offset + idx;
  int32_t x = (int32_t)philox4x32_6((uint32_t)seed, (uint32_t)(seed >> 32), (uint32_t)ctr,
                                    (uint32_t)(ctr >> 32));
  if (x < 0) x = -x - 1;
  return (float)x * 4.6566127342e-10f > dropout_p;
}

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
