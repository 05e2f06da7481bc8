// Producer of piecewise_attention's operands: one tensor x goes through TWO rotary position
// embeddings in one pass (x is read once, both rotated copies are written), and the backward
// folds the two incoming gradients back into one (both read once, dx written once).
// Pure element-wise work, HBM-bound: 6 bytes of traffic per element either way.
//
// Thread = 16 elements of one (position) row = 8 rotation pairs, so both layouts use two 16-byte
// accesses per tensor and the same eight table columns:
//   half-split  (pairs (i, i + D/2)):   chunks at elements 8j and D/2 + 8j
//   interleaved (pairs (2i, 2i + 1)):   chunks at elements 16j and 16j + 8
// The cos / sin values of a position are the same for every head, so a thread fetches its 32
// table values once and walks the heads of its row with them in registers.
//
// The arithmetic is written with explicitly rounded multiplies and adds (no fused multiply-add)
// so that the result is the same bit pattern as the plain fp32 expression evaluated on a CPU.
#include <cuda_runtime.h>

#include <cstdint>

#include "attn_params.cuh"
#include "common.cuh"
#include "flagattn_b200.h"

namespace fa {

struct RotaryTables {
  const float *cos1, *sin1, *cos2, *sin2;
  int64_t stride;   // elements between the rows of two positions
  int rows;
};

constexpr int kRotaryThreads = 128;   // four CTAs per SM at the kernels' register count

struct RotaryCoef {
  float c1[8], s1[8], c2[8], s2[8];
};

__device__ __forceinline__ void load8(float (&dst)[8], const float *src) {
  const float4 a = *reinterpret_cast<const float4 *>(src);
  const float4 b = *reinterpret_cast<const float4 *>(src + 4);
  dst[0] = a.x, dst[1] = a.y, dst[2] = a.z, dst[3] = a.w;
  dst[4] = b.x, dst[5] = b.y, dst[6] = b.z, dst[7] = b.w;
}

template <typename T>
__device__ __forceinline__ void unpack8(float (&dst)[8], const uint4 &u) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = Elem<T>::unpack(w[i]);
    dst[2 * i] = f.x, dst[2 * i + 1] = f.y;
  }
}

template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 u;
  u.x = Elem<T>::pack(v[0], v[1]);
  u.y = Elem<T>::pack(v[2], v[3]);
  u.z = Elem<T>::pack(v[4], v[5]);
  u.w = Elem<T>::pack(v[6], v[7]);
  return u;
}

// a[i], b[i] are the two members of pair i in the half-split layout; in the interleaved layout
// the sixteen values are a[0..7] = elements 0..7 and b[0..7] = elements 8..15 of the thread's run.
template <bool INTERLEAVED>
__device__ __forceinline__ void to_pairs(float (&lo)[8], float (&hi)[8], const float (&a)[8],
                                         const float (&b)[8]) {
  if (INTERLEAVED) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo[i] = a[2 * i], hi[i] = a[2 * i + 1];
      lo[4 + i] = b[2 * i], hi[4 + i] = b[2 * i + 1];
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) lo[i] = a[i], hi[i] = b[i];
  }
}

template <bool INTERLEAVED>
__device__ __forceinline__ void from_pairs(float (&a)[8], float (&b)[8], const float (&lo)[8],
                                           const float (&hi)[8]) {
  if (INTERLEAVED) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      a[2 * i] = lo[i], a[2 * i + 1] = hi[i];
      b[2 * i] = lo[4 + i], b[2 * i + 1] = hi[4 + i];
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = lo[i], b[i] = hi[i];
  }
}

// Row / column bookkeeping shared by the two kernels.  Returns false for idle threads.
struct RotaryWork {
  int b, l, h_lo, h_hi;
  int off_a, off_b;   // element offsets of the thread's two chunks inside a row
};

template <bool INTERLEAVED>
__device__ __forceinline__ bool rotary_setup(RotaryWork &w, RotaryCoef &co, const RotaryTables &t,
                                             const int64_t *positions, int64_t pos_stride_b, int B,
                                             int H, int L, int D, int heads_per_cta) {
  const int tpr = D / 16, rows = kRotaryThreads / tpr;
  const int r = threadIdx.x / tpr, j = threadIdx.x - r * tpr;
  // CTA order: head chunk fastest, then batch, then row block, so that the CTAs that read the same
  // table rows run at the same time and the rows are fetched from DRAM once
  const int Z = (H + heads_per_cta - 1) / heads_per_cta;
  const unsigned bx = blockIdx.x;
  const int hz = bx % Z;
  w.b = (bx / Z) % B;
  w.l = (int)(bx / ((unsigned)Z * B)) * rows + r;
  w.h_lo = hz * heads_per_cta;
  w.h_hi = min(H, w.h_lo + heads_per_cta);
  if (r >= rows || w.l >= L) return false;
  w.off_a = INTERLEAVED ? 16 * j : 8 * j;
  w.off_b = INTERLEAVED ? 16 * j + 8 : D / 2 + 8 * j;
  int64_t pos = positions ? positions[w.b * pos_stride_b + w.l] : w.l;
  // a position outside the tables reads the nearest row instead of foreign memory
  pos = pos < 0 ? 0 : (pos >= t.rows ? t.rows - 1 : pos);
  const int64_t at = pos * t.stride + 8 * j;
  load8(co.c1, t.cos1 + at);
  load8(co.s1, t.sin1 + at);
  load8(co.c2, t.cos2 + at);
  load8(co.s2, t.sin2 + at);
  return true;
}

template <typename T, bool INTERLEAVED>
__global__ void __launch_bounds__(kRotaryThreads, 4)
    rotary_pair_fwd_kernel(const T *__restrict__ x, Strides sx, T *__restrict__ out1, Strides s1,
                           T *__restrict__ out2, Strides s2, RotaryTables t, const int64_t *__restrict__ positions,
                           int64_t pos_stride_b, int B, int H, int L, int D, int heads_per_cta) {
  RotaryWork w;
  RotaryCoef co;
  if (!rotary_setup<INTERLEAVED>(w, co, t, positions, pos_stride_b, B, H, L, D, heads_per_cta))
    return;
#pragma unroll 4
  for (int h = w.h_lo; h < w.h_hi; ++h) {
    const T *src = x + w.b * sx.b + h * sx.h + w.l * sx.l;
    float a[8], b[8], lo[8], hi[8], ylo[8], yhi[8];
    unpack8<T>(a, *reinterpret_cast<const uint4 *>(src + w.off_a));
    unpack8<T>(b, *reinterpret_cast<const uint4 *>(src + w.off_b));
    to_pairs<INTERLEAVED>(lo, hi, a, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      ylo[i] = __fsub_rn(__fmul_rn(lo[i], co.c1[i]), __fmul_rn(hi[i], co.s1[i]));
      yhi[i] = __fadd_rn(__fmul_rn(hi[i], co.c1[i]), __fmul_rn(lo[i], co.s1[i]));
    }
    from_pairs<INTERLEAVED>(a, b, ylo, yhi);
    T *d1 = out1 + w.b * s1.b + h * s1.h + w.l * s1.l;
    *reinterpret_cast<uint4 *>(d1 + w.off_a) = pack8<T>(a);
    *reinterpret_cast<uint4 *>(d1 + w.off_b) = pack8<T>(b);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      ylo[i] = __fsub_rn(__fmul_rn(lo[i], co.c2[i]), __fmul_rn(hi[i], co.s2[i]));
      yhi[i] = __fadd_rn(__fmul_rn(hi[i], co.c2[i]), __fmul_rn(lo[i], co.s2[i]));
    }
    from_pairs<INTERLEAVED>(a, b, ylo, yhi);
    T *d2 = out2 + w.b * s2.b + h * s2.h + w.l * s2.l;
    *reinterpret_cast<uint4 *>(d2 + w.off_a) = pack8<T>(a);
    *reinterpret_cast<uint4 *>(d2 + w.off_b) = pack8<T>(b);
  }
}

// dx = R1^T g1 + R2^T g2; the transpose of a rotation is the rotation by the opposite angle.
template <typename T, bool INTERLEAVED>
__global__ void __launch_bounds__(kRotaryThreads, 4)
    rotary_pair_bwd_kernel(const T *__restrict__ g1, Strides s1, const T *__restrict__ g2,
                           Strides s2, T *__restrict__ dx, Strides sx, RotaryTables t,
                           const int64_t *__restrict__ positions, int64_t pos_stride_b, int B, int H,
                           int L, int D, int heads_per_cta) {
  RotaryWork w;
  RotaryCoef co;
  if (!rotary_setup<INTERLEAVED>(w, co, t, positions, pos_stride_b, B, H, L, D, heads_per_cta))
    return;
#pragma unroll 4
  for (int h = w.h_lo; h < w.h_hi; ++h) {
    const T *p1 = g1 + w.b * s1.b + h * s1.h + w.l * s1.l;
    const T *p2 = g2 + w.b * s2.b + h * s2.h + w.l * s2.l;
    float a[8], b[8], lo1[8], hi1[8], lo2[8], hi2[8], ylo[8], yhi[8];
    unpack8<T>(a, *reinterpret_cast<const uint4 *>(p1 + w.off_a));
    unpack8<T>(b, *reinterpret_cast<const uint4 *>(p1 + w.off_b));
    to_pairs<INTERLEAVED>(lo1, hi1, a, b);
    unpack8<T>(a, *reinterpret_cast<const uint4 *>(p2 + w.off_a));
    unpack8<T>(b, *reinterpret_cast<const uint4 *>(p2 + w.off_b));
    to_pairs<INTERLEAVED>(lo2, hi2, a, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float l1 = __fadd_rn(__fmul_rn(lo1[i], co.c1[i]), __fmul_rn(hi1[i], co.s1[i]));
      const float l2 = __fadd_rn(__fmul_rn(lo2[i], co.c2[i]), __fmul_rn(hi2[i], co.s2[i]));
      const float h1 = __fsub_rn(__fmul_rn(hi1[i], co.c1[i]), __fmul_rn(lo1[i], co.s1[i]));
      const float h2 = __fsub_rn(__fmul_rn(hi2[i], co.c2[i]), __fmul_rn(lo2[i], co.s2[i]));
      ylo[i] = __fadd_rn(l1, l2);
      yhi[i] = __fadd_rn(h1, h2);
    }
    from_pairs<INTERLEAVED>(a, b, ylo, yhi);
    T *d = dx + w.b * sx.b + h * sx.h + w.l * sx.l;
    *reinterpret_cast<uint4 *>(d + w.off_a) = pack8<T>(a);
    *reinterpret_cast<uint4 *>(d + w.off_b) = pack8<T>(b);
  }
}

namespace {

struct RotaryLaunch {
  dim3 grid;
  int heads_per_cta;
};

// Rows of one CTA share nothing, so the heads are split over grid.z until the grid is some twenty
// waves of resident CTAs deep: short sequences then still fill the machine, and long ones end
// without a long under-filled last wave.  A CTA keeps at least a few heads where it can, since
// its threads fetch their table values once per CTA.
RotaryLaunch plan(int B, int H, int L, int D) {
  const int rows = kRotaryThreads / (D / 16);
  const int gx = (L + rows - 1) / rows;
  const int64_t want = 148 * 4 * 20;
  int z = (int)((want + (int64_t)gx * B - 1) / ((int64_t)gx * B));
  z = z < 1 ? 1 : (z > H ? H : z);
  const int hpc = (H + z - 1) / z;
  z = (H + hpc - 1) / hpc;
  return {dim3((unsigned)((int64_t)gx * B * z)), hpc};
}

int check_common(int32_t dtype, int32_t B, int32_t H, int32_t L, int32_t D, const float *cos1,
                 const float *sin1, const float *cos2, const float *sin2, int64_t table_stride,
                 int32_t table_rows) {
  if (dtype != FA_F16 && dtype != FA_BF16) return FA_ERR_BAD_ARG;
  if (B < 0 || H < 0 || L < 0 || D <= 0 || table_rows <= 0) return FA_ERR_BAD_ARG;
  if (D % 16 || D > 512) return FA_ERR_UNSUPPORTED;
  if (!cos1 || !sin1 || !cos2 || !sin2) return FA_ERR_BAD_ARG;
  if (table_stride < D / 2 || table_stride % 4) return FA_ERR_ALIGNMENT;
  if (!aligned16(cos1) || !aligned16(sin1) || !aligned16(cos2) || !aligned16(sin2))
    return FA_ERR_ALIGNMENT;
  if ((int64_t)B * H * ((L + 1) / 2 + 1) >= (1ll << 31)) return FA_ERR_TOO_LARGE;   // one-dimensional grid
  return FA_OK;
}

}  // namespace
}  // namespace fa

using namespace fa;

extern "C" int fa_rotary_pair_fwd(int32_t dtype, int32_t B, int32_t H, int32_t L, int32_t D,
                                  int32_t interleaved, const fa_tensor4 *x, const float *cos1,
                                  const float *sin1, const float *cos2, const float *sin2,
                                  int64_t table_stride, int32_t table_rows,
                                  const int64_t *positions, int64_t pos_stride_b,
                                  const fa_tensor4 *out1, const fa_tensor4 *out2, void *stream) {
  const int rc = check_common(dtype, B, H, L, D, cos1, sin1, cos2, sin2, table_stride, table_rows);
  if (rc != FA_OK) return rc;
  if (B == 0 || H == 0 || L == 0) return FA_OK;
  if (!tensor_ok(x) || !tensor_ok(out1) || !tensor_ok(out2)) return FA_ERR_BAD_ARG;
  if (!tensor_aligned(x) || !tensor_aligned(out1) || !tensor_aligned(out2)) return FA_ERR_ALIGNMENT;
  const RotaryLaunch pl = plan(B, H, L, D);
  const RotaryTables t{cos1, sin1, cos2, sin2, table_stride, table_rows};
  auto s = static_cast<cudaStream_t>(stream);
#define FA_ROT_FWD(T, IL)                                                                       \
  rotary_pair_fwd_kernel<T, IL><<<pl.grid, kRotaryThreads, 0, s>>>(                             \
      static_cast<const T *>(x->ptr), strides_of(x), static_cast<T *>(out1->ptr), strides_of(out1),             \
      static_cast<T *>(out2->ptr), strides_of(out2), t, positions, pos_stride_b, B, H, L, D,            \
      pl.heads_per_cta)
  if (dtype == FA_F16) {
    if (interleaved) FA_ROT_FWD(__half, true); else FA_ROT_FWD(__half, false);
  } else {
    if (interleaved) FA_ROT_FWD(__nv_bfloat16, true); else FA_ROT_FWD(__nv_bfloat16, false);
  }
#undef FA_ROT_FWD
  FA_CHECK_LAUNCH();
  return FA_OK;
}

extern "C" int fa_rotary_pair_bwd(int32_t dtype, int32_t B, int32_t H, int32_t L, int32_t D,
                                  int32_t interleaved, const fa_tensor4 *g1, const fa_tensor4 *g2,
                                  const float *cos1, const float *sin1, const float *cos2,
                                  const float *sin2, int64_t table_stride, int32_t table_rows,
                                  const int64_t *positions, int64_t pos_stride_b,
                                  const fa_tensor4 *dx, void *stream) {
  const int rc = check_common(dtype, B, H, L, D, cos1, sin1, cos2, sin2, table_stride, table_rows);
  if (rc != FA_OK) return rc;
  if (B == 0 || H == 0 || L == 0) return FA_OK;
  if (!tensor_ok(g1) || !tensor_ok(g2) || !tensor_ok(dx)) return FA_ERR_BAD_ARG;
  if (!tensor_aligned(g1) || !tensor_aligned(g2) || !tensor_aligned(dx)) return FA_ERR_ALIGNMENT;
  const RotaryLaunch pl = plan(B, H, L, D);
  const RotaryTables t{cos1, sin1, cos2, sin2, table_stride, table_rows};
  auto s = static_cast<cudaStream_t>(stream);
#define FA_ROT_BWD(T, IL)                                                                       \
  rotary_pair_bwd_kernel<T, IL><<<pl.grid, kRotaryThreads, 0, s>>>(                             \
      static_cast<const T *>(g1->ptr), strides_of(g1), static_cast<const T *>(g2->ptr), strides_of(g2),         \
      static_cast<T *>(dx->ptr), strides_of(dx), t, positions, pos_stride_b, B, H, L, D,                \
      pl.heads_per_cta)
  if (dtype == FA_F16) {
    if (interleaved) FA_ROT_BWD(__half, true); else FA_ROT_BWD(__half, false);
  } else {
    if (interleaved) FA_ROT_BWD(__nv_bfloat16, true); else FA_ROT_BWD(__nv_bfloat16, false);
  }
#undef FA_ROT_BWD
  FA_CHECK_LAUNCH();
  return FA_OK;
}
