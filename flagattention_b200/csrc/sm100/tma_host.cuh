// Host-side construction of TMA tensor maps for (B, H, L, D) operands with
// arbitrary outer strides.  cuTensorMapEncodeTiled is resolved through the
// runtime (cudaGetDriverEntryPoint) so the library does not link libcuda.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "flagattn_b200.h"

namespace fa {
namespace tc {

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Tensor map over a (B, H, L, D) 16-bit tensor; a box is `box_rows` rows of 64
// elements (128 bytes, 128-byte swizzle) of one (b, h).  Coordinates are
// (d, l, h, b).  Rows past L read as zeros.  A stride of 0 is accepted only on
// a dimension of extent 1 (where it is never multiplied by anything but 0 and
// a placeholder takes its place in the map); on a longer dimension it means a
// broadcast view (`expand`), which a tensor map cannot express.  Returns false
// for that, and when the driver rejects the layout: the caller then uses the
// shape-generic kernels, which index with the true strides.
inline bool make_map_bhld(CUtensorMap *map, const fa_tensor4 *t, int dtype, int B, int H, int L,
                          int D, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  if ((t->stride_l == 0 && L > 1) || (t->stride_h == 0 && H > 1) || (t->stride_b == 0 && B > 1))
    return false;
  const int64_t sl = t->stride_l ? t->stride_l : D;
  const int64_t sh = t->stride_h ? t->stride_h : (int64_t)L * sl;
  const int64_t sb = t->stride_b ? t->stride_b : (int64_t)H * sh;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)L, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)sl * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt =
      dtype == FA_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = fn(map, dt, 4, t->ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace tc
}  // namespace fa
