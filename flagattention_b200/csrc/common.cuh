// Shared device-side building blocks: 16-bit element traits, swizzled shared
// memory tiles filled by 16-byte cp.async, ldmatrix fragment loads and the
// m16n8k16 tensor-core MMA used by the shape-generic kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "flagattn_b200.h"

namespace fa {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---------------------------------------------------------------------------
// element traits
// ---------------------------------------------------------------------------
template <typename T>
struct Elem;

template <>
struct Elem<__half> {
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2 *>(&u));
  }
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                             uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};

template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&u));
  }
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                             uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};

// ---------------------------------------------------------------------------
// shared memory tiles: ROWS x D 16-bit elements, 16-byte chunks XOR-swizzled
// so that any 8 consecutive rows of one logical chunk column land in 8
// different 16-byte bank groups (conflict-free ldmatrix for every D).
// ---------------------------------------------------------------------------
template <int D>
struct Tile {
  static constexpr int kChunksPerRow = D / 8;                       // 16-byte chunks
  static constexpr int kRowsPerLine = kChunksPerRow >= 8 ? 1 : 8 / kChunksPerRow;
  static constexpr int kSwzMask = kChunksPerRow >= 8 ? 7 : kChunksPerRow - 1;
  // byte offset of (row, chunk) inside the tile
  static __device__ __forceinline__ uint32_t offset(int row, int chunk) {
    int sw = chunk ^ ((row / kRowsPerLine) & kSwzMask);
    return static_cast<uint32_t>((row * kChunksPerRow + sw) * 16);
  }
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte async copy global -> shared; copies zeros when !valid (no global read).
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid) {
  int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// Cooperative load of a ROWS x D tile whose row r lives at gptr + r*stride
// (elements); rows >= rows_valid are zero-filled.
template <typename T, int D, int ROWS, int NTHREADS>
__device__ __forceinline__ void load_tile_async(uint32_t smem_base, const T *gptr, int64_t stride,
                                                int rows_valid, int tid) {
  constexpr int CPR = Tile<D>::kChunksPerRow;
  constexpr int TOTAL = ROWS * CPR;
#pragma unroll
  for (int i = 0; i < (TOTAL + NTHREADS - 1) / NTHREADS; ++i) {
    int idx = tid + i * NTHREADS;
    if (TOTAL % NTHREADS == 0 || idx < TOTAL) {
      int row = idx / CPR, ch = idx % CPR;
      bool ok = row < rows_valid;
      const T *src = gptr + (ok ? (int64_t)row * stride + ch * 8 : 0);
      cp_async16(smem_base + Tile<D>::offset(row, ch), src, ok);
    }
  }
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// A fragment (16 rows x 16 k) of a row-major [row][k] tile: rows row0..row0+15,
// k columns kk*16..kk*16+15.
template <int D>
__device__ __forceinline__ void load_A(uint32_t (&a)[4], uint32_t tile, int row0, int kk,
                                       int lane) {
  ldsm_x4(a, tile + Tile<D>::offset(row0 + (lane & 15), kk * 2 + (lane >> 4)));
}
// B fragments for two adjacent n8 tiles from a row-major [n][k] tile (e.g. K
// for S = Q K^T): r[0],r[1] = (b0,b1) of n rows n0..n0+7, r[2],r[3] of n0+8..n0+15.
template <int D>
__device__ __forceinline__ void load_B_nk(uint32_t (&r)[4], uint32_t tile, int n0, int kk,
                                          int lane) {
  ldsm_x4(r, tile + Tile<D>::offset(n0 + (lane & 7) + ((lane >> 4) << 3),
                                    kk * 2 + ((lane >> 3) & 1)));
}
// B fragments for two adjacent n8 tiles from a row-major [k][n] tile (e.g. V
// for O = P V): k rows k0..k0+15, n chunks nc and nc+1 (8 columns each);
// r[0],r[1] = (b0,b1) of chunk nc, r[2],r[3] of chunk nc+1.
template <int D>
__device__ __forceinline__ void load_B_kn(uint32_t (&r)[4], uint32_t tile, int k0, int nc,
                                          int lane) {
  ldsm_x4_t(r, tile + Tile<D>::offset(k0 + (lane & 15), nc + (lane >> 4)));
}

__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  return v;
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// ---------------------------------------------------------------------------
// host-side helpers
// ---------------------------------------------------------------------------
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline bool tensor_ok(const fa_tensor4 *t) {
  return t && t->ptr;
}
inline bool tensor_aligned(const fa_tensor4 *t) {
  return aligned16(t->ptr) && t->stride_b % 8 == 0 && t->stride_h % 8 == 0 && t->stride_l % 8 == 0;
}

// Opt a kernel in to more than 48 KB of dynamic shared memory, once per device.
template <typename K>
inline int ensure_dyn_smem(K kernel, int bytes, unsigned long long *done_mask) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return FA_ERR_LAUNCH;
  const unsigned long long bit = 1ull << (dev & 63);
  if (!(*done_mask & bit)) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) !=
        cudaSuccess)
      return FA_ERR_LAUNCH;
    *done_mask |= bit;
  }
  return FA_OK;
}

#define FA_CHECK_LAUNCH()                                   \
  do {                                                      \
    if (cudaGetLastError() != cudaSuccess) return FA_ERR_LAUNCH; \
  } while (0)

}  // namespace fa
