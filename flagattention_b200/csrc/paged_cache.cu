// Writer of the paged KV cache that paged_attention reads: the step a serving loop runs right
// before the decode kernel (new tokens' key / value rows -> their slots in the block pool).
// Pure data movement, HBM-bound: one CTA per token, 16-byte chunks, reads and writes coalesced.
#include <cuda_runtime.h>

#include <cstdint>

#include "common.cuh"
#include "flagattn_b200.h"

namespace fa {

// chunks = kv_heads * head_size / 8 sixteen-byte chunks per token and tensor
__global__ void __launch_bounds__(128)
    paged_cache_append_kernel(const uint4 *__restrict__ key, const uint4 *__restrict__ value,
                              int64_t src_stride_t, int64_t src_stride_h, uint4 *key_cache,
                              uint4 *value_cache, int64_t stride_b, int64_t stride_h,
                              int64_t stride_t, const int64_t *__restrict__ slot_mapping,
                              int block_size, int chunks_per_head, int chunks) {
  const int token = blockIdx.x;
  const int64_t slot = slot_mapping[token];
  if (slot < 0) return;   // padding token
  const int64_t blk = slot / block_size, off = slot % block_size;
  // all strides below are in 16-byte chunks
  const int64_t src = (int64_t)token * src_stride_t;
  const int64_t dst = blk * stride_b + off * stride_t;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const int h = c / chunks_per_head, d = c - h * chunks_per_head;
    const int64_t s = src + h * src_stride_h + d, t = dst + h * stride_h + d;
    key_cache[t] = key[s];
    value_cache[t] = value[s];
  }
}

}  // namespace fa

using namespace fa;

extern "C" int fa_paged_cache_append(int32_t dtype, int32_t num_tokens, int32_t num_kv_heads,
                                     int32_t head_size, int32_t block_size, const void *key,
                                     const void *value, int64_t src_stride_t, int64_t src_stride_h,
                                     void *key_cache, void *value_cache, int64_t cache_stride_b,
                                     int64_t cache_stride_h, int64_t cache_stride_t,
                                     const int64_t *slot_mapping, void *stream) {
  if (dtype != FA_F16 && dtype != FA_BF16) return FA_ERR_BAD_ARG;
  if (num_tokens < 0 || num_kv_heads <= 0 || head_size <= 0 || block_size <= 0) return FA_ERR_BAD_ARG;
  if (num_tokens == 0) return FA_OK;
  if (!key || !value || !key_cache || !value_cache || !slot_mapping) return FA_ERR_BAD_ARG;
  if (head_size % 8) return FA_ERR_UNSUPPORTED;
  auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al16(key) || !al16(value) || !al16(key_cache) || !al16(value_cache)) return FA_ERR_ALIGNMENT;
  if (src_stride_t % 8 || src_stride_h % 8 || cache_stride_b % 8 || cache_stride_h % 8 ||
      cache_stride_t % 8)
    return FA_ERR_ALIGNMENT;
  const int cph = head_size / 8;
  paged_cache_append_kernel<<<num_tokens, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4 *>(key), static_cast<const uint4 *>(value), src_stride_t / 8,
      src_stride_h / 8, static_cast<uint4 *>(key_cache), static_cast<uint4 *>(value_cache),
      cache_stride_b / 8, cache_stride_h / 8, cache_stride_t / 8, slot_mapping, block_size, cph,
      cph * num_kv_heads);
  FA_CHECK_LAUNCH();
  return FA_OK;
}
