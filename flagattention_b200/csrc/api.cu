// Status strings, build identification and the device status word.
#include <cuda_runtime.h>

#include "attn_params.cuh"
#include "flagattn_b200.h"

namespace fa {

__global__ void dropout_mask_kernel(uint8_t *mask, uint64_t total, float dropout_p, uint64_t seed,
                                    uint64_t offset) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (uint64_t)gridDim.x * blockDim.x)
    mask[i] = dropout_keep(seed, offset, i, dropout_p) ? 1 : 0;
}


// Written by a kernel whose bounded wait ran out (the code says which wait);
// zero in normal operation.  One word per device, inside the library image.
__device__ int g_device_status[4];

// Device address of the status word of the current device, or null.
int *device_status_word() {
  void *ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, g_device_status) != cudaSuccess) return nullptr;
  return static_cast<int *>(ptr);
}

namespace tc {
int reset_fwd_sched();   // flash_fwd_tc.cu
}

}  // namespace fa

extern "C" const char *fa_status_string(int status) {
  switch (status) {
    case FA_OK: return "ok";
    case FA_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size or bad enum)";
    case FA_ERR_UNSUPPORTED: return "unsupported head size, dtype or group size";
    case FA_ERR_ALIGNMENT: return "pointer or stride is not 16-byte aligned";
    case FA_ERR_LAUNCH: return "CUDA launch failed";
    case FA_ERR_WORKSPACE: return "workspace pointer missing or too small";
    case FA_ERR_TOO_LARGE: return "request exceeds a fixed built-in capacity";
  }
  return "unknown status";
}

extern "C" const char *fa_version(void) { return "flagattn_b200 1 sm_100a"; }

extern "C" int fa_dropout_mask(int32_t B, int32_t H, int32_t M, int32_t N, float dropout_p,
                               uint64_t philox_seed, uint64_t philox_offset, uint8_t *mask,
                               void *stream) {
  if (!mask || B <= 0 || H <= 0 || M <= 0 || N <= 0) return FA_ERR_BAD_ARG;
  const uint64_t total = (uint64_t)B * H * M * N;
  const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 32 ? (total + 255) / 256 : 148 * 32);
  fa::dropout_mask_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      mask, total, dropout_p, philox_seed, philox_offset);
  return cudaGetLastError() == cudaSuccess ? FA_OK : FA_ERR_LAUNCH;
}

extern "C" int fa_device_status(int32_t *out, int32_t clear) {
  if (!out) return FA_ERR_BAD_ARG;
  int *word = fa::device_status_word();
  if (!word) return FA_ERR_LAUNCH;
  if (cudaMemcpy(out, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return FA_ERR_LAUNCH;
  if (clear && *out != 0) {
    int zero = 0;
    if (cudaMemcpy(word, &zero, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess)
      return FA_ERR_LAUNCH;
    // a forward launch that gave up may have left its work-item counter mid-way
    if (fa::tc::reset_fwd_sched() != FA_OK) return FA_ERR_LAUNCH;
  }
  return FA_OK;
}
