// A self-test of the bounded waits: one small CTA waits, with a short limit, on an mbarrier that
// nobody arrives at, and then leaves the way every tensor-core kernel leaves after a wait that ran
// out: the code of the wait goes into the device status word, the CTA-wide abort flag goes up and
// the kernel returns.  Nothing traps, faults or spins without end; the context stays usable.
#include "tc_common.cuh"
#include "../common.cuh"

namespace fa {
int *device_status_word();

namespace tc {

constexpr int kWaitProbeCode = 990;

__global__ void __launch_bounds__(64, 1) wait_probe_kernel(int *status, long long limit_cycles,
                                                           int *left_ok) {
  __shared__ __align__(8) uint64_t bar_mem;
  __shared__ int abort_flag;
  // like the real kernels: a poisoned status word means "do nothing"
  if (status && *reinterpret_cast<volatile int *>(status) != 0) return;
  const uint32_t bar = smem_u32(&bar_mem);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(bar, 1);
    fence_barrier_init();
  }
  __syncthreads();
  const AbortCtx actx{&abort_flag, status};
  // warp 0 waits for a phase that never completes; warp 1 waits on the same barrier and must be
  // released by the abort flag (or by its own limit), not by an arrival
  const bool ok = mbar_wait_limit(bar, 0, actx, kWaitProbeCode, limit_cycles);
  __syncthreads();
  if (threadIdx.x == 0 && left_ok) *left_ok = ok ? 0 : 1;
}

}  // namespace tc
}  // namespace fa

extern "C" int fa_debug_wait_probe(int64_t limit_cycles, int32_t *left_flag, void *stream) {
  if (limit_cycles <= 0 || limit_cycles > 20000000) return FA_ERR_BAD_ARG;  // at most ~10 ms
  int *status = fa::device_status_word();
  if (!status) return FA_ERR_LAUNCH;
  fa::tc::wait_probe_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(
      status, (long long)limit_cycles, left_flag);
  return cudaGetLastError() == cudaSuccess ? FA_OK : FA_ERR_LAUNCH;
}
