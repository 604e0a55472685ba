// Test hooks that exercise the failure path of the bounded waits without faulting or hanging
// the GPU: a wait that nothing will ever satisfy runs out after a small, caller-chosen number
// of polls, the kernel records the caller's code in the device's error word and returns.
#include "../common.h"
#include "sm100.cuh"

namespace fb {
namespace {

__global__ void wait_timeout_kernel(uint32_t spins, uint32_t code, uint32_t *err) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t b = sm100::smem_u32(&bar);
  if (threadIdx.x == 0) {
    sm100::mbar_init(b, 1);
    sm100::fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    bool arrived = false;
    for (uint32_t it = 0; it < spins && !arrived; ++it) arrived = sm100::mbar_try_wait(b, 0);
    if (!arrived) atomicOr(err, code); // the path every production wait takes when it gives up
  }
}

} // namespace
} // namespace fb

using namespace fb;

FB_EXPORT fb_status fb_device_selftest_wait_timeout(fb_device *dev, uint32_t spins, uint32_t code) {
  clear_error();
  FB_REQUIRE(dev != nullptr, FB_INVALID_ARGUMENT, "fb_device_selftest_wait_timeout: device is NULL");
  FB_REQUIRE(spins >= 1 && spins <= (1u << 20), FB_INVALID_ARGUMENT,
             "fb_device_selftest_wait_timeout: spins must be 1..2^20");
  FB_CUDA_OK(cudaSetDevice(dev->ordinal));
  wait_timeout_kernel<<<1, 32, 0, dev->stream>>>(spins, code, dev->error_word);
  FB_CUDA_OK(cudaGetLastError());
  return FB_OK;
}

FB_EXPORT fb_status fb_device_clear_kernel_error(fb_device *dev) {
  clear_error();
  FB_REQUIRE(dev != nullptr, FB_INVALID_ARGUMENT, "fb_device_clear_kernel_error: device is NULL");
  FB_CUDA_OK(cudaSetDevice(dev->ordinal));
  FB_CUDA_OK(cudaMemsetAsync(dev->error_word, 0, sizeof(uint32_t), dev->stream));
  return FB_OK;
}
