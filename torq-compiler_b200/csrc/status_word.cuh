// The device status block a kernel reports an expired bounded wait into.
// Layout (16 bytes, device memory): int code at byte 0 (0 = nothing failed; kernels poll it inside their
// wait loops so that one failure ends every other wait early), and at byte 8 a device-visible pointer to a
// word in mapped pinned host memory (or NULL). The failing thread stores the code to both, so the host
// reads the outcome of a dispatch from its own memory once the stream has drained: no copy is queued on
// the success path.
#pragma once
#include <cuda_runtime.h>

namespace tb200 {

constexpr size_t kStatusBlockBytes = 16;

__device__ __forceinline__ void report_expired_wait(int* status, int code) {
  if (atomicCAS(status, 0, code) == 0) {
    int* mirror = *reinterpret_cast<int* const*>(status + 2);
    if (mirror) {
      *reinterpret_cast<volatile int*>(mirror) = code;
      __threadfence_system();
    }
  }
}

}  // namespace tb200
