// Programmatic dependent launch: a kernel launched through launch_dependent() may be scheduled while the kernel
// before it in the stream is still running (its blocks take the SMs the predecessor's blocks leave, and its
// prologue - shared-memory setup, barrier and TMEM allocation, loads of constants - runs in the predecessor's
// tail). Such a kernel must call grid_dependency_wait() before it reads or writes anything the predecessor may
// write or read: the wait returns once the predecessor has completed and its writes are visible. Without the
// launch attribute both device calls do nothing. TB200_NO_PDL=1 launches everything fully serialised (A/B aid).
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>
#include <utility>

namespace tb200 {

__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel's blocks be scheduled as soon as every block of this one has called it (or exited).
__device__ __forceinline__ void grid_dependency_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool dependent_launch_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("TB200_NO_PDL");
    v = !(e && *e && *e != '0');
  }
  return v != 0;
}

// Measured on MobileNetV2: with every launch programmatic the batch-256 step gains 1.3 %, the batch-1 inference
// (64 launches of a few microseconds each) loses 17 % - a programmatic edge costs about a microsecond that only a
// kernel with a real tail pays back. So the attribute is set for launches of at least kDependentMinBlocks blocks
// (or tiles, for the persistent kernels, which pass `large` themselves).
constexpr long long kDependentMinBlocks = 4 * 148;

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent_if(bool large, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                       cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = large && dependent_launch_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
  const long long blocks = (long long)grid.x * grid.y * grid.z;
  return launch_dependent_if(blocks >= kDependentMinBlocks, kernel, grid, block, smem, stream, std::forward<Args>(args)...);
}

}  // namespace tb200
