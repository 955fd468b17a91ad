// Measured ceiling of the int8 tensor pipe: every SM issues tcgen05.mma kind::i8 (M = 128, N = 256,
// K = 32 per instruction) back to back on operands that stay in shared memory, accumulating in TMEM.
// No global memory traffic inside the loop, so the rate it reaches is the denominator the contraction
// kernels' tensor-pipe fractions are quoted against. A measurement aid: the reference has no counterpart.
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/torq_b200.h"
#include "kernels.h"
#include "tcgen05_ptx.cuh"

namespace tb200 {
namespace {

constexpr int kPeakN = 256;          // columns of one accumulator; two of them fill the 512 TMEM columns
constexpr int kRowBytes = 128;       // one swizzle-128B row = 4 K steps of 32 bytes
constexpr int kBatch = 32;           // K blocks between two commits

__global__ void __launch_bounds__(128, 1) peak_i8_kernel(int rounds, int* status, unsigned long long wait_ns) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_done[2];
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_a = base, smem_b = base + 128 * kRowBytes;
  // any bytes will do as operands; a non-trivial pattern keeps the data path toggling as real tiles would
  for (uint32_t i = threadIdx.x; i < (128 + kPeakN) * kRowBytes / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(smem_raw + (base - smem_u32(smem_raw)))[i] = 0x9e3779b9u * (i + 1u + blockIdx.x);
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar_done[0]), 1);
    mbar_init(smem_u32(&bar_done[1]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kPeakN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    const uint64_t da = make_smem_desc(smem_a, kRowBytes), db = make_smem_desc(smem_b, kRowBytes);
    bool ok = true;
    // two accumulators in alternation; a commit per batch, and the issuer stays at most two batches ahead
    for (int r = 0; r < rounds && ok; r++) {
      const int acc = r & 1;
      if (r >= 2) ok = mbar_wait(smem_u32(&bar_done[acc]), ((r >> 1) - 1) & 1, status, 6, wait_ns);
      if (!ok) break;
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + (uint32_t)(acc * kPeakN);
      for (int kb = 0; kb < kBatch; kb++)
#pragma unroll
        for (int k = 0; k < 4; k++) mma_i8(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
      mma_commit(smem_u32(&bar_done[acc]));
    }
    // drain: the last commit of each accumulator
    for (int acc = 0; acc < 2 && ok; acc++) {
      const int uses = (rounds + 1 - acc) / 2;  // rounds with (r & 1) == acc
      if (uses > 0) ok = mbar_wait(smem_u32(&bar_done[acc]), (uses - 1) & 1, status, 6, wait_ns);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_measure_i8_mma_peak(int cuda_ordinal, int rounds, double* tera_ops_per_s, double* ms_out) {
  using namespace tb200;
  if (!tera_ops_per_s || rounds < 2 || rounds > (1 << 20) || cuda_ordinal < 0) return TB200_INVALID_ARGUMENT;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) return TB200_UNAVAILABLE;
  if (cuda_ordinal >= count) return TB200_NOT_FOUND;
  int caller = -1;
  if (cudaGetDevice(&caller) != cudaSuccess) return TB200_INTERNAL;
  struct Restore {
    int dev;
    ~Restore() { if (dev >= 0) cudaSetDevice(dev); }
  } restore{caller == cuda_ordinal ? -1 : caller};
  if (caller != cuda_ordinal && cudaSetDevice(cuda_ordinal) != cudaSuccess) return TB200_INTERNAL;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, cuda_ordinal) != cudaSuccess) return TB200_INTERNAL;
  if (prop.major != 10) return TB200_UNAVAILABLE;
  const size_t smem = 1024 + (size_t)(128 + kPeakN) * kRowBytes;
  if (cudaFuncSetAttribute(peak_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return TB200_INTERNAL;
  int* status = nullptr;
  cudaStream_t stream = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  int result = TB200_INTERNAL;
  float ms = 0.f;
  int code = 0;
  const int sms = current_sm_count();
  if (cudaMalloc(&status, kStatusBlockBytes) != cudaSuccess) return TB200_RESOURCE_EXHAUSTED;
  if (cudaMemset(status, 0, kStatusBlockBytes) == cudaSuccess && cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) == cudaSuccess &&
      cudaEventCreate(&e0) == cudaSuccess && cudaEventCreate(&e1) == cudaSuccess) {
    peak_i8_kernel<<<sms, 128, smem, stream>>>(rounds, status, wait_limit_ns());  // warm-up (clocks, instruction cache)
    cudaEventRecord(e0, stream);
    peak_i8_kernel<<<sms, 128, smem, stream>>>(rounds, status, wait_limit_ns());
    cudaEventRecord(e1, stream);
    if (cudaStreamSynchronize(stream) == cudaSuccess && cudaGetLastError() == cudaSuccess &&
        cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess &&
        cudaMemcpy(&code, status, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess)
      result = code == 0 ? TB200_OK : TB200_ABORTED;
  }
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  if (stream) cudaStreamDestroy(stream);
  cudaFree(status);
  if (result == TB200_OK) {
    const double ops = 2.0 * 128.0 * kPeakN * 32.0 * 4.0 * kBatch * (double)rounds * sms;
    *tera_ops_per_s = ops / ((double)ms * 1e-3) / 1e12;
    if (ms_out) *ms_out = ms;
  }
  return result;
}
