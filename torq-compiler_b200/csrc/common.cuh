// Shared device helpers: the integer requantisation every layer op ends with.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb200 {

// Per-output-channel epilogue constants, one 16-byte load per channel.
// bias already holds every input-zero-point correction that can be folded
// (bias - izp * sum(w) [+ K * izp * wzp]); mult/shift are the tosa.rescale pair
// (requant mode A) or the common-shift pair derived from it (mode B).
struct __align__(16) ChanParams {
  int32_t bias;
  int32_t mult;
  int32_t shift;
  int32_t wsum;  // sum over K of raw weights (used by kernels that correct per border)
};

// TOSA apply_scale_32. The reference matches the chain
// apply_scale -> addi(zp) -> maxsi -> minsi -> trunci
// (compiler/torq/Conversions/LinalgToTorqHL/PatternUtils.cpp:3441-3451).
__device__ __forceinline__ int32_t apply_scale_32(int32_t v, int32_t mult, int32_t shift, bool dround) {
  long long round = 1ll << (shift - 1);
  if (dround && shift > 31) round += (v >= 0) ? (1ll << 30) : -(1ll << 30);
  long long r = (long long)v * (long long)mult + round;
  return (int32_t)(r >> shift);
}

__device__ __forceinline__ int32_t requant(int32_t acc, int32_t mult, int32_t shift, bool dround,
                                           int32_t ozp, int32_t cmin, int32_t cmax) {
  int32_t r = apply_scale_32(acc, mult, shift, dround) + ozp;  // int32 wraps on device
  return max(cmin, min(cmax, r));
}

__device__ __forceinline__ int32_t sx8(uint32_t word, int j) {
  return (int32_t)(int8_t)(word >> (8 * j));
}

__device__ __forceinline__ uint32_t pack4(int32_t a, int32_t b, int32_t c, int32_t d) {
  return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) |
         ((uint32_t)(d & 0xff) << 24);
}

}  // namespace tb200
