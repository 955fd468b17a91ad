// Shared device helpers: the integer requantisation every layer op ends with.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb200 {

// Per-output-channel epilogue constants (32 bytes, two 16-byte loads).
// bias already holds every input-zero-point correction that can be folded
// (bias - izp * sum(w) [+ K * izp * wzp]); mult/shift are the tosa.rescale pair
// (requant mode A) or the common-shift pair derived from it (mode B).
// rnd and dmul pre-compute the rounding of apply_scale_32 so that the epilogue is
//   t = acc * mult + rnd + [acc < 0] * dmul ;  r = t >> shift
// with rnd = 2^(S-1) (+ 2^30 when DOUBLE_ROUND applies, i.e. S > 31) and
// dmul = -2^31 in that case (so a negative acc sees 2^30 - 2^31 = -2^30), else 0.
struct __align__(16) ChanParams {
  int32_t bias;
  int32_t mult;
  int32_t shift;
  int32_t dmul;
  long long rnd;
  int32_t wsum;    // sum over K of raw weights (for kernels that correct per border class)
  int32_t hshift;  // shift - 32 (meaningful when every shift of the op is >= 32)
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

// Same result as requant() with the constants of ChanParams; HI = every shift of the op is >= 32,
// which turns the 64-bit shift into one shift of the high word.
template <bool HI>
__device__ __forceinline__ int32_t requant_cp(int32_t acc, const ChanParams& cp, int32_t ozp, int32_t cmin,
                                              int32_t cmax) {
  long long t = (long long)acc * (long long)cp.mult + cp.rnd;
  t += (long long)(int32_t)((uint32_t)acc >> 31) * (long long)cp.dmul;
  int32_t r = HI ? ((int32_t)(t >> 32) >> cp.hshift) : (int32_t)(t >> cp.shift);
  r += ozp;
  return max(cmin, min(cmax, r));
}

// 64-bit value from two 32-bit registers without any instruction (register pairing).
__device__ __forceinline__ long long make_i64(int32_t hi, int32_t lo) {
  return __double_as_longlong(__hiloint2double(hi, lo));
}

// Compact form of the rescale ("Q4"), one 16-byte record {4 * bias, mult, rh, shift - 30} per channel and no
// 64-bit arithmetic. With v = acc + bias:
//   (v * M + R) >> S  ==  (4v * M + 4R) >> (S + 2),
// and for S >= 32 the rounding constant 4R = 2^(S+1) (+- 2^32 with DOUBLE_ROUND) has a zero low word, so the
// low word of the product never carries into the result:
//   r = (mulhi(4v, M) + rh [+- 1 by the sign of v]) >> (S - 30),   rh = 2^(S-31) + (out_zp << (S - 30)).
// The output zero point rides in rh. The planner uses this form only when it has shown, from the weights and
// the bias, that |4v| stays below 2^31 and that every shift of the op lies in [32, 52].
// Double rounding: rh additionally holds the +1 of a non-negative v, and a negative v takes 2 back.
__device__ __forceinline__ int32_t scale_q4_sign(int32_t acc, const int4& c) {
  const int32_t v4 = acc * 4 + c.x;
  const int32_t neg = v4 >> 31;  // -1 for a negative accumulator
  return (__mulhi(v4, c.y) + c.z + neg + neg) >> c.w;
}
// Without the sign term: single rounding, or a clamp whose lower end is at or above the output zero point
// (ReLU-like): every negative v then lands on that lower end whichever way it is rounded.
__device__ __forceinline__ int32_t scale_q4(int32_t acc, const int4& c) {
  return (__mulhi(acc * 4 + c.x, c.y) + c.z) >> c.w;
}

// apply_scale_32 part of requant_cp (no zero point, no clamp).
template <bool HI>
__device__ __forceinline__ int32_t scale_cp(int32_t acc, const ChanParams& cp) {
  long long t = (long long)acc * (long long)cp.mult + cp.rnd;
  t += (long long)(int32_t)((uint32_t)acc >> 31) * (long long)cp.dmul;
  return HI ? ((int32_t)(t >> 32) >> cp.hshift) : (int32_t)(t >> cp.shift);
}

// Clamp four int32 values to [lo, hi] (a sub-range of int8, given replicated as s16x2)
// and pack them into one word: saturating pack to s16x2, packed min/max, byte select.
__device__ __forceinline__ uint32_t clamp_pack4(int32_t r0, int32_t r1, int32_t r2, int32_t r3, uint32_t lo2,
                                                uint32_t hi2) {
  uint32_t a, b;
  asm("cvt.pack.sat.s16.s32 %0, %1, %2;" : "=r"(a) : "r"(r1), "r"(r0));
  asm("cvt.pack.sat.s16.s32 %0, %1, %2;" : "=r"(b) : "r"(r3), "r"(r2));
  asm("max.s16x2 %0, %0, %1;" : "+r"(a) : "r"(lo2));
  asm("max.s16x2 %0, %0, %1;" : "+r"(b) : "r"(lo2));
  asm("min.s16x2 %0, %0, %1;" : "+r"(a) : "r"(hi2));
  asm("min.s16x2 %0, %0, %1;" : "+r"(b) : "r"(hi2));
  return __byte_perm(a, b, 0x6420);
}

// The same for the full int8 range: two saturating packs.
__device__ __forceinline__ uint32_t sat_pack4(int32_t r0, int32_t r1, int32_t r2, int32_t r3) {
  uint32_t a, b;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(a) : "r"(r3), "r"(r2));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(b) : "r"(r1), "r"(r0), "r"(a));
  return b;
}

__device__ __forceinline__ int32_t sx8(uint32_t word, int j) {
  return (int32_t)(int8_t)(word >> (8 * j));
}

__device__ __forceinline__ uint32_t pack4(int32_t a, int32_t b, int32_t c, int32_t d) {
  return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) |
         ((uint32_t)(d & 0xff) << 24);
}

}  // namespace tb200
