// Bandwidth-bound layer kernels: pooling, rescaled add/sub/mul, 256-entry table,
// standalone rescale (also the building block of a rescaled concat), 2x nearest
// resize. 128-bit accesses wherever the channel count allows; grids sized in
// whole multiples of the SM count with grid-stride loops.
#include "kernels.h"
#include "dependent_launch.cuh"

namespace tb200 {

namespace {

constexpr int kThreads = 256;

inline unsigned grid_for(long long work_items, int per_block = kThreads) {
  long long blocks = (work_items + per_block - 1) / per_block;
  const long long cap = 148LL * 16;  // 148 SMs x resident blocks; the loops stride over the rest
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

// ---- max pool: torq_hl.maxpool2d (PoolingPattern.cpp:128-258) ----
template <int VEC>  // channels per thread: 16 (uint4) or 1
__global__ void __launch_bounds__(kThreads) maxpool_kernel(PoolArgs a) {
  grid_dependency_release();
  grid_dependency_wait();
  const int groups = a.C / VEC;
  const long long total = (long long)a.N * a.OH * a.OW * groups;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    int g = (int)(idx % groups);
    long long p = idx / groups;
    int ow = (int)(p % a.OW);
    long long t = p / a.OW;
    int oh = (int)(t % a.OH);
    int n = (int)(t / a.OH);
    const int8_t* xin = a.x + (size_t)n * a.H * a.W * a.C + g * VEC;
    if (VEC == 16) {
      uint32_t best[4] = {0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u};
      const uint32_t padw = (uint32_t)(a.pad_value & 0xff) * 0x01010101u;
      for (int kh = 0; kh < a.KH; kh++) {
        int ih = oh * a.stride_h - a.pad_t + kh;
        for (int kw = 0; kw < a.KW; kw++) {
          int iw = ow * a.stride_w - a.pad_l + kw;
          uint4 v;
          if (ih < 0 || ih >= a.H || iw < 0 || iw >= a.W) v = make_uint4(padw, padw, padw, padw);
          else v = *reinterpret_cast<const uint4*>(xin + ((size_t)ih * a.W + iw) * a.C);
          best[0] = __vmaxs4(best[0], v.x);
          best[1] = __vmaxs4(best[1], v.y);
          best[2] = __vmaxs4(best[2], v.z);
          best[3] = __vmaxs4(best[3], v.w);
        }
      }
      *reinterpret_cast<uint4*>(a.out + (size_t)p * a.C + g * 16) = make_uint4(best[0], best[1], best[2], best[3]);
    } else {
      int best = -128;
      for (int kh = 0; kh < a.KH; kh++) {
        int ih = oh * a.stride_h - a.pad_t + kh;
        for (int kw = 0; kw < a.KW; kw++) {
          int iw = ow * a.stride_w - a.pad_l + kw;
          int v = (ih < 0 || ih >= a.H || iw < 0 || iw >= a.W) ? a.pad_value
                                                               : (int)xin[((size_t)ih * a.W + iw) * a.C];
          best = max(best, v);
        }
      }
      a.out[(size_t)p * a.C + g] = (int8_t)best;
    }
  }
}

// The same on int16 tensors (the reference's MaxPool2D i16 -> i16): 8 channels per thread, or 1.
template <int VEC>
__global__ void __launch_bounds__(kThreads) maxpool_i16_kernel(PoolArgs a) {
  const int16_t* x = reinterpret_cast<const int16_t*>(a.x);
  int16_t* out = reinterpret_cast<int16_t*>(a.out);
  const int groups = a.C / VEC;
  const long long total = (long long)a.N * a.OH * a.OW * groups;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int g = (int)(idx % groups);
    const long long p = idx / groups;
    const int ow = (int)(p % a.OW);
    const long long t = p / a.OW;
    const int oh = (int)(t % a.OH);
    const int n = (int)(t / a.OH);
    const int16_t* xin = x + (size_t)n * a.H * a.W * a.C + g * VEC;
    if (VEC == 8) {
      uint32_t best[4] = {0x80008000u, 0x80008000u, 0x80008000u, 0x80008000u};
      const uint32_t padw = (uint32_t)(a.pad_value & 0xffff) * 0x00010001u;
      for (int kh = 0; kh < a.KH; kh++) {
        const int ih = oh * a.stride_h - a.pad_t + kh;
        for (int kw = 0; kw < a.KW; kw++) {
          const int iw = ow * a.stride_w - a.pad_l + kw;
          uint4 v;
          if (ih < 0 || ih >= a.H || iw < 0 || iw >= a.W) v = make_uint4(padw, padw, padw, padw);
          else v = *reinterpret_cast<const uint4*>(xin + ((size_t)ih * a.W + iw) * a.C);
          best[0] = __vmaxs2(best[0], v.x);
          best[1] = __vmaxs2(best[1], v.y);
          best[2] = __vmaxs2(best[2], v.z);
          best[3] = __vmaxs2(best[3], v.w);
        }
      }
      *reinterpret_cast<uint4*>(out + (size_t)p * a.C + g * 8) = make_uint4(best[0], best[1], best[2], best[3]);
    } else {
      int best = -32768;
      for (int kh = 0; kh < a.KH; kh++) {
        const int ih = oh * a.stride_h - a.pad_t + kh;
        for (int kw = 0; kw < a.KW; kw++) {
          const int iw = ow * a.stride_w - a.pad_l + kw;
          const int v = (ih < 0 || ih >= a.H || iw < 0 || iw >= a.W) ? a.pad_value : (int)xin[((size_t)ih * a.W + iw) * a.C];
          best = max(best, v);
        }
      }
      out[(size_t)p * a.C + g] = (int16_t)best;
    }
  }
}

// reciprocal_scale of the TOSA spec (compiler/torq/Conversions/TosaToTorqHL/Patterns.cpp:796-805)
__device__ __forceinline__ void reciprocal_scale(uint32_t count, int32_t& mult, int32_t& shift) {
  int k = 32 - __clz((int)(count - 1));
  if (count == 1) k = 0;
  long long numerator = ((1ll << 30) + 1) << k;
  mult = (int32_t)(numerator / (long long)count);
  shift = 30 + k;
}

// ---- average pool: tosa.avg_pool2d acc_type=i32; count excludes padding ----
// The rescale depends only on the number of taps inside the image, so the block fills a table indexed by that
// count once (one 64-bit division per entry instead of one per output). Entry {M, 2^(S-30), S-29, count}:
// TOSA's (v * M + 2^(S-1)) >> S with S = 30 + k >= 30 equals (8v * M + 2^(S+2)) >> (S + 3), and since the constant
// has a zero low word that is (mulhi(8v, M) + 2^(S-30)) >> (S - 29): exact, 32-bit.
constexpr int kAvgMaxTaps = 256;
template <int VEC>  // 16, 4 or 1 channels per thread
__global__ void __launch_bounds__(kThreads) avgpool_kernel(PoolArgs a) {
  grid_dependency_release();
  grid_dependency_wait();
  __shared__ int4 by_count[kAvgMaxTaps + 1];
  for (int c = threadIdx.x; c <= a.KH * a.KW; c += blockDim.x) {
    int32_t mult, shift;
    reciprocal_scale(c ? (uint32_t)c : 1u, mult, shift);
    by_count[c] = make_int4(mult, 1 << (shift - 30), shift - 29, c);
  }
  __syncthreads();
  const int groups = a.C / VEC;
  const long long total = (long long)a.N * a.OH * a.OW * groups;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    int g = (int)(idx % groups);
    long long p = idx / groups;
    int ow = (int)(p % a.OW);
    long long t = p / a.OW;
    int oh = (int)(t % a.OH);
    int n = (int)(t / a.OH);
    const int8_t* xin = a.x + (size_t)n * a.H * a.W * a.C + g * VEC;
    int acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; j++) acc[j] = 0;
    int count = 0;
    for (int kh = 0; kh < a.KH; kh++) {
      int ih = oh * a.stride_h - a.pad_t + kh;
      if (ih < 0 || ih >= a.H) continue;
      for (int kw = 0; kw < a.KW; kw++) {
        int iw = ow * a.stride_w - a.pad_l + kw;
        if (iw < 0 || iw >= a.W) continue;
        count++;
        const int8_t* px = xin + ((size_t)ih * a.W + iw) * a.C;
        if (VEC == 16) {
          const uint4 v = *reinterpret_cast<const uint4*>(px);
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int j = 0; j < 16; j++) acc[j] = __dp4a((int)w[j >> 2], 1 << (8 * (j & 3)), acc[j]);  // adds byte j, sign-extended
        } else if (VEC == 4) {
          const uint32_t v = *reinterpret_cast<const uint32_t*>(px);
#pragma unroll
          for (int j = 0; j < 4; j++) acc[j] = __dp4a((int)v, 1 << (8 * j), acc[j]);
        } else {
          acc[0] += (int)px[0];
        }
      }
    }
    const int4 k = by_count[count];
    const int zsum = count * a.input_zp;
    int q[VEC];
#pragma unroll
    for (int j = 0; j < VEC; j++) {
      const int r = ((__mulhi((acc[j] - zsum) * 8, k.x) + k.y) >> k.z) + a.output_zp;
      q[j] = max(-128, min(127, r));
    }
    if (VEC == 16)
      *reinterpret_cast<uint4*>(a.out + (size_t)p * a.C + g * 16) =
          make_uint4(pack4(q[0], q[1], q[2], q[3]), pack4(q[4], q[5], q[6], q[7]), pack4(q[8], q[9], q[10], q[11]),
                     pack4(q[12], q[13], q[14], q[15]));
    else if (VEC == 4) *reinterpret_cast<uint32_t*>(a.out + (size_t)p * a.C + g * 4) = pack4(q[0], q[1], q[2], q[3]);
    else a.out[(size_t)p * a.C + g] = (int8_t)q[0];
  }
}

// Large windows over few outputs (the global pool at the end of a classifier: 7x7 -> 1x1): a warp per output pixel
// and group of 16 channels, the taps spread over the lanes, sums combined by shuffles. Same arithmetic as above.
__global__ void __launch_bounds__(kThreads) avgpool_warp_kernel(PoolArgs a) {
  grid_dependency_release();
  grid_dependency_wait();
  __shared__ int4 by_count[kAvgMaxTaps + 1];
  for (int c = threadIdx.x; c <= a.KH * a.KW; c += blockDim.x) {
    int32_t mult, shift;
    reciprocal_scale(c ? (uint32_t)c : 1u, mult, shift);
    by_count[c] = make_int4(mult, 1 << (shift - 30), shift - 29, c);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int groups = a.C / 16;
  const long long total = (long long)a.N * a.OH * a.OW * groups;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int taps = a.KH * a.KW;
  for (long long idx = warp0; idx < total; idx += nwarps) {
    const int g = (int)(idx % groups);
    const long long p = idx / groups;
    const int ow = (int)(p % a.OW);
    const long long t = p / a.OW;
    const int oh = (int)(t % a.OH);
    const int n = (int)(t / a.OH);
    const int8_t* xin = a.x + (size_t)n * a.H * a.W * a.C + g * 16;
    int acc[16];
#pragma unroll
    for (int j = 0; j < 16; j++) acc[j] = 0;
    int count = 0;
    for (int tap = lane; tap < taps; tap += 32) {
      const int kh = tap / a.KW, kw = tap - kh * a.KW;
      const int ih = oh * a.stride_h - a.pad_t + kh, iw = ow * a.stride_w - a.pad_l + kw;
      if (ih < 0 || ih >= a.H || iw < 0 || iw >= a.W) continue;
      count++;
      const uint4 v = *reinterpret_cast<const uint4*>(xin + ((size_t)ih * a.W + iw) * a.C);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 16; j++) acc[j] = __dp4a((int)w[j >> 2], 1 << (8 * (j & 3)), acc[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      count += __shfl_xor_sync(0xffffffffu, count, o);
#pragma unroll
      for (int j = 0; j < 16; j++) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
    }
    if (lane == 0) {
      const int4 k = by_count[count];
      const int zsum = count * a.input_zp;
      int q[16];
#pragma unroll
      for (int j = 0; j < 16; j++) {
        const int r = ((__mulhi((acc[j] - zsum) * 8, k.x) + k.y) >> k.z) + a.output_zp;
        q[j] = max(-128, min(127, r));
      }
      *reinterpret_cast<uint4*>(a.out + (size_t)p * a.C + g * 16) =
          make_uint4(pack4(q[0], q[1], q[2], q[3]), pack4(q[4], q[5], q[6], q[7]), pack4(q[8], q[9], q[10], q[11]),
                     pack4(q[12], q[13], q[14], q[15]));
    }
  }
}

// ---- add / sub / mul in TOSA form (ElementWiseBinaryPattern.cpp:385-570, MulPattern.cpp:229-238) ----
// An int8 operand takes 256 values, so its input-side rescale is a 256-entry table (filled here by the
// same apply_scale_32, one entry per thread): per element two shared-memory loads replace two 64-bit
// multiply-shift sequences; the output rescale stays arithmetic.
// EPI: the output rescale, 0 = 64-bit arithmetic, 1 / 2 = the compact 32-bit record (common.cuh) with / without the sign
// term, chosen by the planner when it can bound |operand sum or product| (it evaluates the same two tables).
template <int EPI>
__global__ void __launch_bounds__(kThreads) binary_kernel(BinaryArgs a) {
  grid_dependency_release();
  grid_dependency_wait();
  __shared__ int ta[256], tb[256];  // indexed by the raw byte
  {
    const bool dr = a.double_round != 0;
    const int v = (int)(int8_t)threadIdx.x;
    ta[threadIdx.x] = apply_scale_32((v - a.a_zp) * (1 << a.a_lshift), a.a_mult, a.a_shift, dr);
    tb[threadIdx.x] = apply_scale_32((v - a.b_zp) * (1 << a.b_lshift), a.b_mult, a.b_shift, dr);
  }
  __syncthreads();
  const bool dr = a.double_round != 0;
  auto one = [&](uint32_t xa, uint32_t xb) {
    const int ra = ta[xa], rb = tb[xb];
    const int v = a.kind == 0 ? ra + rb : a.kind == 1 ? ra - rb : ra * rb;
    if (EPI == 0) return requant(v, a.out_mult, a.out_shift, dr, a.out_zp, a.clamp_min, a.clamp_max);
    const int r = EPI == 1 ? scale_q4_sign(v, a.q4) : scale_q4(v, a.q4);  // the output zero point rides in the record
    return max(a.clamp_min, min(a.clamp_max, r));
  };
  const long long nvec = a.n >> 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (long long i = tid; i < nvec; i += stride) {
    uint4 va = reinterpret_cast<const uint4*>(a.a)[i];
    uint4 vb = reinterpret_cast<const uint4*>(a.b)[i];
    uint32_t wa[4] = {va.x, va.y, va.z, va.w};
    uint32_t wb[4] = {vb.x, vb.y, vb.z, vb.w};
    uint32_t wo[4];
#pragma unroll
    for (int w = 0; w < 4; w++) {
      int q[4];
#pragma unroll
      for (int j = 0; j < 4; j++) q[j] = one((wa[w] >> (8 * j)) & 0xff, (wb[w] >> (8 * j)) & 0xff);
      wo[w] = pack4(q[0], q[1], q[2], q[3]);
    }
    reinterpret_cast<uint4*>(a.out)[i] = make_uint4(wo[0], wo[1], wo[2], wo[3]);
  }
  for (long long i = (nvec << 4) + tid; i < a.n; i += stride)
    a.out[i] = (int8_t)one((uint8_t)a.a[i], (uint8_t)a.b[i]);
}

// ---- table: out = table[x + 128] (ExtractPattern.cpp:97-135) ----
__global__ void __launch_bounds__(kThreads) table_kernel(const int8_t* __restrict__ x,
                                                         const int8_t* __restrict__ table,
                                                         int8_t* __restrict__ out, long long n) {
  grid_dependency_release();
  grid_dependency_wait();
  __shared__ uint8_t lut[256];
  // index by the raw byte: entry for byte b is table[(int8)b + 128]
  lut[threadIdx.x] = (uint8_t)table[(int)(int8_t)threadIdx.x + 128];
  __syncthreads();
  const long long nvec = n >> 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (long long i = tid; i < nvec; i += stride) {
    uint4 v = reinterpret_cast<const uint4*>(x)[i];
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; k++) {
      uint32_t r = 0;
#pragma unroll
      for (int j = 0; j < 4; j++) r |= (uint32_t)lut[(w[k] >> (8 * j)) & 0xff] << (8 * j);
      w[k] = r;
    }
    reinterpret_cast<uint4*>(out)[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  for (long long i = (nvec << 4) + tid; i < n; i += stride) out[i] = (int8_t)lut[(uint8_t)x[i]];
}

// ---- standalone rescale i8 -> i8 (PatternUtils.cpp:426-435,3441-3451) ----
__global__ void __launch_bounds__(kThreads) rescale_kernel(RescaleArgs a) {
  grid_dependency_release();
  grid_dependency_wait();
  const long long total = a.rows * a.C;
  const bool dr = a.double_round != 0;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    int c = (int)(idx % a.C);
    long long r = idx / a.C;
    ChanParams cp = a.chan[a.per_channel ? c : 0];
    int v = (int)a.x[idx] - a.input_zp;
    a.out[(size_t)r * a.out_row_stride + a.out_col_offset + c] =
        (int8_t)requant(v, cp.mult, cp.shift, dr, a.out_zp, a.clamp_min, a.clamp_max);
  }
}

// 16 channels per thread when the rows allow 16-byte accesses; IDENT: the rescale is a pass-through
// (multiplier 2^30, shift 30, equal zero points, full clamp range), i.e. a strided copy
template <bool IDENT>
__global__ void __launch_bounds__(kThreads) rescale_vec16_kernel(RescaleArgs a) {
  grid_dependency_release();
  grid_dependency_wait();
  const int cv = a.C >> 4;
  const long long total = a.rows * cv;
  const bool dr = a.double_round != 0;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c16 = (int)(idx % cv);
    const long long r = idx / cv;
    uint4 v = __ldg(reinterpret_cast<const uint4*>(a.x + (size_t)r * a.C) + c16);
    if (!IDENT) {
      uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; q++) {
        int o[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const ChanParams cp = a.chan[a.per_channel ? c16 * 16 + q * 4 + j : 0];
          o[j] = requant(sx8(w[q], j) - a.input_zp, cp.mult, cp.shift, dr, a.out_zp, a.clamp_min, a.clamp_max);
        }
        w[q] = pack4(o[0], o[1], o[2], o[3]);
      }
      v = make_uint4(w[0], w[1], w[2], w[3]);
    }
    *reinterpret_cast<uint4*>(a.out + (size_t)r * a.out_row_stride + a.out_col_offset + c16 * 16) = v;
  }
}

// Per-tensor constants: the rescale is a function of the input byte alone, so it runs as a 256-entry table
// in shared memory (one entry per thread, filled by the same requant), 16 channels per thread.
__global__ void __launch_bounds__(kThreads) rescale_lut_vec16_kernel(RescaleArgs a) {
  grid_dependency_release();
  grid_dependency_wait();
  __shared__ uint8_t lut[256];  // indexed by the raw byte
  {
    const ChanParams cp = a.chan[0];
    lut[threadIdx.x] = (uint8_t)requant((int)(int8_t)threadIdx.x - a.input_zp, cp.mult, cp.shift, a.double_round != 0,
                                        a.out_zp, a.clamp_min, a.clamp_max);
  }
  __syncthreads();
  const int cv = a.C >> 4;
  const long long total = a.rows * cv;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c16 = (int)(idx % cv);
    const long long r = idx / cv;
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(a.x + (size_t)r * a.C) + c16);
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; k++) {
      uint32_t o = 0;
#pragma unroll
      for (int j = 0; j < 4; j++) o |= (uint32_t)lut[(w[k] >> (8 * j)) & 0xff] << (8 * j);
      w[k] = o;
    }
    *reinterpret_cast<uint4*>(a.out + (size_t)r * a.out_row_stride + a.out_col_offset + c16 * 16) =
        make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// ---- nearest 2x (PatternUtils.cpp:489-491): out[y,x] = in[y/2, x/2] ----
__global__ void __launch_bounds__(kThreads) resize_nn2x_vec16_kernel(const int8_t* __restrict__ x, int8_t* __restrict__ out,
                                                                     int N, int H, int W, int C) {
  grid_dependency_release();
  grid_dependency_wait();
  const int cv = C >> 4;
  const long long total = (long long)N * 2 * H * 2 * W * cv;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c16 = (int)(idx % cv);
    long long p = idx / cv;
    const int ow = (int)(p % (2 * W));
    long long t = p / (2 * W);
    const int oh = (int)(t % (2 * H));
    const int n = (int)(t / (2 * H));
    reinterpret_cast<uint4*>(out)[idx] =
        __ldg(reinterpret_cast<const uint4*>(x + (((size_t)n * H + (oh >> 1)) * W + (ow >> 1)) * C) + c16);
  }
}

__global__ void __launch_bounds__(kThreads) resize_nn2x_kernel(const int8_t* __restrict__ x,
                                                               int8_t* __restrict__ out, int N, int H,
                                                               int W, int C) {
  const long long total = (long long)N * 2 * H * 2 * W * C;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    int c = (int)(idx % C);
    long long p = idx / C;
    int ow = (int)(p % (2 * W));
    long long t = p / (2 * W);
    int oh = (int)(t % (2 * H));
    int n = (int)(t / (2 * H));
    out[idx] = x[(((size_t)n * H + (oh >> 1)) * W + (ow >> 1)) * C + c];
  }
}

}  // namespace

void launch_maxpool(const PoolArgs& a, cudaStream_t stream) {
  if (a.elem16) {
    if ((a.C & 7) == 0) maxpool_i16_kernel<8><<<grid_for((long long)a.N * a.OH * a.OW * (a.C / 8)), kThreads, 0, stream>>>(a);
    else maxpool_i16_kernel<1><<<grid_for((long long)a.N * a.OH * a.OW * a.C), kThreads, 0, stream>>>(a);
    return;
  }
  if ((a.C & 15) == 0) {
    long long total = (long long)a.N * a.OH * a.OW * (a.C / 16);
    launch_dependent(maxpool_kernel<16>, dim3(grid_for(total)), dim3(kThreads), 0, stream, a);
  } else {
    long long total = (long long)a.N * a.OH * a.OW * a.C;
    launch_dependent(maxpool_kernel<1>, dim3(grid_for(total)), dim3(kThreads), 0, stream, a);
  }
}

void launch_avgpool(const PoolArgs& a, cudaStream_t stream) {
  if ((a.C & 15) == 0 && ((uintptr_t)a.x & 15) == 0 && ((uintptr_t)a.out & 15) == 0) {
    long long total = (long long)a.N * a.OH * a.OW * (a.C / 16);
    // few outputs with many taps each: spread the taps over a warp
    if (a.KH * a.KW >= 16 && total < 148ll * 2048) launch_dependent(avgpool_warp_kernel, dim3(grid_for(total * 32)), dim3(kThreads), 0, stream, a);
    else launch_dependent(avgpool_kernel<16>, dim3(grid_for(total)), dim3(kThreads), 0, stream, a);
  } else if ((a.C & 3) == 0) {
    long long total = (long long)a.N * a.OH * a.OW * (a.C / 4);
    launch_dependent(avgpool_kernel<4>, dim3(grid_for(total)), dim3(kThreads), 0, stream, a);
  } else {
    long long total = (long long)a.N * a.OH * a.OW * a.C;
    launch_dependent(avgpool_kernel<1>, dim3(grid_for(total)), dim3(kThreads), 0, stream, a);
  }
}

void launch_binary(const BinaryArgs& a, cudaStream_t stream) {
  if (a.epi == 1) launch_dependent(binary_kernel<1>, dim3(grid_for((a.n + 15) / 16)), dim3(kThreads), 0, stream, a);
  else if (a.epi == 2) launch_dependent(binary_kernel<2>, dim3(grid_for((a.n + 15) / 16)), dim3(kThreads), 0, stream, a);
  else launch_dependent(binary_kernel<0>, dim3(grid_for((a.n + 15) / 16)), dim3(kThreads), 0, stream, a);
}

void launch_table(const int8_t* x, const int8_t* table, int8_t* out, long long n, cudaStream_t stream) {
  launch_dependent(table_kernel, dim3(grid_for((n + 15) / 16)), dim3(kThreads), 0, stream, x, table, out, n);
}

void launch_rescale(const RescaleArgs& a, cudaStream_t stream) {
  const bool vec = (a.C & 15) == 0 && (a.out_row_stride & 15) == 0 && (a.out_col_offset & 15) == 0 &&
                   ((uintptr_t)a.x & 15) == 0 && ((uintptr_t)a.out & 15) == 0;
  if (vec && a.identity) launch_dependent(rescale_vec16_kernel<true>, dim3(grid_for(a.rows * (a.C >> 4))), dim3(kThreads), 0, stream, a);
  else if (vec && !a.per_channel) launch_dependent(rescale_lut_vec16_kernel, dim3(grid_for(a.rows * (a.C >> 4))), dim3(kThreads), 0, stream, a);
  else if (vec) launch_dependent(rescale_vec16_kernel<false>, dim3(grid_for(a.rows * (a.C >> 4))), dim3(kThreads), 0, stream, a);
  else launch_dependent(rescale_kernel, dim3(grid_for(a.rows * a.C)), dim3(kThreads), 0, stream, a);
}

void launch_resize_nn2x(const int8_t* x, int8_t* out, int N, int H, int W, int C, cudaStream_t stream) {
  if ((C & 15) == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    launch_dependent(resize_nn2x_vec16_kernel, dim3(grid_for((long long)N * 4 * H * W * (C >> 4))), dim3(kThreads), 0, stream, x, out, N, H, W, C);
    return;
  }
  resize_nn2x_kernel<<<grid_for((long long)N * 4 * H * W * C), kThreads, 0, stream>>>(x, out, N, H, W, C);
}

}  // namespace tb200
