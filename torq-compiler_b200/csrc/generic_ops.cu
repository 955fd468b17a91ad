// Tensor ops outside the layer set (TB200_OP_EW, the generic tosa.rescale, TRANSPOSE / SLICE / PAD /
// CONCAT_AXIS / PERMUTE, REDUCE, TABLE16, SOFTMAX, GATHER / SCATTER): what the reference's op fixtures exercise
// around the layers (tests/testdata/tosa_ops: cast-*, Elementwise_*, rescale-*, transpose-*, d2s_*, pad_*, reduce-*,
// argmax-*, gather*, scatter*, mbv2-softmax-i8).
// All are bandwidth-bound index arithmetic on dense row-major tensors of rank <= 4 with element types
// i8 / i16 / i32 / f32 / bf16. Integers are computed in int32 with wrap-around and truncated to the result
// type; floats in fp32, rounded once to nearest even; float -> int casts round to nearest even and saturate.
#include <cuda_bf16.h>

#include "../../include/torq_b200_ops.h"
#include "kernels.h"

namespace tb200 {

namespace {

__device__ __forceinline__ bool is_float_dtype(int d) { return d == TB200_F32 || d == TB200_BF16; }

__device__ __forceinline__ int load_int(const void* p, int dtype, long long i) {
  switch (dtype) {
    case TB200_I8: return ((const int8_t*)p)[i];
    case TB200_I16: return ((const int16_t*)p)[i];
    default: return ((const int32_t*)p)[i];
  }
}
__device__ __forceinline__ float load_float(const void* p, int dtype, long long i) {
  switch (dtype) {
    case TB200_F32: return ((const float*)p)[i];
    case TB200_BF16: return __uint_as_float((uint32_t)((const uint16_t*)p)[i] << 16);
    default: return (float)load_int(p, dtype, i);
  }
}
__device__ __forceinline__ void store_int(void* p, int dtype, long long i, int v) {
  switch (dtype) {
    case TB200_I8: ((int8_t*)p)[i] = (int8_t)v; break;
    case TB200_I16: ((int16_t*)p)[i] = (int16_t)v; break;
    case TB200_I32: ((int32_t*)p)[i] = v; break;
    case TB200_F32: ((float*)p)[i] = (float)v; break;
    default: ((uint16_t*)p)[i] = __bfloat16_as_ushort(__float2bfloat16_rn((float)v)); break;
  }
}
__device__ __forceinline__ void store_float(void* p, int dtype, long long i, float v) {
  switch (dtype) {
    case TB200_F32: ((float*)p)[i] = v; break;
    case TB200_BF16: ((uint16_t*)p)[i] = __bfloat16_as_ushort(__float2bfloat16_rn(v)); break;
    default: {  // float -> int: nearest even, saturating, NaN -> 0
      const int bits = dtype == TB200_I8 ? 8 : dtype == TB200_I16 ? 16 : 32;
      const float lo = -ldexpf(1.0f, bits - 1), hi = ldexpf(1.0f, bits - 1);
      int r;
      if (v != v) r = 0;
      else if (v <= lo) r = bits == 32 ? INT32_MIN : -(1 << (bits - 1));
      else if (v >= hi) r = bits == 32 ? INT32_MAX : (1 << (bits - 1)) - 1;
      else r = __float2int_rn(v);
      if (bits < 32) r = max(-(1 << (bits - 1)), min((1 << (bits - 1)) - 1, r));
      store_int(p, dtype, i, r);
    }
  }
}

__global__ void __launch_bounds__(256) ew_kernel(EwArgs a) {
  const bool flt = is_float_dtype(a.a_dtype) || (a.b && is_float_dtype(a.b_dtype));
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += stride) {
    long long ia = i, ib = i;
    if (!a.contiguous) {  // broadcast: operand offsets from the output coordinates
      long long r = i;
      ia = ib = 0;
#pragma unroll
      for (int d = 3; d >= 0; d--) {
        const int c = (int)(r % a.dims[d]);
        r /= a.dims[d];
        ia += (long long)c * a.a_str[d];
        ib += (long long)c * a.b_str[d];
      }
    }
    if (flt) {
      const float x = load_float(a.a, a.a_dtype, ia);
      const float y = a.b ? load_float(a.b, a.b_dtype, ib) : 0.f;
      float r = 0.f;
      int cmp = -1;
      switch (a.fn) {
        case TB200_EW_CAST: r = x; if (a.bool_result) cmp = x != 0.f; break;
        case TB200_EW_ABS: r = fabsf(x); break;
        case TB200_EW_NEGATE: r = -x; break;
        case TB200_EW_CLAMP: r = fminf(fmaxf(x, a.fmin), a.fmax); break;
        case TB200_EW_CEIL: r = ceilf(x); break;
        case TB200_EW_FLOOR: r = floorf(x); break;
        case TB200_EW_EXP: r = expf(x); break;
        case TB200_EW_LOG: r = logf(x); break;
        case TB200_EW_RECIPROCAL: r = 1.0f / x; break;
        case TB200_EW_RSQRT: r = 1.0f / sqrtf(x); break;
        case TB200_EW_TANH: r = tanhf(x); break;
        case TB200_EW_SIGMOID: r = 1.0f / (1.0f + expf(-x)); break;
        case TB200_EW_ERF: r = erff(x); break;
        case TB200_EW_ADD: r = x + y; break;
        case TB200_EW_SUB: r = x - y; break;
        case TB200_EW_MUL: r = x * y; break;
        case TB200_EW_MAX: r = fmaxf(x, y); break;
        case TB200_EW_MIN: r = fminf(x, y); break;
        case TB200_EW_EQ: cmp = x == y; break;
        case TB200_EW_GT: cmp = x > y; break;
        case TB200_EW_GE: cmp = x >= y; break;
        default: break;
      }
      if (cmp >= 0) store_int(a.out, a.out_dtype, i, cmp);
      else store_float(a.out, a.out_dtype, i, r);
    } else {
      const int x = load_int(a.a, a.a_dtype, ia);
      const int y = a.b ? load_int(a.b, a.b_dtype, ib) : 0;
      int r = 0;
      switch (a.fn) {
        case TB200_EW_CAST: r = a.bool_result ? (x != 0) : x; break;
        case TB200_EW_ABS: r = x < 0 ? (int)(0u - (uint32_t)x) : x; break;
        case TB200_EW_NEGATE: r = (int)((uint32_t)a.out_zp - ((uint32_t)x - (uint32_t)a.in_zp)); break;
        case TB200_EW_BITWISE_NOT: r = ~x; break;
        case TB200_EW_LOGICAL_NOT: r = x == 0; break;
        case TB200_EW_CLZ: r = __clz(x); break;
        case TB200_EW_CLAMP: r = max(a.clamp_min, min(a.clamp_max, x)); break;
        case TB200_EW_ADD: r = (int)((uint32_t)x + (uint32_t)y); break;
        case TB200_EW_SUB: r = (int)((uint32_t)x - (uint32_t)y); break;
        case TB200_EW_MUL:
          if (a.arg > 0) r = (int)(((long long)x * y + (1ll << (a.arg - 1))) >> a.arg);
          else r = (int)((uint32_t)x * (uint32_t)y);
          break;
        case TB200_EW_MAX: r = max(x, y); break;
        case TB200_EW_MIN: r = min(x, y); break;
        case TB200_EW_AND: r = x & y; break;
        case TB200_EW_OR: r = x | y; break;
        case TB200_EW_XOR: r = x ^ y; break;
        case TB200_EW_LSL: r = (int)((uint32_t)x << (y & 31)); break;
        case TB200_EW_ASR: {
          const int s = y & 31;
          r = x >> s;
          if (a.arg && s > 0) r += (x >> (s - 1)) & 1;
          break;
        }
        case TB200_EW_EQ: r = x == y; break;
        case TB200_EW_GT: r = x > y; break;
        case TB200_EW_GE: r = x >= y; break;
        case TB200_EW_LOGICAL_AND: r = (x != 0) && (y != 0); break;
        case TB200_EW_LOGICAL_OR: r = (x != 0) || (y != 0); break;
        case TB200_EW_LOGICAL_XOR: r = (x != 0) != (y != 0); break;
        default: break;
      }
      store_int(a.out, a.out_dtype, i, r);
    }
  }
}

// tosa.rescale between integer types (scale32): v = in - in_zp (int32, wrapping), apply_scale_32, + out_zp, clamp.
__global__ void __launch_bounds__(256) rescale_generic_kernel(RescaleGenericArgs a) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += stride) {
    int x = load_int(a.x, a.in_dtype, i);
    if (a.input_unsigned) x &= a.in_dtype == TB200_I8 ? 0xff : a.in_dtype == TB200_I16 ? 0xffff : -1;
    const int v = (int)((uint32_t)x - (uint32_t)a.in_zp);
    const int c = a.per_channel ? (int)(i % a.C) : 0;
    const int m = a.mult[c], s = a.shift[c];
    long long rnd = 1ll << (s - 1);
    if (a.double_round && s > 31) rnd += v >= 0 ? (1ll << 30) : -(1ll << 30);
    const int r = (int)(((long long)v * m + rnd) >> s);
    const long long q = (long long)r + a.out_zp;
    const long long clamped = q < a.clamp_min ? a.clamp_min : q > a.clamp_max ? a.clamp_max : q;
    store_int(a.out, a.out_dtype, i, (int)clamped);
  }
}

// one piece of padding: the element's value repeated over the piece
template <typename T>
__device__ __forceinline__ T pad_piece(int value, int elem_bytes);
template <> __device__ __forceinline__ uint8_t pad_piece<uint8_t>(int value, int) { return (uint8_t)value; }
template <> __device__ __forceinline__ uint16_t pad_piece<uint16_t>(int value, int) { return (uint16_t)value; }
__device__ __forceinline__ uint32_t pad_word(int value, int elem_bytes) {
  return elem_bytes == 1 ? (uint32_t)(value & 0xff) * 0x01010101u
         : elem_bytes == 2 ? (uint32_t)(value & 0xffff) * 0x00010001u
                           : (uint32_t)value;
}
template <> __device__ __forceinline__ uint32_t pad_piece<uint32_t>(int value, int eb) { return pad_word(value, eb); }
template <> __device__ __forceinline__ uint2 pad_piece<uint2>(int value, int eb) {
  const uint32_t w = pad_word(value, eb);
  return make_uint2(w, w);
}
template <> __device__ __forceinline__ uint4 pad_piece<uint4>(int value, int eb) {
  const uint32_t w = pad_word(value, eb);
  return make_uint4(w, w, w, w);
}

// out[o] = in[in_offset + sum (o_d - lo_d) * in_str_d] when every (o_d - lo_d) lies in [0, in_dims_d), else the pad
// value; the output element sits at out_offset + sum o_d * out_str_d. One kernel for transpose, slice, pad and concat.
// ND = dimensions walked (4 when the two leading slots are 1: the common case keeps its shorter index arithmetic)
template <typename T, int ND>
__global__ void __launch_bounds__(256) strided_copy_kernel(StridedCopyArgs a) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const T* src = (const T*)a.in;
  T* dst = (T*)a.out;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += stride) {
    long long r = i, si = a.in_offset, di = a.out_offset;
    bool inside = true;
#pragma unroll
    for (int d = 5; d >= 6 - ND; d--) {
      const int c = (int)(r % a.dims[d]);
      r /= a.dims[d];
      const int ci = c - a.lo[d];
      inside = inside && ci >= 0 && ci < a.in_dims[d];
      si += (long long)ci * a.in_str[d];
      di += (long long)c * a.out_str[d];
    }
    dst[di] = inside ? src[si] : pad_piece<T>(a.pad_value, a.pad_elem_bytes);
  }
}

// x viewed as [outer, axis, inner]; one thread per (outer, inner).
__global__ void __launch_bounds__(256) reduce_kernel(ReduceArgs a) {
  const long long total = (long long)a.outer * a.inner;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long o = i / a.inner, in = i - o * a.inner;
  const long long base = o * a.axis * a.inner + in;
  if (is_float_dtype(a.in_dtype)) {
    float best = load_float(a.x, a.in_dtype, base);
    int arg = 0;
    for (int k = 1; k < a.axis; k++) {
      const float v = load_float(a.x, a.in_dtype, base + (long long)k * a.inner);
      if (a.fn == 2 ? v < best : v > best) { best = v; arg = k; }
    }
    if (a.fn == 0 || a.fn == 4) {  // fp32 sum in index order; mean = sum / count
      float sum = 0.f;
      for (int k = 0; k < a.axis; k++) sum = sum + load_float(a.x, a.in_dtype, base + (long long)k * a.inner);
      store_float(a.out, a.out_dtype, i, a.fn == 4 ? sum / (float)a.axis : sum);
    } else if (a.fn == 3) store_int(a.out, a.out_dtype, i, arg);
    else store_float(a.out, a.out_dtype, i, best);
  } else {
    int best = load_int(a.x, a.in_dtype, base), arg = 0;
    uint32_t sum = (uint32_t)best;
    for (int k = 1; k < a.axis; k++) {
      const int v = load_int(a.x, a.in_dtype, base + (long long)k * a.inner);
      sum += (uint32_t)v;
      if (a.fn == 2 ? v < best : v > best) { best = v; arg = k; }
    }
    store_int(a.out, a.out_dtype, i, a.fn == 0 ? (int)sum : a.fn == 3 ? arg : best);
  }
}

__global__ void __launch_bounds__(256) table16_kernel(const int16_t* __restrict__ x, const int16_t* __restrict__ table,
                                                      int32_t* __restrict__ out, long long n) {
  __shared__ int16_t t[513];
  for (int i = threadIdx.x; i < 513; i += blockDim.x) t[i] = table[i];
  __syncthreads();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int v = x[i];
    const int index = (v + 32768) >> 7, frac = v & 0x7f;
    const int base = t[index], next = t[index + 1];
    out[i] = base * 128 + (next - base) * frac;
  }
}

// One warp per row: maximum, exp and sum in fp32, then one multiplication by the reciprocal of the sum.
__global__ void __launch_bounds__(256) softmax_kernel(const void* __restrict__ x, void* __restrict__ out, long long rows, int cols,
                                                      int dtype) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const long long base = row * cols;
  float m = -INFINITY;
  for (int c = lane; c < cols; c += 32) m = fmaxf(m, load_float(x, dtype, base + c));
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float sum = 0.f;
  for (int c = lane; c < cols; c += 32) sum += expf(load_float(x, dtype, base + c) - m);
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.0f / sum;
  for (int c = lane; c < cols; c += 32) store_float(out, dtype, base + c, expf(load_float(x, dtype, base + c) - m) * inv);
}

unsigned grid_for(long long n) {
  const long long blocks = (n + 255) / 256;
  const long long cap = (long long)current_sm_count() * 16;
  return (unsigned)(blocks < 1 ? 1 : blocks < cap ? blocks : cap);
}

}  // namespace

void launch_ew(const EwArgs& a, cudaStream_t stream) { ew_kernel<<<grid_for(a.n), 256, 0, stream>>>(a); }
void launch_rescale_generic(const RescaleGenericArgs& a, cudaStream_t stream) {
  rescale_generic_kernel<<<grid_for(a.n), 256, 0, stream>>>(a);
}
void launch_strided_copy(const StridedCopyArgs& a, cudaStream_t stream) {
  const bool six = a.dims[0] != 1 || a.dims[1] != 1;
#define TB200_COPY(T)                                                                  \
  do {                                                                                 \
    if (six) strided_copy_kernel<T, 6><<<grid_for(a.n), 256, 0, stream>>>(a);          \
    else strided_copy_kernel<T, 4><<<grid_for(a.n), 256, 0, stream>>>(a);              \
  } while (0)
  if (a.elem_bytes == 1) TB200_COPY(uint8_t);
  else if (a.elem_bytes == 2) TB200_COPY(uint16_t);
  else if (a.elem_bytes == 4) TB200_COPY(uint32_t);
  else if (a.elem_bytes == 8) TB200_COPY(uint2);
  else TB200_COPY(uint4);
#undef TB200_COPY
}
void widen_strided_copy(StridedCopyArgs& a) {
  if (a.in_str[5] != 1 || a.out_str[5] != 1) return;
  for (int bytes = 16; bytes > a.elem_bytes; bytes >>= 1) {
    const int v = bytes / a.elem_bytes;
    bool fits = a.dims[5] % v == 0 && a.lo[5] % v == 0 && (a.in_dims[5] == (1 << 30) || a.in_dims[5] % v == 0) &&
                a.in_offset % v == 0 && a.out_offset % v == 0;
    for (int d = 0; d < 5 && fits; d++) fits = a.in_str[d] % v == 0 && a.out_str[d] % v == 0;
    if (!fits) continue;
    a.dims[5] /= v;
    a.lo[5] /= v;
    if (a.in_dims[5] != (1 << 30)) a.in_dims[5] /= v;
    for (int d = 0; d < 5; d++) {
      a.in_str[d] /= v;
      a.out_str[d] /= v;
    }
    a.in_offset /= v;
    a.out_offset /= v;
    a.n /= v;
    a.elem_bytes = bytes;
    return;
  }
}
namespace {
// one thread per byte of the W rows; rows are short (a few channels), so byte granularity keeps every type and alignment
template <bool SCATTER>
__global__ void __launch_bounds__(256) rows_by_index_kernel(const uint8_t* __restrict__ src, const int32_t* __restrict__ idx,
                                                            uint8_t* __restrict__ out, int N, int K, int W, int row_bytes) {
  const long long total = (long long)N * W * row_bytes;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % row_bytes);
    const long long nw = i / row_bytes;
    const int n = (int)(nw / W);
    const int k = __ldg(idx + nw);
    const bool inside = k >= 0 && k < K;
    if (SCATTER) {
      if (inside) out[((long long)n * K + k) * row_bytes + c] = src[i];
    } else {
      out[i] = inside ? src[((long long)n * K + k) * row_bytes + c] : (uint8_t)0;
    }
  }
}
}  // namespace

namespace {
// tosa.matmul on floats: one thread per output, products and sums rounded separately (no fused multiply-add), k in order
__global__ void __launch_bounds__(256) matmul_f_kernel(const void* __restrict__ a, const void* __restrict__ b, void* __restrict__ out,
                                                       int M, int K, int N, int in_dtype, int out_dtype) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)M * N) return;
  const int n = (int)(idx % N), m = (int)(idx / N);
  float acc = 0.f;
  for (int k = 0; k < K; k++)
    acc = __fadd_rn(acc, __fmul_rn(load_float(a, in_dtype, (long long)m * K + k), load_float(b, in_dtype, (long long)k * N + n)));
  store_float(out, out_dtype, idx, acc);
}
}  // namespace

namespace {
// tosa.depthwise_conv2d on floats: one thread per output; products and sums rounded separately, taps in (kh, kw) order,
// taps outside the frame skipped, the bias added last
__global__ void __launch_bounds__(256) depthwise_f_kernel(DepthwiseFArgs a) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)a.N * a.OH * a.OW * a.C * a.M;
  if (idx >= total) return;
  const int CM = a.C * a.M;
  const int cm = (int)(idx % CM);
  long long t = idx / CM;
  const int ow = (int)(t % a.OW); t /= a.OW;
  const int oh = (int)(t % a.OH);
  const int n = (int)(t / a.OH);
  const int c = cm / a.M, m = cm - c * a.M;
  float acc = 0.f;
  for (int kh = 0; kh < a.KH; kh++) {
    const int ih = oh * a.stride_h - a.pad_t + kh * a.dil_h;
    if (ih < 0 || ih >= a.H) continue;
    for (int kw = 0; kw < a.KW; kw++) {
      const int iw = ow * a.stride_w - a.pad_l + kw * a.dil_w;
      if (iw < 0 || iw >= a.W) continue;
      const float xv = load_float(a.x, a.dtype, (((long long)n * a.H + ih) * a.W + iw) * a.C + c);
      const float wv = load_float(a.w, a.dtype, (((long long)kh * a.KW + kw) * a.C + c) * a.M + m);
      acc = __fadd_rn(acc, __fmul_rn(xv, wv));
    }
  }
  store_float(a.out, a.dtype, idx, __fadd_rn(acc, load_float(a.bias, a.dtype, cm)));
}
}  // namespace

void launch_depthwise_f(const DepthwiseFArgs& a, cudaStream_t stream) {
  const long long total = (long long)a.N * a.OH * a.OW * a.C * a.M;
  depthwise_f_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(a);
}

void launch_matmul_f(const void* a, const void* b, void* out, int M, int K, int N, int in_dtype, int out_dtype, cudaStream_t stream) {
  matmul_f_kernel<<<(unsigned)(((long long)M * N + 255) / 256), 256, 0, stream>>>(a, b, out, M, K, N, in_dtype, out_dtype);
}

void launch_gather_rows(const void* values, const int32_t* idx, void* out, int N, int K, int W, int row_bytes, cudaStream_t stream) {
  rows_by_index_kernel<false><<<grid_for((long long)N * W * row_bytes), 256, 0, stream>>>((const uint8_t*)values, idx, (uint8_t*)out, N, K, W, row_bytes);
}
void launch_scatter_rows(const void* updates, const int32_t* idx, void* out, int N, int K, int W, int row_bytes, cudaStream_t stream) {
  rows_by_index_kernel<true><<<grid_for((long long)N * W * row_bytes), 256, 0, stream>>>((const uint8_t*)updates, idx, (uint8_t*)out, N, K, W, row_bytes);
}
void launch_softmax(const void* x, void* out, long long rows, int cols, int dtype, cudaStream_t stream) {
  softmax_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(x, out, rows, cols, dtype);
}
void launch_table16(const int16_t* x, const int16_t* table, int32_t* out, long long n, cudaStream_t stream) {
  table16_kernel<<<grid_for(n), 256, 0, stream>>>(x, table, out, n);
}
void launch_reduce(const ReduceArgs& a, cudaStream_t stream) {
  const long long total = (long long)a.outer * a.inner;
  reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(a);
}

}  // namespace tb200
