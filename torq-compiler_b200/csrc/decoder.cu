// Decoder-side kernels: bf16 activations, int8 per-output-channel weights with bf16
// scales, fp32 accumulation, bf16 KV cache. They implement the op set the reference
// reaches for an LLM decode step: weight expansion + matmul
// (torq_hl.expand_weights + bf16 torq_hl.matmul, compiler/torq/Dialect/TorqHL/TorqHLOps.td:943-957,
// tests/testdata/torch_ops/matmul_dql_q8_0.mlir; here block = K, zero point 0), the
// RMSNorm pieces (ReduceMeanPattern.cpp:37-466), tanh-GELU (GeluPattern.cpp:35-46), softmax
// over the keys (SoftmaxPattern.cpp:23-333) and the KV cache passed through as tied
// state (tests/testdata/torch_ops/tied_operands_kv_cache.mlir).
//
// Every one of them is bandwidth-bound at decode batch sizes: the design goal is bytes in
// flight (split-K GEMV, split-T attention) and one pass over the weights.
// Rounding points (bf16, round-to-nearest-even) are stated at each kernel; the torch
// reference used by the tests rounds at the same points.
#include <cuda_bf16.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "kernels.h"

namespace tb200 {

namespace {

__device__ __forceinline__ float bf2f(uint16_t v) { return __uint_as_float((uint32_t)v << 16); }
__device__ __forceinline__ uint16_t f2bf(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  return warp_sum(t);
}
// One launch helper for every kernel of this file. (Launching them as programmatic dependents of one
// another - blocks resident early, griddepcontrol.wait before the first memory access - was measured on
// B200 inside the captured graph of a decode step: 4-6 % slower at batches 8 and 32, so it is not used.)
template <typename... KArgs, typename... Args>
void launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  kernel<<<grid, block, smem, stream>>>(KArgs(args)...);
}

// int8 -> float without the conversion pipe: place the biased byte in the mantissa of 2^23
__device__ __forceinline__ float s8_to_float(uint32_t word, int j) {
  const uint32_t b = ((word >> (8 * j)) & 0xffu) ^ 0x80u;
  return __uint_as_float(0x4B000000u | b) - 8388736.0f;  // 2^23 + 128
}

// x[b, :] = bf16( bf16(E[tok[b], :] * scale[tok[b]]) * mult )
__global__ void __launch_bounds__(128) embed_kernel(const int32_t* __restrict__ tok, const int8_t* __restrict__ table,
                                                    const uint16_t* __restrict__ scale, uint16_t* __restrict__ out,
                                                    int H, int V, float mult) {
  const int b = blockIdx.x;
  int t = tok[b];
  t = t < 0 ? 0 : (t >= V ? V - 1 : t);
  const float s = bf2f(scale[t]);
  const int8_t* row = table + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[(size_t)b * H + i] = f2bf(bf2f(f2bf((float)row[i] * s)) * mult);
}

// y = [res +] bf16( x * rsqrt(mean(x^2) + eps) * (1 + w) )   (sum of res and the rounded norm is rounded again)
__global__ void __launch_bounds__(1024) rmsnorm_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ res,
                                                      const uint16_t* __restrict__ w, uint16_t* __restrict__ out,
                                                      int H, float eps) {
  __shared__ float red[32];
  const size_t base = (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = bf2f(x[base + i]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float n = bf2f(f2bf(bf2f(x[base + i]) * inv * (1.0f + bf2f(w[i]))));
    out[base + i] = res ? f2bf(bf2f(res[base + i]) + n) : f2bf(n);
  }
}

// One element of a bf16 [B, N] operand: the tensor itself, or the finalized sum of split-K partials.
__device__ __forceinline__ float operand_at(const uint16_t* __restrict__ x, const GemvPartials& gp, size_t bn, size_t idx,
                                            int n) {
  if (gp.splits == 0) return bf2f(x[idx]);
  float s = 0.f;
#pragma unroll 4
  for (int sp = 0; sp < gp.splits; sp++) s += __ldg(gp.partial + (size_t)sp * bn + idx);
  return bf2f(f2bf(s * bf2f(__ldg(gp.scale + n))));
}

// rmsnorm_kernel, its input optionally split-K partials, and optionally a second norm (no residual) of the
// result in the same launch: out2 = bf16( out * rsqrt(mean(out^2) + eps2) * (1 + w2) ). One block per row,
// the row kept in shared memory as fp32.
__global__ void __launch_bounds__(1024) rmsnorm_fused_kernel(const uint16_t* __restrict__ x, GemvPartials gp,
                                                            const uint16_t* __restrict__ res,
                                                            const uint16_t* __restrict__ w, uint16_t* __restrict__ out,
                                                            const uint16_t* __restrict__ w2, uint16_t* __restrict__ out2,
                                                            int rows, int H, float eps, float eps2) {
  extern __shared__ float row_s[];
  __shared__ float red[32];
  const size_t base = (size_t)blockIdx.x * H;
  const size_t bn = (size_t)rows * H;
  float ss = 0.f;
  if (gp.splits > 0 && H <= 4 * (int)blockDim.x) {
    // up to four elements per thread: slices outermost, so that 4 x 8 loads are in flight together;
    // every element still adds its slices in order
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    const float* p0 = gp.partial + base + threadIdx.x;
#pragma unroll 8
    for (int sp = 0; sp < gp.splits; sp++) {
#pragma unroll
      for (int e = 0; e < 4; e++)
        if ((int)threadIdx.x + e * (int)blockDim.x < H) a[e] += __ldg(p0 + (size_t)sp * bn + e * blockDim.x);
    }
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const int i = threadIdx.x + e * blockDim.x;
      if (i < H) {
        const float v = bf2f(f2bf(a[e] * bf2f(__ldg(gp.scale + i))));
        row_s[i] = v;
        ss += v * v;
      }
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = operand_at(x, gp, bn, base + i, i);
      row_s[i] = v;
      ss += v * v;
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  float ss2 = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float n = bf2f(f2bf(row_s[i] * inv * (1.0f + bf2f(w[i]))));
    const uint16_t o = res ? f2bf(bf2f(res[base + i]) + n) : f2bf(n);
    out[base + i] = o;
    const float ov = bf2f(o);
    row_s[i] = ov;
    ss2 += ov * ov;
  }
  if (!w2) return;
  __syncthreads();  // red is reused
  ss2 = block_sum(ss2, red);
  const float inv2 = rsqrtf(ss2 / (float)H + eps2);
  for (int i = threadIdx.x; i < H; i += blockDim.x) out2[base + i] = f2bf(row_s[i] * inv2 * (1.0f + bf2f(w2[i])));
}

// Split-K GEMV / skinny GEMM with int8 weights: one warp per output row n and K slice.
//   acc[b] = sum_{k in slice} x[b,k] * W[n,k]      (fp32)
// splits == 1: y[b,n] = bf16(acc * scale[n]); otherwise the partial sums go to scratch
// [split][b][n] and gemv_finalize_kernel adds them in split order.
template <int BT>
__global__ void __launch_bounds__(256) gemv_w8_kernel(const uint16_t* __restrict__ x, const int8_t* __restrict__ W,
                                                      const uint16_t* __restrict__ scale, void* __restrict__ y,
                                                      float* __restrict__ partial, int B, int N, int K, int k_slice,
                                                      int y_f32) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const int split = blockIdx.y, splits = gridDim.y;
  const int k_begin = split * k_slice;
  const int k_end = min(K, k_begin + k_slice);
  float acc[BT];
#pragma unroll
  for (int b = 0; b < BT; b++) acc[b] = 0.f;
  const int8_t* wrow = W + (size_t)n * K;
  for (int k = k_begin + lane * 16; k < k_end; k += 32 * 16) {
    const uint4 wv = *reinterpret_cast<const uint4*>(wrow + k);
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
    float wf[16];
#pragma unroll
    for (int j = 0; j < 16; j++) wf[j] = s8_to_float(ww[j >> 2], j & 3);
#pragma unroll
    for (int b = 0; b < BT; b++) {
      if (b < B) {
        const uint4 x0 = __ldg(reinterpret_cast<const uint4*>(x + (size_t)b * K + k));
        const uint4 x1 = __ldg(reinterpret_cast<const uint4*>(x + (size_t)b * K + k + 8));
        const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        float s = acc[b];
#pragma unroll
        for (int j = 0; j < 8; j++) {
          s = fmaf(wf[2 * j], __uint_as_float(xw[j] << 16), s);
          s = fmaf(wf[2 * j + 1], __uint_as_float(xw[j] & 0xffff0000u), s);
        }
        acc[b] = s;
      }
    }
  }
#pragma unroll
  for (int b = 0; b < BT; b++) acc[b] = warp_sum(acc[b]);
  if (lane == 0) {
    const float s = bf2f(scale[n]);
#pragma unroll
    for (int b = 0; b < BT; b++) {
      if (b < B) {
        if (splits == 1) {
          if (y_f32) ((float*)y)[(size_t)b * N + n] = acc[b] * s;
          else ((uint16_t*)y)[(size_t)b * N + n] = f2bf(acc[b] * s);
        } else partial[((size_t)split * B + b) * N + n] = acc[b];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// The same product for larger batches on the tensor cores (mma.sync m16n8k16, bf16 operands,
// fp32 accumulation): with many tokens the CUDA-core kernel above spends one FMA per token and weight
// byte and is FMA-bound at a few percent of the HBM rate. Block = 128 weight rows (8 warps x 16
// rows) x one K slice; the slice of x for all tokens is staged in shared memory once per block
// (bf16, token rows 16 bytes apart modulo 128 so that the fragment loads do not conflict);
// every warp streams its 16 rows straight from global memory, 64 bytes of K at a time, turns
// the int8 weights into bf16 fragments (exact) and issues one MMA per group of 8 tokens.
// The weights are the 16-row operand, the tokens the 8-column operand, as in decode_step.cu.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void s8x4_to_bf16x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t u = w ^ 0x80808080u;  // bytes biased by 128
  const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.0f;  // 2^23 + 128
  const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.0f;
  const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.0f;
  const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.0f;
  lo = __byte_perm(__float_as_uint(f0), __float_as_uint(f1), 0x7632);  // high halves = the bf16 values
  hi = __byte_perm(__float_as_uint(f2), __float_as_uint(f3), 0x7632);
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT>  // groups of 8 tokens
__global__ void __launch_bounds__(256) gemv_w8_mma_kernel(const uint16_t* __restrict__ x, const int8_t* __restrict__ W,
                                                          const uint16_t* __restrict__ scale, void* __restrict__ y,
                                                          float* __restrict__ partial, int B, int N, int K, int k_slice,
                                                          int y_f32) {
  extern __shared__ __align__(16) unsigned char xs_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int split = blockIdx.y, splits = gridDim.y;
  const int k_begin = split * k_slice;
  const int k_len = min(k_slice, K - k_begin);  // a multiple of 64
  const int xstride = ((k_slice * 2 + 127) / 128) * 128 + 16;  // bytes per token row in shared memory
  const int row0 = blockIdx.x * 128 + warp * 16;
  const bool active = row0 < N;
  const int r_lo = row0 + g, r_hi = row0 + g + 8;
  const int8_t* w_lo = W + (size_t)min(r_lo, N - 1) * K + k_begin + tig * 16;
  const int8_t* w_hi = W + (size_t)min(r_hi, N - 1) * K + k_begin + tig * 16;
  const int kbs = k_len >> 6;
  // the first two 64-byte blocks of this lane's weight rows are requested before x is staged, so that
  // their latency overlaps the staging
  uint4 pa[2], pb[2];
#pragma unroll
  for (int p = 0; p < 2; p++) {
    pa[p] = pb[p] = make_uint4(0, 0, 0, 0);
    if (active && p < kbs) {
      pa[p] = __ldg(reinterpret_cast<const uint4*>(w_lo + p * 64));
      pb[p] = __ldg(reinterpret_cast<const uint4*>(w_hi + p * 64));
    }
  }
  // stage x[:, k_begin : k_begin + k_len]; tokens beyond B read as zero
  for (int i = threadIdx.x; i < NT * 8 * (k_len / 8); i += blockDim.x) {
    const int b = i / (k_len / 8), c = i % (k_len / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (b < B) v = __ldg(reinterpret_cast<const uint4*>(x + (size_t)b * K + k_begin) + c);
    *reinterpret_cast<uint4*>(xs_raw + (size_t)b * xstride + 16 * c) = v;
  }
  __syncthreads();
  if (!active) return;
  float c[NT][4];
#pragma unroll
  for (int t = 0; t < NT; t++)
#pragma unroll
    for (int j = 0; j < 4; j++) c[t][j] = 0.f;
  const unsigned char* xrow = xs_raw + (size_t)g * xstride + tig * 32;
  auto block64 = [&](int kb, const uint4& wa, const uint4& wb) {
    uint32_t a[4][4];  // [mma within the block of 64][a0..a3]
    s8x4_to_bf16x4(wa.x, a[0][0], a[0][2]); s8x4_to_bf16x4(wb.x, a[0][1], a[0][3]);
    s8x4_to_bf16x4(wa.y, a[1][0], a[1][2]); s8x4_to_bf16x4(wb.y, a[1][1], a[1][3]);
    s8x4_to_bf16x4(wa.z, a[2][0], a[2][2]); s8x4_to_bf16x4(wb.z, a[2][1], a[2][3]);
    s8x4_to_bf16x4(wa.w, a[3][0], a[3][2]); s8x4_to_bf16x4(wb.w, a[3][1], a[3][3]);
#pragma unroll
    for (int t = 0; t < NT; t++) {
      const uint4 x0 = *reinterpret_cast<const uint4*>(xrow + (size_t)t * 8 * xstride + kb * 128);
      const uint4 x1 = *reinterpret_cast<const uint4*>(xrow + (size_t)t * 8 * xstride + kb * 128 + 16);
      mma_bf16(c[t], a[0][0], a[0][1], a[0][2], a[0][3], x0.x, x0.y);
      mma_bf16(c[t], a[1][0], a[1][1], a[1][2], a[1][3], x0.z, x0.w);
      mma_bf16(c[t], a[2][0], a[2][1], a[2][2], a[2][3], x1.x, x1.y);
      mma_bf16(c[t], a[3][0], a[3][1], a[3][2], a[3][3], x1.z, x1.w);
    }
  };
  if (kbs > 0) block64(0, pa[0], pb[0]);
  if (kbs > 1) block64(1, pa[1], pb[1]);
#pragma unroll 2
  for (int kb = 2; kb < kbs; kb++) {
    const uint4 wa = __ldg(reinterpret_cast<const uint4*>(w_lo + kb * 64));
    const uint4 wb = __ldg(reinterpret_cast<const uint4*>(w_hi + kb * 64));
    block64(kb, wa, wb);
  }
  // c[t][0], c[t][1]: row r_lo, tokens 8t + 2tig, + 1; c[t][2], c[t][3]: row r_hi
  const float s_lo = r_lo < N ? bf2f(__ldg(scale + r_lo)) : 0.f, s_hi = r_hi < N ? bf2f(__ldg(scale + r_hi)) : 0.f;
#pragma unroll
  for (int t = 0; t < NT; t++)
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int b = 8 * t + 2 * tig + (j & 1), r = (j & 2) ? r_hi : r_lo;
      if (b < B && r < N) {
        if (splits == 1) {
          const float v = c[t][j] * ((j & 2) ? s_hi : s_lo);
          if (y_f32) ((float*)y)[(size_t)b * N + r] = v;
          else ((uint16_t*)y)[(size_t)b * N + r] = f2bf(v);
        } else
          partial[((size_t)split * B + b) * N + r] = c[t][j];
      }
    }
}

__global__ void __launch_bounds__(256) gemv_finalize_kernel(const float* __restrict__ partial,
                                                            const uint16_t* __restrict__ scale,
                                                            void* __restrict__ y, int B, int N, int splits, int y_f32) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)B * N) return;
  const int n = (int)(i % N);
  float s = 0.f;
  for (int sp = 0; sp < splits; sp++) s += partial[(size_t)sp * B * N + i];
  if (y_f32) ((float*)y)[i] = s * bf2f(scale[n]);
  else ((uint16_t*)y)[i] = f2bf(s * bf2f(scale[n]));
}

// Per head: RMSNorm over head_dim (q and k heads; v is copied), rotate-half RoPE at position
// pos, q heads to q_out, the k/v heads appended to the caches [B, T, kv_heads * D].
// Rounding: the normalised head is rounded to bf16, the rotated value is rounded once.
__global__ void __launch_bounds__(128) rope_kv_kernel(const uint16_t* __restrict__ qkv, const int32_t* __restrict__ pos_p,
                                                      const uint16_t* __restrict__ qw, const uint16_t* __restrict__ kw,
                                                      uint16_t* __restrict__ q_out, uint16_t* __restrict__ kcache,
                                                      uint16_t* __restrict__ vcache, int n_q, int n_kv, int D, int T,
                                                      float theta, float eps, GemvPartials gp) {
  __shared__ float red[32];
  __shared__ float hv[512];
  const int b = blockIdx.x, h = blockIdx.y;  // h: q heads, then k heads, then v heads
  int pos = pos_p[0];
  pos = pos < 0 ? 0 : (pos >= T ? T - 1 : pos);
  const int width = (n_q + 2 * n_kv) * D;
  const size_t src = (size_t)b * width + (size_t)h * D;  // element offset of this head in qkv
  const size_t bn = (size_t)gridDim.x * width;
  const bool is_q = h < n_q, is_k = !is_q && h < n_q + n_kv;
  if (!is_q && !is_k) {  // v head: plain copy into the cache
    const int hk = h - n_q - n_kv;
    uint16_t* dst = vcache + (((size_t)b * T + pos) * n_kv + hk) * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = f2bf(operand_at(qkv, gp, bn, src + i, h * D + i));
    return;
  }
  const uint16_t* w = is_q ? qw : kw;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float v = operand_at(qkv, gp, bn, src + i, h * D + i);
    hv[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)D + eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x) hv[i] = bf2f(f2bf(hv[i] * inv * (1.0f + bf2f(w[i]))));
  __syncthreads();
  uint16_t* dst = is_q ? q_out + ((size_t)b * n_q + h) * D
                       : kcache + (((size_t)b * T + pos) * n_kv + (h - n_q)) * D;
  const int half = D >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float inv_freq = powf(theta, -(float)i / (float)half);
    float sn, cs;
    sincosf((float)pos * inv_freq, &sn, &cs);
    const float x1 = hv[i], x2 = hv[i + half];
    dst[i] = f2bf(x1 * cs - x2 * sn);
    dst[i + half] = f2bf(x2 * cs + x1 * sn);
  }
}

// Split-T single-query attention (one KV head shared by n_q query heads, D = 256):
// block = (batch b, T slice), warp w = query head w. Each warp keeps a running (max, sum,
// acc[D]) over its slice and writes it to scratch; attn_combine_kernel merges the slices.
constexpr int kAttnD = 256;
__global__ void __launch_bounds__(128) attn_partial_kernel(const uint16_t* __restrict__ q, const int32_t* __restrict__ pos_p,
                                                           const uint16_t* __restrict__ kcache,
                                                           const uint16_t* __restrict__ vcache, float* __restrict__ part,
                                                           int n_q, int T, int window, float scale) {
  const int b = blockIdx.x, sp = blockIdx.y, S = gridDim.y;
  const int h = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (h >= n_q) return;
  int pos = pos_p[0];
  pos = pos < 0 ? 0 : (pos >= T ? T - 1 : pos);
  const int t_lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int span = pos + 1 - t_lo;
  const int per = (span + S - 1) / S;
  const int t0 = t_lo + sp * per, t1 = min(pos + 1, t0 + per);
  // this lane's 8 dims of the query, pre-scaled
  float qv[8];
  {
    const uint4 qq = *reinterpret_cast<const uint4*>(q + ((size_t)b * n_q + h) * kAttnD + lane * 8);
    const uint32_t w[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      qv[2 * j] = __uint_as_float(w[j] << 16) * scale;
      qv[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u) * scale;
    }
  }
  float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
  for (int j = 0; j < 8; j++) acc[j] = 0.f;
  // four keys per round: their score reductions interleave and one rescale serves all four
  // and the next pass's rows are loaded before this pass's arithmetic (registers as the second buffer)
  uint4 kk[4], vv[4], nk[4], nv[4];
  auto load_round = [&](int t, uint4 (&kd)[4], uint4 (&vd)[4]) {
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const size_t off = ((size_t)b * T + min(t + u, t1 - 1)) * kAttnD + lane * 8;
      kd[u] = __ldg(reinterpret_cast<const uint4*>(kcache + off));
      vd[u] = __ldg(reinterpret_cast<const uint4*>(vcache + off));
    }
  };
  if (t0 < t1) load_round(t0, kk, vv);
  for (int t = t0; t < t1; t += 4) {
    if (t + 4 < t1) load_round(t + 4, nk, nv);
    float s[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const uint32_t kw[4] = {kk[u].x, kk[u].y, kk[u].z, kk[u].w};
      float d = 0.f;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        d = fmaf(qv[2 * j], __uint_as_float(kw[j] << 16), d);
        d = fmaf(qv[2 * j + 1], __uint_as_float(kw[j] & 0xffff0000u), d);
      }
      s[u] = d;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int u = 0; u < 4; u++) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
#pragma unroll
    for (int u = 1; u < 4; u++)
      if (t + u >= t1) s[u] = -INFINITY;  // past the slice: weight 0
    const float m_new = fmaxf(fmaxf(m, s[0]), fmaxf(fmaxf(s[1], s[2]), s[3]));
    const float corr = expf(m - m_new);
    float p[4];
#pragma unroll
    for (int u = 0; u < 4; u++) p[u] = expf(s[u] - m_new);
    l = l * corr + ((p[0] + p[1]) + (p[2] + p[3]));
#pragma unroll
    for (int j = 0; j < 8; j++) acc[j] *= corr;
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const uint32_t vw[4] = {vv[u].x, vv[u].y, vv[u].z, vv[u].w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        acc[2 * j] = fmaf(p[u], __uint_as_float(vw[j] << 16), acc[2 * j]);
        acc[2 * j + 1] = fmaf(p[u], __uint_as_float(vw[j] & 0xffff0000u), acc[2 * j + 1]);
      }
    }
    m = m_new;
#pragma unroll
    for (int u = 0; u < 4; u++) {
      kk[u] = nk[u];
      vv[u] = nv[u];
    }
  }
  float* dst = part + (((size_t)b * n_q + h) * S + sp) * (kAttnD + 2);
  if (lane == 0) {
    dst[0] = m;
    dst[1] = l;
  }
#pragma unroll
  for (int j = 0; j < 8; j++) dst[2 + lane * 8 + j] = acc[j];
}

__global__ void __launch_bounds__(256) attn_combine_kernel(const float* __restrict__ part, uint16_t* __restrict__ out,
                                                           int S) {
  const int bh = blockIdx.x, d = threadIdx.x;  // one block per (b, head), one thread per dim
  const float* p = part + (size_t)bh * S * (kAttnD + 2);
  float m = -INFINITY;
  for (int s = 0; s < S; s++) m = fmaxf(m, p[(size_t)s * (kAttnD + 2)]);
  float l = 0.f, o = 0.f;
  for (int s = 0; s < S; s++) {
    const float* ps = p + (size_t)s * (kAttnD + 2);
    if (ps[1] > 0.f) {
      const float c = expf(ps[0] - m);
      l += ps[1] * c;
      o += ps[2 + d] * c;
    }
  }
  out[(size_t)bh * kAttnD + d] = f2bf(o / l);
}

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.0f + tanhf(k0 * (x + k1 * x * x * x)));
}
// out[b, i] = bf16( bf16(gelu_tanh(gate)) * up ), gate = gu[b, i], up = gu[b, I + i]
__global__ void __launch_bounds__(256) geglu_kernel(const uint16_t* __restrict__ gu, uint16_t* __restrict__ out, int B,
                                                    int I, GemvPartials gp) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)B * I) return;
  const int i = (int)(idx % I);
  const size_t b = idx / I;
  const size_t bn = (size_t)B * 2 * I;
  const float g = operand_at(gu, gp, bn, b * 2 * I + i, i), u = operand_at(gu, gp, bn, b * 2 * I + I + i, I + i);
  out[idx] = f2bf(bf2f(f2bf(gelu_tanh(g))) * u);
}

// Block-quantised weights (the reference's Gemma form): y[b, n] = bf16( sum_k x[b, k] * wd[k, n] ),
// wd = bf16((W - zp) * scale), scale and zp per (block of `bs` consecutive k, n). The planner has
// transposed W to [N, K] and the per-block tables to [N, K / bs], so a warp streams one output row.
template <int BT>
__global__ void __launch_bounds__(256) gemv_q8b_kernel(const uint16_t* __restrict__ x, const int8_t* __restrict__ W,
                                                       const uint16_t* __restrict__ scale, const int8_t* __restrict__ zp,
                                                       uint16_t* __restrict__ y, int B, int N, int K, int bs) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const int nblk = K / bs;
  float acc[BT];
#pragma unroll
  for (int b = 0; b < BT; b++) acc[b] = 0.f;
  const int8_t* wrow = W + (size_t)n * K;
  for (int k = lane * 16; k < K; k += 32 * 16) {
    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wrow + k));
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
    const int blk = k / bs;  // bs is a multiple of 16: the 16 weights share a block
    const float s = bf2f(__ldg(scale + (size_t)n * nblk + blk));
    const int z = zp ? (int)__ldg(zp + (size_t)n * nblk + blk) : 0;
    float wd[16];
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const int w8 = (int)(int8_t)(ww[j >> 2] >> (8 * (j & 3)));
      wd[j] = bf2f(f2bf((float)(w8 - z) * s));
    }
#pragma unroll
    for (int b = 0; b < BT; b++)
      if (b < B) {
        const uint4 x0 = __ldg(reinterpret_cast<const uint4*>(x + (size_t)b * K + k));
        const uint4 x1 = __ldg(reinterpret_cast<const uint4*>(x + (size_t)b * K + k + 8));
        const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        float a = acc[b];
#pragma unroll
        for (int j = 0; j < 8; j++) {
          a = fmaf(wd[2 * j], __uint_as_float(xw[j] << 16), a);
          a = fmaf(wd[2 * j + 1], __uint_as_float(xw[j] & 0xffff0000u), a);
        }
        acc[b] = a;
      }
  }
#pragma unroll
  for (int b = 0; b < BT; b++) acc[b] = warp_sum(acc[b]);
  if (lane == 0)
#pragma unroll
    for (int b = 0; b < BT; b++)
      if (b < B) y[(size_t)b * N + n] = f2bf(acc[b]);
}

// four signed bytes -> (byte - zp) * scale, each rounded to bf16: two bf16x2 words (k, k+1) and (k+2, k+3)
__device__ __forceinline__ void s8x4_dequant_bf16x4(uint32_t w, int z, float s, uint32_t& lo, uint32_t& hi) {
  const float f0 = (float)((int)(int8_t)w - z) * s, f1 = (float)((int)(int8_t)(w >> 8) - z) * s;
  const float f2 = (float)((int)(int8_t)(w >> 16) - z) * s, f3 = (float)(((int)w >> 24) - z) * s;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(f1), "f"(f0));
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(f3), "f"(f2));
}

// The same product for batches above 8 on the tensor cores: blocks of 128 output rows, the activations of all
// tokens staged in shared memory one K chunk at a time, the weights dequantised to bf16 in registers exactly as
// above ((W - zp) * scale, one rounding) and fed to mma.sync m16n8k16 with fp32 accumulation. K % 64 == 0 and a
// block size that is a multiple of 16 (the 16 consecutive weights a lane holds share a block).
template <int NT>  // groups of 8 tokens
__global__ void __launch_bounds__(256) gemv_q8b_mma_kernel(const uint16_t* __restrict__ x, const int8_t* __restrict__ W,
                                                           const uint16_t* __restrict__ scale,
                                                           const int8_t* __restrict__ zp, uint16_t* __restrict__ y, int B,
                                                           int N, int K, int bs, int k_chunk) {
  extern __shared__ __align__(16) unsigned char xs_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int xstride = ((k_chunk * 2 + 127) / 128) * 128 + 16;  // bytes per token row in shared memory
  const int row0 = blockIdx.x * 128 + warp * 16;
  const bool active = row0 < N;
  const int r_lo = min(row0 + g, N - 1), r_hi = min(row0 + g + 8, N - 1);
  const int nblk = K / bs;
  const int8_t* w_lo = W + (size_t)r_lo * K + tig * 16;
  const int8_t* w_hi = W + (size_t)r_hi * K + tig * 16;
  float c[NT][4];
#pragma unroll
  for (int t = 0; t < NT; t++)
#pragma unroll
    for (int j = 0; j < 4; j++) c[t][j] = 0.f;
  const unsigned char* xrow = xs_raw + (size_t)g * xstride + tig * 32;
  for (int k0 = 0; k0 < K; k0 += k_chunk) {
    const int k_len = min(k_chunk, K - k0);  // a multiple of 64
    if (k0 > 0) __syncthreads();
    for (int i = threadIdx.x; i < NT * 8 * (k_len / 8); i += blockDim.x) {
      const int b = i / (k_len / 8), cc = i % (k_len / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (b < B) v = __ldg(reinterpret_cast<const uint4*>(x + (size_t)b * K + k0) + cc);
      *reinterpret_cast<uint4*>(xs_raw + (size_t)b * xstride + 16 * cc) = v;
    }
    __syncthreads();
    if (!active) continue;
#pragma unroll 2
    for (int kb = 0; kb < (k_len >> 6); kb++) {
      const int k = k0 + kb * 64;
      const uint4 wa = __ldg(reinterpret_cast<const uint4*>(w_lo + k));
      const uint4 wb = __ldg(reinterpret_cast<const uint4*>(w_hi + k));
      const int blk = (k + tig * 16) / bs;
      const float s_lo = bf2f(__ldg(scale + (size_t)r_lo * nblk + blk)), s_hi = bf2f(__ldg(scale + (size_t)r_hi * nblk + blk));
      const int z_lo = zp ? (int)__ldg(zp + (size_t)r_lo * nblk + blk) : 0, z_hi = zp ? (int)__ldg(zp + (size_t)r_hi * nblk + blk) : 0;
      uint32_t a[4][4];
      s8x4_dequant_bf16x4(wa.x, z_lo, s_lo, a[0][0], a[0][2]); s8x4_dequant_bf16x4(wb.x, z_hi, s_hi, a[0][1], a[0][3]);
      s8x4_dequant_bf16x4(wa.y, z_lo, s_lo, a[1][0], a[1][2]); s8x4_dequant_bf16x4(wb.y, z_hi, s_hi, a[1][1], a[1][3]);
      s8x4_dequant_bf16x4(wa.z, z_lo, s_lo, a[2][0], a[2][2]); s8x4_dequant_bf16x4(wb.z, z_hi, s_hi, a[2][1], a[2][3]);
      s8x4_dequant_bf16x4(wa.w, z_lo, s_lo, a[3][0], a[3][2]); s8x4_dequant_bf16x4(wb.w, z_hi, s_hi, a[3][1], a[3][3]);
#pragma unroll
      for (int t = 0; t < NT; t++) {
        const uint4 x0 = *reinterpret_cast<const uint4*>(xrow + (size_t)t * 8 * xstride + kb * 128);
        const uint4 x1 = *reinterpret_cast<const uint4*>(xrow + (size_t)t * 8 * xstride + kb * 128 + 16);
        mma_bf16(c[t], a[0][0], a[0][1], a[0][2], a[0][3], x0.x, x0.y);
        mma_bf16(c[t], a[1][0], a[1][1], a[1][2], a[1][3], x0.z, x0.w);
        mma_bf16(c[t], a[2][0], a[2][1], a[2][2], a[2][3], x1.x, x1.y);
        mma_bf16(c[t], a[3][0], a[3][1], a[3][2], a[3][3], x1.z, x1.w);
      }
    }
  }
  if (!active) return;
  // c[t][0], c[t][1]: row g, tokens 8t + 2tig, + 1; c[t][2], c[t][3]: row g + 8
#pragma unroll
  for (int t = 0; t < NT; t++)
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int b = 8 * t + 2 * tig + (j & 1), r = row0 + g + ((j & 2) ? 8 : 0);
      if (b < B && r < N) y[(size_t)b * N + r] = f2bf(c[t][j]);
    }
}

// y = bf16(f(x)), f evaluated in fp32: the host semantics of the reference's bf16 activation
// patterns (python/torq/testing/numpy.py:13-27 is the fp32 form its tests compare with; the NPU's
// piecewise-linear tables, scripts/bf16luts.py, approximate the same functions).
__global__ void __launch_bounds__(256) act_bf16_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ out,
                                                       long long n, int fn) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = bf2f(x[i]);
    float r;
    switch (fn) {
      case 0: r = 1.0f / (1.0f + expf(-v)); break;
      case 1: r = gelu_tanh(v); break;
      case 2: r = expf(v); break;
      case 3: r = tanhf(v); break;
      default: r = v / (1.0f + expf(-v)); break;
    }
    out[i] = f2bf(r);
  }
}

// greedy token: arg max over the vocabulary, lowest index on ties; two stages through scratch
constexpr int kArgmaxChunks = 64;
__global__ void __launch_bounds__(256) argmax_partial_kernel(const void* __restrict__ logits, int is_f32,
                                                             float* __restrict__ pv, int32_t* __restrict__ pi, int V) {
  __shared__ float sv[256];
  __shared__ int si[256];
  const int b = blockIdx.x, ch = blockIdx.y;
  const int per = (V + kArgmaxChunks - 1) / kArgmaxChunks;
  const int v0 = ch * per, v1 = min(V, v0 + per);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
    const float x = is_f32 ? ((const float*)logits)[(size_t)b * V + v] : bf2f(((const uint16_t*)logits)[(size_t)b * V + v]);
    if (x > best || (x == best && v < bi)) {
      best = x;
      bi = v;
    }
  }
  sv[threadIdx.x] = best;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      const float x = sv[threadIdx.x + o];
      const int i = si[threadIdx.x + o];
      if (x > sv[threadIdx.x] || (x == sv[threadIdx.x] && i < si[threadIdx.x])) {
        sv[threadIdx.x] = x;
        si[threadIdx.x] = i;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    pv[b * kArgmaxChunks + ch] = sv[0];
    pi[b * kArgmaxChunks + ch] = si[0];
  }
}
__global__ void argmax_final_kernel(const float* __restrict__ pv, const int32_t* __restrict__ pi, int32_t* __restrict__ out) {
  const int b = blockIdx.x;
  if (threadIdx.x != 0) return;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = 0; c < kArgmaxChunks; c++) {
    const float x = pv[b * kArgmaxChunks + c];
    const int i = pi[b * kArgmaxChunks + c];
    if (x > best || (x == best && i < bi)) {
      best = x;
      bi = i;
    }
  }
  out[b] = bi;
}

}  // namespace

void launch_embed(const int32_t* tok, const int8_t* table, const uint16_t* scale, uint16_t* out, int B, int H, int V,
                  float mult, cudaStream_t stream) {
  launch_k(embed_kernel, dim3(B), dim3(128), 0, stream, tok, table, scale, out, H, V, mult);
}

void launch_rmsnorm(const uint16_t* x, const uint16_t* res, const uint16_t* w, uint16_t* out, int rows, int H, float eps,
                    cudaStream_t stream) {
  launch_k(rmsnorm_kernel, dim3(rows), dim3(1024), 0, stream, x, res, w, out, H, eps);
}

// Batches of 3 and more with K a multiple of 64 take the tensor-core kernel (measured crossover with the
// CUDA-core kernel and with the fused step; TB200_GEMV_MMA_MIN_B moves it): K slices of a multiple of 64.
static bool gemv_use_mma(int B, int K) {
  static int min_b = -1;
  if (min_b < 0) { const char* e = getenv("TB200_GEMV_MMA_MIN_B"); min_b = e ? atoi(e) : 3; }
  return B >= min_b && (K % 64) == 0;
}
static int gemv_mma_slice(int N, int K, int splits) {
  int slice = ((K + splits - 1) / splits + 63) / 64 * 64;
  (void)N;
  return slice;
}

int gemv_w8_splits(int B, int N, int K) {
  if (gemv_use_mma(B, K)) {
    // blocks of 128 rows: split K until about two blocks per SM exist, slices >= 128 bytes, <= 16 slices;
    // a slice of x for 32 tokens must fit in shared memory (K = 1152 unsplit: 74 KB)
    const long long row_blocks = (N + 127) / 128;
    int splits = (int)((2 * 148 + row_blocks - 1) / row_blocks);
    const int max_splits = K / 128 > 0 ? K / 128 : 1;
    if (splits > max_splits) splits = max_splits;
    static int cap = -1;  // TB200_GEMV_MAX_SPLITS: upper bound on the K slices of the tensor-core kernel
    if (cap < 0) { const char* e = getenv("TB200_GEMV_MAX_SPLITS"); cap = e && atoi(e) > 0 ? atoi(e) : 16; }
    if (splits > cap) splits = cap;
    if (splits < 1) splits = 1;
    while (gemv_mma_slice(N, K, splits) > 2048) splits++;  // shared-memory bound on the x slice
    return splits;
  }
  // enough warps to fill the machine: one warp per (row, slice); slices are multiples of 512 bytes
  const long long warps_wanted = 148LL * 32;
  int splits = (int)((warps_wanted + N - 1) / N);
  const int max_splits = K / 512 > 0 ? K / 512 : 1;
  if (splits > max_splits) splits = max_splits;
  if (splits > 16) splits = 16;
  if (splits < 1) splits = 1;
  (void)B;
  return splits;
}

bool gemv_w8_splits_fit(int B, int N, int K, int splits) {
  return splits >= 1 && (!gemv_use_mma(B, K) || gemv_mma_slice(N, K, splits) <= 2048);
}

size_t gemv_w8_scratch_bytes(int B, int N, int splits) { return splits > 1 ? (size_t)splits * B * N * sizeof(float) : 0; }

int gemv_w8_used_splits(int B, int N, int K, int splits) {
  const int slice = gemv_use_mma(B, K) ? gemv_mma_slice(N, K, splits) : ((K + splits - 1) / splits + 511) / 512 * 512;
  return (K + slice - 1) / slice;
}

void launch_rmsnorm_fused(const uint16_t* x, GemvPartials gp, const uint16_t* res, const uint16_t* w, uint16_t* out,
                          const uint16_t* w2, uint16_t* out2, int rows, int H, float eps, float eps2,
                          cudaStream_t stream) {
  launch_k(rmsnorm_fused_kernel, dim3(rows), dim3(1024), (size_t)H * sizeof(float), stream, x, gp, res, w, out, w2, out2, rows, H, eps, eps2);
}

void launch_gemv_w8(const uint16_t* x, const int8_t* W, const uint16_t* scale, void* y, int y_f32, float* scratch, int B,
                    int N, int K, int splits, cudaStream_t stream, bool finalize) {
  if (gemv_use_mma(B, K)) {
    const int slice = gemv_mma_slice(N, K, splits);
    const int used = (K + slice - 1) / slice;
    const int nt = (B + 7) / 8;
    const int xstride = ((slice * 2 + 127) / 128) * 128 + 16;
    const size_t smem = (size_t)nt * 8 * xstride;
    dim3 grid((N + 127) / 128, used);
    auto run = [&](auto kernel) {
      // one flag per kernel (the four instantiations share the lambda's type); function attributes are per device
      static std::atomic<unsigned long long> attr_done[5];
      if (first_use_on_device(attr_done[nt])) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        mark_used_on_device(attr_done[nt]);
      }
      launch_k(kernel, dim3(grid), dim3(256), smem, stream, x, W, scale, y, scratch, B, N, K, slice, y_f32);
    };
    if (nt == 1) run(gemv_w8_mma_kernel<1>);
    else if (nt == 2) run(gemv_w8_mma_kernel<2>);
    else if (nt == 3) run(gemv_w8_mma_kernel<3>);
    else run(gemv_w8_mma_kernel<4>);
    if (used > 1 && finalize) {
      const size_t total = (size_t)B * N;
      launch_k(gemv_finalize_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, scratch, scale, y, B, N, used, y_f32);
    }
    return;
  }
  const int slice = ((K + splits - 1) / splits + 511) / 512 * 512;
  const int used = (K + slice - 1) / slice;  // slices that really hold data
  dim3 grid((N + 7) / 8, used);
  if (B <= 1) launch_k(gemv_w8_kernel<1>, dim3(grid), dim3(256), 0, stream, x, W, scale, y, scratch, B, N, K, slice, y_f32);
  else if (B <= 4) launch_k(gemv_w8_kernel<4>, dim3(grid), dim3(256), 0, stream, x, W, scale, y, scratch, B, N, K, slice, y_f32);
  else if (B <= 8) launch_k(gemv_w8_kernel<8>, dim3(grid), dim3(256), 0, stream, x, W, scale, y, scratch, B, N, K, slice, y_f32);
  else if (B <= 16) launch_k(gemv_w8_kernel<16>, dim3(grid), dim3(256), 0, stream, x, W, scale, y, scratch, B, N, K, slice, y_f32);
  else launch_k(gemv_w8_kernel<32>, dim3(grid), dim3(256), 0, stream, x, W, scale, y, scratch, B, N, K, slice, y_f32);
  if (used > 1 && finalize) {
    const size_t total = (size_t)B * N;
    launch_k(gemv_finalize_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, scratch, scale, y, B, N, used, y_f32);
  }
}

void launch_rope_kv(const uint16_t* qkv, const int32_t* pos, const uint16_t* qw, const uint16_t* kw, uint16_t* q_out,
                    uint16_t* kcache, uint16_t* vcache, int B, int n_q, int n_kv, int D, int T, float theta, float eps,
                    cudaStream_t stream, GemvPartials gp) {
  launch_k(rope_kv_kernel, dim3(dim3(B, n_q + 2 * n_kv)), dim3(128), 0, stream, qkv, pos, qw, kw, q_out, kcache, vcache, n_q, n_kv, D, T,
                                                              theta, eps, gp);
}

int attn_decode_splits(int B) {
  static int forced = -1;  // TB200_ATTN_SPLITS: T slices of the split-T attention (1..64), else by batch
  if (forced < 0) { const char* e = getenv("TB200_ATTN_SPLITS"); forced = e && atoi(e) > 0 && atoi(e) <= 64 ? atoi(e) : 0; }
  if (forced) return forced;
  return B >= 16 ? 16 : 32;
}
size_t attn_decode_scratch_bytes(int B, int n_q, int splits) {
  return (size_t)B * n_q * splits * (kAttnD + 2) * sizeof(float);
}
void launch_attn_decode(const uint16_t* q, const int32_t* pos, const uint16_t* kcache, const uint16_t* vcache,
                        uint16_t* out, float* scratch, int B, int n_q, int T, int window, float scale, int splits,
                        cudaStream_t stream) {
  launch_k(attn_partial_kernel, dim3(dim3(B, splits)), dim3(128), 0, stream, q, pos, kcache, vcache, scratch, n_q, T, window, scale);
  launch_k(attn_combine_kernel, dim3(B * n_q), dim3(kAttnD), 0, stream, scratch, out, splits);
}

void launch_geglu(const uint16_t* gu, uint16_t* out, int B, int I, cudaStream_t stream, GemvPartials gp) {
  const size_t total = (size_t)B * I;
  launch_k(geglu_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, gu, out, B, I, gp);
}

void launch_gemv_q8b(const uint16_t* x, const int8_t* W, const uint16_t* scale, const int8_t* zp, uint16_t* y, int B, int N,
                     int K, int bs, cudaStream_t stream) {
  if (B > 8) {  // tensor cores; the planner has checked K % 64 == 0 and B <= 32
    const int nt = (B + 7) / 8;
    const int k_chunk = K < 1024 ? K : 1024;
    const int xstride = ((k_chunk * 2 + 127) / 128) * 128 + 16;
    const size_t smem = (size_t)nt * 8 * xstride;
    auto run = [&](auto kernel) {
      static std::atomic<unsigned long long> attr_done[5];  // per instantiation (index nt) and device
      if (first_use_on_device(attr_done[nt])) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        mark_used_on_device(attr_done[nt]);
      }
      launch_k(kernel, dim3((N + 127) / 128), dim3(256), smem, stream, x, W, scale, zp, y, B, N, K, bs, k_chunk);
    };
    if (nt == 2) run(gemv_q8b_mma_kernel<2>);
    else if (nt == 3) run(gemv_q8b_mma_kernel<3>);
    else run(gemv_q8b_mma_kernel<4>);
    return;
  }
  const dim3 grid((N + 7) / 8);
  if (B <= 1) launch_k(gemv_q8b_kernel<1>, dim3(grid), dim3(256), 0, stream, x, W, scale, zp, y, B, N, K, bs);
  else if (B <= 4) launch_k(gemv_q8b_kernel<4>, dim3(grid), dim3(256), 0, stream, x, W, scale, zp, y, B, N, K, bs);
  else launch_k(gemv_q8b_kernel<8>, dim3(grid), dim3(256), 0, stream, x, W, scale, zp, y, B, N, K, bs);
}

void launch_act_bf16(const uint16_t* x, uint16_t* out, long long n, int fn, cudaStream_t stream) {
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  launch_k(act_bf16_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, x, out, n, fn);
}

size_t argmax_scratch_bytes(int B) { return (size_t)B * kArgmaxChunks * 8; }
void launch_argmax(const void* logits, int is_f32, int32_t* out, void* scratch, int B, int V, cudaStream_t stream) {
  float* pv = (float*)scratch;
  int32_t* pi = (int32_t*)((char*)scratch + (size_t)B * kArgmaxChunks * 4);
  launch_k(argmax_partial_kernel, dim3(dim3(B, kArgmaxChunks)), dim3(256), 0, stream, logits, is_f32, pv, pi, V);
  launch_k(argmax_final_kernel, dim3(B), dim3(32), 0, stream, pv, pi, out);
}

// ---------------------------------------------------------------------------------------
// tb200_gemv_w8_noalloc: the split-K int8-weight GEMV for callers that must not allocate.
//
// Who that is: a host that has handed all device memory to its own allocator (a HAL
// allocator that reserved the HBM, a serving engine with a fixed memory plan) has no free
// memory left for a cudaMalloc made behind its back, and a latency-critical loop cannot take
// the device-wide synchronisation an allocation may imply. For them the partial sums of
// the split-K reduction live in the fixed array below instead of a buffer from the arena.
//
// The array belongs to the library image: every GPU that loads the library holds its
// 4 MiB until the process exits. All calls on a device share it and it keeps whatever the
// last call left there. Nothing in it has to start at zero - each (slice, row, column)
// partial is written by exactly one warp before the reduction kernel reads it - but two
// calls whose kernels overlap on the GPU (different streams, or different host threads
// without ordering) would overwrite each other's partial sums: callers must order them.
// ---------------------------------------------------------------------------------------
namespace {
constexpr size_t kNoAllocScratchFloats = 1u << 20;  // 4 MiB: slices * batch * N must fit
static __device__ __align__(256) float g_noalloc_gemv_scratch[kNoAllocScratchFloats];
constexpr int kMaxDevices = 64;
float* g_noalloc_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mutex;
}  // namespace

}  // namespace tb200

// Status numbers are those of include/torq_b200.h (0 OK, 3 INVALID_ARGUMENT, 11 OUT_OF_RANGE,
// 13 INTERNAL). All pointers are device pointers on GPU `cuda_ordinal`; `stream` is a
// cudaStream_t (NULL = the default stream). The first call on a device looks up the device
// address of the scratch array (cudaGetSymbolAddress with that device current); make that
// first call before any stream capture begins. No cudaMalloc, cudaFree or allocating
// library routine is called, on the first call or later.
extern "C" int tb200_gemv_w8_noalloc(int cuda_ordinal, void* stream, const void* x_bf16, const void* w_i8,
                                     const void* scale_bf16, void* y, int y_is_f32, int B, int N, int K,
                                     int splits) {
  using namespace tb200;
  if (!x_bf16 || !w_i8 || !scale_bf16 || !y || B < 1 || B > 32 || N < 1 || K < 16 || (K % 16) != 0 ||
      cuda_ordinal < 0 || cuda_ordinal >= kMaxDevices)
    return 3;
  // the kernels read x and W with 16-byte vector loads; the scales and y are accessed element by element
  if (((uintptr_t)x_bf16 & 15) || ((uintptr_t)w_i8 & 15) || ((uintptr_t)y & (y_is_f32 ? 3 : 1)) || ((uintptr_t)scale_bf16 & 1)) {
    fprintf(stderr, "tb200_gemv_w8_noalloc: x and W must be 16-byte aligned, y and the scales aligned to their element\n");
    return 3;
  }
  if (splits <= 0) splits = gemv_w8_splits(B, N, K);
  if (!gemv_w8_splits_fit(B, N, K, splits)) {
    fprintf(stderr,
            "tb200_gemv_w8_noalloc: %d slices of K = %d leave a slice of the input too long for the tensor-core kernel's "
            "shared memory (at most 2048 values per slice at batch >= 3); use more slices\n", splits, K);
    return 11;
  }
  if ((size_t)splits * (size_t)B * (size_t)N > kNoAllocScratchFloats) {
    fprintf(stderr,
            "tb200_gemv_w8_noalloc: %d slices x batch %d x %d columns = %zu partial sums exceed the fixed scratch of "
            "%zu floats; use fewer slices or the executable path\n",
            splits, B, N, (size_t)splits * B * N, (size_t)kNoAllocScratchFloats);
    return 11;
  }
  // the caller's current device is put back before returning
  int caller_device = -1;
  if (cudaGetDevice(&caller_device) != cudaSuccess) return 13;
  struct RestoreDevice {
    int dev;
    ~RestoreDevice() { if (dev >= 0) cudaSetDevice(dev); }
  } restore{caller_device == cuda_ordinal ? -1 : caller_device};
  if (caller_device != cuda_ordinal && cudaSetDevice(cuda_ordinal) != cudaSuccess) return 13;
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_scratch_ptr[cuda_ordinal]) {
      // In host code the array's name is only a handle: the device address has to be asked for,
      // once per device, with that device current.
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_noalloc_gemv_scratch) != cudaSuccess || !p) return 13;
      g_noalloc_scratch_ptr[cuda_ordinal] = (float*)p;
    }
    scratch = g_noalloc_scratch_ptr[cuda_ordinal];
  }
  (void)cudaGetLastError();  // an earlier, unrelated error of the host must not be reported as this call's
  launch_gemv_w8((const uint16_t*)x_bf16, (const int8_t*)w_i8, (const uint16_t*)scale_bf16, y, y_is_f32 ? 1 : 0, scratch,
                 B, N, K, splits, (cudaStream_t)stream);
  return cudaGetLastError() == cudaSuccess ? 0 : 13;
}
