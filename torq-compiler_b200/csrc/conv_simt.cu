// CUDA-core (dp4a) convolution kernels: the general path for any kernel size,
// stride, dilation, padding and channel count. The tensor-core path in
// gemm_tcgen05.cu takes over the shapes it supports; results are bit-identical.
//
// Arithmetic (torq_hl.conv2d, compiler/torq/Conversions/LinalgToTorqHL/Conv2DPattern.cpp:478-654):
//   acc = bias + sum (x - izp) * (w - wzp), taps outside the image hold izp.
// The kernel accumulates raw x*w with dp4a, staging izp bytes for outside taps, so
//   sum (x-izp)(w-wzp) = sum x*w - izp*sum(w) - wzp*sum(x) + K*izp*wzp
// with sums over ALL K taps; the izp terms are constants per output channel and
// arrive folded into ChanParams::bias. int32 wrap-around keeps this exact.
#include "kernels.h"
#include "dependent_launch.cuh"

namespace tb200 {

namespace {

constexpr int BM = 64;   // output pixels per block
constexpr int BN = 64;   // output channels per block
constexpr int BK = 32;   // K bytes per step
constexpr int KW4 = BK / 4;
constexpr int LDS = KW4 + 1;  // padded row (words) -> conflict-free column reads

template <bool IC4>
__global__ void __launch_bounds__(256) conv2d_simt_kernel(ConvArgs a) {
  __shared__ uint32_t As[BM][LDS];
  __shared__ uint32_t Bs[BN][LDS];

  const int tid = threadIdx.x;
  const int tx = tid & 15;   // pixel lane
  const int ty = tid >> 4;   // oc lane
  const long long P = (long long)a.N * a.OH * a.OW;
  const long long p_base = (long long)blockIdx.x * BM;
  const int oc_base = blockIdx.y * BN;

  // this thread stages word `lw` of pixels lp0 and lp0 + 32, and of oc rows lp0, lp0 + 32
  const int lw = tid & 7;
  const int lp0 = tid >> 3;
  int ih0[2], iw0[2];
  const int8_t* xin[2];
  bool pvalid[2];
#pragma unroll
  for (int r = 0; r < 2; r++) {
    long long p = p_base + lp0 + 32 * r;
    pvalid[r] = p < P;
    long long pp = pvalid[r] ? p : 0;
    int ow = (int)(pp % a.OW);
    long long t = pp / a.OW;
    int oh = (int)(t % a.OH);
    int n = (int)(t / a.OH);
    ih0[r] = oh * a.stride_h - a.pad_t;
    iw0[r] = ow * a.stride_w - a.pad_l;
    xin[r] = a.x + (size_t)n * a.H * a.W * a.IC;
  }
  const uint32_t zp_byte = (uint32_t)(a.input_zp & 0xff);
  const uint32_t zp_word = zp_byte * 0x01010101u;

  int acc[4][4];
  int xsum[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    xsum[i] = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0;
  }

  for (int k0 = 0; k0 < a.Kpad; k0 += BK) {
    const int k = k0 + lw * 4;
    // ---- stage A (implicit im2col gather) ----
    if (IC4) {
      int tap = k / a.IC;
      int ic = k - tap * a.IC;
      int kh = tap / a.KW;
      int kw = tap - kh * a.KW;
#pragma unroll
      for (int r = 0; r < 2; r++) {
        uint32_t v = 0;
        if (pvalid[r] && k < a.K) {
          int ih = ih0[r] + kh * a.dil_h;
          int iw = iw0[r] + kw * a.dil_w;
          if (ih >= 0 && ih < a.H && iw >= 0 && iw < a.W)
            v = *reinterpret_cast<const uint32_t*>(xin[r] + ((size_t)ih * a.W + iw) * a.IC + ic);
          else
            v = zp_word;
        }
        As[lp0 + 32 * r][lw] = v;
      }
    } else {
#pragma unroll
      for (int r = 0; r < 2; r++) {
        uint32_t v = 0;
        if (pvalid[r]) {
#pragma unroll
          for (int b = 0; b < 4; b++) {
            int kk = k + b;
            uint32_t byte = 0;
            if (kk < a.K) {
              int tap = kk / a.IC;
              int ic = kk - tap * a.IC;
              int kh = tap / a.KW;
              int kw = tap - kh * a.KW;
              int ih = ih0[r] + kh * a.dil_h;
              int iw = iw0[r] + kw * a.dil_w;
              if (ih >= 0 && ih < a.H && iw >= 0 && iw < a.W)
                byte = (uint8_t)xin[r][((size_t)ih * a.W + iw) * a.IC + ic];
              else
                byte = zp_byte;
            }
            v |= byte << (8 * b);
          }
        }
        As[lp0 + 32 * r][lw] = v;
      }
    }
    // ---- stage B (packed weights, rows padded to Kpad with zeros) ----
#pragma unroll
    for (int r = 0; r < 2; r++) {
      int oc = oc_base + lp0 + 32 * r;
      uint32_t v = 0;
      if (oc < a.OC) v = *reinterpret_cast<const uint32_t*>(a.w + (size_t)oc * a.Kpad + k);
      Bs[lp0 + 32 * r][lw] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < KW4; kk++) {
      uint32_t av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) av[i] = As[tx + 16 * i][kk];
#pragma unroll
      for (int j = 0; j < 4; j++) bv[j] = Bs[ty * 4 + j][kk];
#pragma unroll
      for (int i = 0; i < 4; i++) {
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = __dp4a((int)av[i], (int)bv[j], acc[i][j]);
      }
      if (a.weight_zp != 0) {
#pragma unroll
        for (int i = 0; i < 4; i++) xsum[i] = __dp4a((int)av[i], 0x01010101, xsum[i]);
      }
    }
    __syncthreads();
  }

  // ---- epilogue: bias, per-channel rescale, zero point, clamp ----
  const int oc0 = oc_base + ty * 4;
  ChanParams cp[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    if (oc0 + j < a.OC) cp[j] = a.chan[oc0 + j];
    else cp[j] = ChanParams{};
  }
  const bool hi = a.hi_shift != 0;
  const bool vec_ok = ((a.OC & 3) == 0) && (oc0 + 3 < a.OC);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    long long p = p_base + tx + 16 * i;
    if (p >= P) continue;
    int q[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int v = acc[i][j] - a.weight_zp * xsum[i] + cp[j].bias;
      q[j] = hi ? requant_cp<true>(v, cp[j], a.out_zp, a.clamp_min, a.clamp_max)
                : requant_cp<false>(v, cp[j], a.out_zp, a.clamp_min, a.clamp_max);
      if (a.lut) q[j] = __ldg(a.lut + q[j] + 128);
    }
    int8_t* o = a.out + (size_t)p * a.OC + oc0;
    if (vec_ok) {
      *reinterpret_cast<uint32_t*>(o) = pack4(q[0], q[1], q[2], q[3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; j++)
        if (oc0 + j < a.OC) o[j] = (int8_t)q[j];
    }
  }
}

// Few input channels (IC <= 4, K = KH*KW*IC <= 64), e.g. the 3x3x3 stem of an image
// network: a thread gathers the K patch bytes of kPix output pixels into registers once
// and runs every output channel against weights broadcast from shared memory, so each
// weight word read serves kPix pixels. Same arithmetic as conv2d_simt_kernel (izp staged
// for taps outside the image).
constexpr int kPix = 2;
// S333: the 3x3 window over 3 channels, with the tap arithmetic folded at compile time.
template <int KWORDS, bool S333>
__global__ void __launch_bounds__(128) conv2d_smallic_kernel(ConvArgs a) {
  extern __shared__ uint32_t w_s[];  // [OC][KWORDS]
  for (int i = threadIdx.x; i < a.OC * KWORDS; i += blockDim.x) {
    const int oc = i / KWORDS, kw = i - oc * KWORDS;
    w_s[i] = (kw * 4 < a.Kpad) ? *reinterpret_cast<const uint32_t*>(a.w + (size_t)oc * a.Kpad + kw * 4) : 0u;
  }
  __syncthreads();
  const long long P = (long long)a.N * a.OH * a.OW;
  // pixel i of this thread: block base + i * 128 + thread, so a warp's stores stay adjacent
  const long long p_base = (long long)blockIdx.x * (128 * kPix) + threadIdx.x;
  const uint32_t zp_byte = (uint32_t)(a.input_zp & 0xff);

  uint32_t patch[kPix][KWORDS];
#pragma unroll
  for (int px = 0; px < kPix; px++) {
    const long long p = p_base + px * 128;
    const long long pp = p < P ? p : 0;
    const int ow = (int)(pp % a.OW);
    long long t = pp / a.OW;
    const int oh = (int)(t % a.OH);
    const int n = (int)(t / a.OH);
    const int ih0 = oh * a.stride_h - a.pad_t, iw0 = ow * a.stride_w - a.pad_l;
    const int8_t* xin = a.x + (size_t)n * a.H * a.W * a.IC;
#pragma unroll
    for (int i = 0; i < KWORDS; i++) {
      uint32_t word = 0;
#pragma unroll
      for (int b = 0; b < 4; b++) {
        const int k = 4 * i + b;
        if (S333) {
          if (k < 27) {
            constexpr int kdiv3[28] = {0, 0, 0, 1, 1, 1, 2, 2, 2, 3, 3, 3, 4, 4, 4, 5, 5, 5, 6, 6, 6, 7, 7, 7, 8, 8, 8, 9};
            const int tap = kdiv3[k < 27 ? k : 27], ic = k - tap * 3;
            const int kh = kdiv3[tap], kw = tap - kh * 3;
            const int ih = ih0 + kh * a.dil_h, iw = iw0 + kw * a.dil_w;
            const uint32_t byte = (ih >= 0 && ih < a.H && iw >= 0 && iw < a.W)
                                      ? (uint32_t)(uint8_t)xin[((size_t)ih * a.W + iw) * 3 + ic]
                                      : zp_byte;
            word |= byte << (8 * b);
          }
        } else if (k < a.K) {
          const int tap = k / a.IC, ic = k - tap * a.IC;
          const int kh = tap / a.KW, kw = tap - kh * a.KW;
          const int ih = ih0 + kh * a.dil_h, iw = iw0 + kw * a.dil_w;
          const uint32_t byte = (ih >= 0 && ih < a.H && iw >= 0 && iw < a.W)
                                    ? (uint32_t)(uint8_t)xin[((size_t)ih * a.W + iw) * a.IC + ic]
                                    : zp_byte;
          word |= byte << (8 * b);
        }
      }
      patch[px][i] = word;
    }
  }
  const bool hi = a.hi_shift != 0;
  for (int oc0 = 0; oc0 < a.OC; oc0 += 4) {
    int q[kPix][4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int oc = min(oc0 + j, a.OC - 1);
      int acc[kPix];
#pragma unroll
      for (int px = 0; px < kPix; px++) acc[px] = 0;
#pragma unroll
      for (int i = 0; i < KWORDS; i++) {
        const int w = (int)w_s[oc * KWORDS + i];
#pragma unroll
        for (int px = 0; px < kPix; px++) acc[px] = __dp4a((int)patch[px][i], w, acc[px]);
      }
      const ChanParams cp = a.chan[oc];
#pragma unroll
      for (int px = 0; px < kPix; px++)
      {
        q[px][j] = hi ? requant_cp<true>(acc[px] + cp.bias, cp, a.out_zp, a.clamp_min, a.clamp_max)
                      : requant_cp<false>(acc[px] + cp.bias, cp, a.out_zp, a.clamp_min, a.clamp_max);
        if (a.lut) q[px][j] = __ldg(a.lut + q[px][j] + 128);
      }
    }
#pragma unroll
    for (int px = 0; px < kPix; px++) {
      const long long p = p_base + px * 128;
      if (p >= P) continue;
      int8_t* o = a.out + (size_t)p * a.OC;
      if ((a.OC & 3) == 0) {
        *reinterpret_cast<uint32_t*>(o + oc0) = pack4(q[px][0], q[px][1], q[px][2], q[px][3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; j++)
          if (oc0 + j < a.OC) o[oc0 + j] = (int8_t)q[px][j];
      }
    }
  }
}

// Convolutions over exactly 16 input channels (the first stages of detector backbones: large
// frames, few channels). A tap of one pixel is one 16-byte load; a thread gathers the TAPS taps
// of its output pixel once (input zero point for taps outside the frame) and runs them against
// every output channel's weights, broadcast from shared memory: 4 dp4a per tap and channel.
// Weight rows are Kpad bytes apart (K = TAPS * 16 is a multiple of 16, Kpad of 32).
template <int TAPS>
__global__ void __launch_bounds__(128) conv2d_c16_kernel(ConvArgs a) {
  grid_dependency_release();
  grid_dependency_wait();
  extern __shared__ uint4 w16[];  // [OC][TAPS]
  for (int i = threadIdx.x; i < a.OC * TAPS; i += blockDim.x) {
    const int oc = i / TAPS, t = i - oc * TAPS;
    w16[i] = *reinterpret_cast<const uint4*>(a.w + (size_t)oc * a.Kpad + t * 16);
  }
  __syncthreads();
  const long long P = (long long)a.N * a.OH * a.OW;
  const long long p = (long long)blockIdx.x * 128 + threadIdx.x;
  if (p >= P) return;
  const int ow = (int)(p % a.OW);
  const long long t0 = p / a.OW;
  const int oh = (int)(t0 % a.OH), n = (int)(t0 / a.OH);
  const int ih0 = oh * a.stride_h - a.pad_t, iw0 = ow * a.stride_w - a.pad_l;
  const int8_t* xin = a.x + (size_t)n * a.H * a.W * 16;
  const uint32_t zw = (uint32_t)(a.input_zp & 0xff) * 0x01010101u;
  uint4 tap[TAPS];
#pragma unroll
  for (int t = 0; t < TAPS; t++) {
    const int kh = t / a.KW, kw = t - kh * a.KW;
    const int ih = ih0 + kh * a.dil_h, iw = iw0 + kw * a.dil_w;
    tap[t] = (ih >= 0 && ih < a.H && iw >= 0 && iw < a.W)
                 ? __ldg(reinterpret_cast<const uint4*>(xin + ((size_t)ih * a.W + iw) * 16))
                 : make_uint4(zw, zw, zw, zw);
  }
  const bool hi = a.hi_shift != 0;
  int8_t* o = a.out + (size_t)p * a.OC;
  for (int oc0 = 0; oc0 < a.OC; oc0 += 4) {
    int q[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int oc = min(oc0 + j, a.OC - 1);
      int acc = 0;
#pragma unroll
      for (int t = 0; t < TAPS; t++) {
        const uint4 w = w16[oc * TAPS + t];
        acc = __dp4a((int)tap[t].x, (int)w.x, acc);
        acc = __dp4a((int)tap[t].y, (int)w.y, acc);
        acc = __dp4a((int)tap[t].z, (int)w.z, acc);
        acc = __dp4a((int)tap[t].w, (int)w.w, acc);
      }
      const ChanParams cp = a.chan[oc];
      q[j] = hi ? requant_cp<true>(acc + cp.bias, cp, a.out_zp, a.clamp_min, a.clamp_max)
                : requant_cp<false>(acc + cp.bias, cp, a.out_zp, a.clamp_min, a.clamp_max);
      if (a.lut) q[j] = __ldg(a.lut + q[j] + 128);
    }
    if ((a.OC & 3) == 0) {
      *reinterpret_cast<uint32_t*>(o + oc0) = pack4(q[0], q[1], q[2], q[3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; j++)
        if (oc0 + j < a.OC) o[oc0 + j] = (int8_t)q[j];
    }
  }
}

// raw torq_hl.matmul (tests/testdata/tosa_ops/matmul-in-int8-out-int32.mlir, matmul-in-int16-out-int32.mlir,
// matmul-in-int16-out-int16.mlir): int8 x int8 or int16 x int16, accumulated in int32 with wrap-around, stored as
// int32 or truncated to int16. A block computes a 64 x 64 tile of the result from 64 x 16 / 16 x 64 tiles of the
// operands in shared memory; a thread owns a 4 x 4 patch.
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256) matmul_int_kernel(const TIn* __restrict__ a, const TIn* __restrict__ b,
                                                         TOut* __restrict__ out, int M, int K, int N, int a_zp, int b_zp) {
  __shared__ int sa[16][64 + 1];  // [k][m]
  __shared__ int sb[16][64];      // [k][n]
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  int acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0;
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      const int am = i >> 4, ak = i & 15;  // a: consecutive threads along k
      sa[ak][am] = (m0 + am < M && k0 + ak < K) ? (int)a[(size_t)(m0 + am) * K + k0 + ak] - a_zp : 0;
      const int bk = i >> 6, bn = i & 63;  // b: consecutive threads along n
      sb[bk][bn] = (k0 + bk < K && n0 + bn < N) ? (int)b[(size_t)(k0 + bk) * N + n0 + bn] - b_zp : 0;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; k++) {
      int av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) av[i] = sa[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) bv[j] = sb[k][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] += av[i] * bv[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int m = m0 + ty * 4 + i, n = n0 + tx + 16 * j;
      if (m < M && n < N) out[(size_t)m * N + n] = (TOut)acc[i][j];
    }
}

// The 3x3 window over 3 channels (the stem of an image network) with the compact 32-bit epilogue records. A thread
// owns kStemPix output pixels (adjacent threads adjacent pixels). A kernel row of a pixel is 9 consecutive bytes of
// the input: three aligned words and two funnel shifts bring them in (pixels whose window leaves the image, or whose
// words would reach past the tensor, gather byte by byte with the input zero point outside). The 27 bytes are packed
// into 7 dp4a operands once and run against every output channel's 7 weight words (two 16-byte shared-memory loads
// per channel, shared by the thread's pixels): 7 dp4a + about 7 instructions of rescale per output.
constexpr int kStemPix = 4;
template <int EPI, bool LUT>
__global__ void __launch_bounds__(128) conv2d_stem333_kernel(ConvArgs a) {
  grid_dependency_release();
  grid_dependency_wait();
  extern __shared__ __align__(16) uint32_t stem_s[];  // [OC][8] weight words (word 7 zero), [OC] Q4 records, 256-byte table
  uint4* w_s = reinterpret_cast<uint4*>(stem_s);
  int4* q_s = reinterpret_cast<int4*>(stem_s + (size_t)a.OC * 8);
  const int8_t* lut_s = reinterpret_cast<const int8_t*>(stem_s + (size_t)a.OC * 12);
  if (LUT)
    for (int i = threadIdx.x; i < 256; i += blockDim.x) reinterpret_cast<int8_t*>(stem_s + (size_t)a.OC * 12)[i] = a.lut[i];
  for (int i = threadIdx.x; i < a.OC * 8; i += blockDim.x) {
    const int oc = i >> 3, kw = i & 7;
    stem_s[i] = kw < 7 ? *reinterpret_cast<const uint32_t*>(a.w + (size_t)oc * a.Kpad + kw * 4) : 0u;
  }
  for (int i = threadIdx.x; i < a.OC; i += blockDim.x) q_s[i] = a.q4[i];
  __syncthreads();
  const long long P = (long long)a.N * a.OH * a.OW;
  const long long p_base = (long long)blockIdx.x * (128 * kStemPix) + threadIdx.x;
  const uint32_t zp_byte = (uint32_t)(a.input_zp & 0xff);
  uint32_t patch[kStemPix][7];
#pragma unroll
  for (int px = 0; px < kStemPix; px++) {
    const long long p = p_base + px * 128;
    const long long pp = p < P ? p : 0;
    const int ow = (int)(pp % a.OW);
    const long long t = pp / a.OW;
    const int oh = (int)(t % a.OH);
    const int n = (int)(t / a.OH);
    const int ih0 = oh * a.stride_h - a.pad_t, iw0 = ow * a.stride_w - a.pad_l;
    uint32_t row[3][3];  // per kernel row: bytes 0-3, 4-7, 8 (upper bytes of the third word are not used)
    const long long off0 = (((long long)n * a.H + ih0) * a.W + iw0) * 3;
    const bool inside = ih0 >= 0 && ih0 + 2 < a.H && iw0 >= 0 && iw0 + 2 < a.W &&
                        ((off0 + 2ll * a.W * 3) & ~3ll) + 12 <= a.x_bytes;
    if (inside) {
#pragma unroll
      for (int kh = 0; kh < 3; kh++) {
        const long long off = off0 + (long long)kh * a.W * 3;
        const uint32_t* wp = reinterpret_cast<const uint32_t*>(a.x + (off & ~3ll));
        const uint32_t w0 = __ldg(wp), w1 = __ldg(wp + 1), w2 = __ldg(wp + 2);
        const uint32_t sh = (uint32_t)(off & 3) * 8;
        row[kh][0] = __funnelshift_r(w0, w1, sh);
        row[kh][1] = __funnelshift_r(w1, w2, sh);
        row[kh][2] = w2 >> sh;
      }
    } else {
      const int8_t* xin = a.x + (size_t)n * a.H * a.W * 3;
#pragma unroll
      for (int kh = 0; kh < 3; kh++) {
        const int ih = ih0 + kh;
        uint32_t b[12];
#pragma unroll
        for (int j = 0; j < 9; j++) {
          const int iw = iw0 + j / 3;
          b[j] = (ih >= 0 && ih < a.H && iw >= 0 && iw < a.W) ? (uint32_t)(uint8_t)xin[((size_t)ih * a.W + iw) * 3 + j % 3] : zp_byte;
        }
        row[kh][0] = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
        row[kh][1] = b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24);
        row[kh][2] = b[8];
      }
    }
    // K order (kh, kw, ic): bytes 0-8 row 0, 9-17 row 1, 18-26 row 2, byte 27 meets a zero weight
    patch[px][0] = row[0][0];
    patch[px][1] = row[0][1];
    patch[px][2] = (row[0][2] & 0xffu) | (row[1][0] << 8);
    patch[px][3] = __funnelshift_r(row[1][0], row[1][1], 24);
    patch[px][4] = (row[1][1] >> 24) | ((row[1][2] & 0xffu) << 8) | (row[2][0] << 16);
    patch[px][5] = __funnelshift_r(row[2][0], row[2][1], 16);
    patch[px][6] = (row[2][1] >> 16) | ((row[2][2] & 0xffu) << 16);
  }
  for (int oc0 = 0; oc0 < a.OC; oc0 += 16) {
    uint32_t packed[kStemPix][4];
#pragma unroll
    for (int g = 0; g < 4; g++) {
      int q[kStemPix][4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int oc = min(oc0 + 4 * g + j, a.OC - 1);
        const uint4 wa = w_s[oc * 2], wb = w_s[oc * 2 + 1];
        const int4 c = q_s[oc];
#pragma unroll
        for (int px = 0; px < kStemPix; px++) {
          int acc = __dp4a((int)patch[px][0], (int)wa.x, 0);
          acc = __dp4a((int)patch[px][1], (int)wa.y, acc);
          acc = __dp4a((int)patch[px][2], (int)wa.z, acc);
          acc = __dp4a((int)patch[px][3], (int)wa.w, acc);
          acc = __dp4a((int)patch[px][4], (int)wb.x, acc);
          acc = __dp4a((int)patch[px][5], (int)wb.y, acc);
          acc = __dp4a((int)patch[px][6], (int)wb.z, acc);
          const int r = EPI == 1 ? scale_q4_sign(acc, c) : scale_q4(acc, c);
          q[px][j] = max(a.clamp_min, min(a.clamp_max, r));
          if (LUT) q[px][j] = lut_s[q[px][j] + 128];  // a fused 256-entry table
        }
      }
#pragma unroll
      for (int px = 0; px < kStemPix; px++) packed[px][g] = pack4(q[px][0], q[px][1], q[px][2], q[px][3]);
    }
#pragma unroll
    for (int px = 0; px < kStemPix; px++) {
      const long long p = p_base + px * 128;
      if (p >= P) continue;
      *reinterpret_cast<uint4*>(a.out + (size_t)p * a.OC + oc0) = make_uint4(packed[px][0], packed[px][1], packed[px][2], packed[px][3]);
    }
  }
}

// FullyConnected on at most MR rows: one warp per output channel. The row(s) of x sit in shared memory (K bytes each);
// a lane takes 16 weights per step with one 16-byte load and runs them against the staged activations with dp4a;
// the warp adds its lanes' sums and lane 0 applies the exact rescale. Weights are read once, coalesced: HBM-bound.
template <int MR>
__global__ void __launch_bounds__(256) fc_rows_kernel(FcRowsArgs a) {
  extern __shared__ __align__(16) int8_t fc_x[];  // [MR][K]
  for (int i = threadIdx.x * 16; i < MR * a.K; i += blockDim.x * 16) {
    const int m = i / a.K, k = i - m * a.K;
    *reinterpret_cast<uint4*>(fc_x + i) = m < a.M ? *reinterpret_cast<const uint4*>(a.x + (size_t)m * a.K + k) : make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  if (n >= a.N) return;
  const int8_t* wrow = a.w + (size_t)n * a.K;
  int acc[MR];
#pragma unroll
  for (int m = 0; m < MR; m++) acc[m] = 0;
#pragma unroll 4
  for (int k = lane * 16; k < a.K; k += 32 * 16) {
    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wrow + k));
#pragma unroll
    for (int m = 0; m < MR; m++) {
      const uint4 xv = *reinterpret_cast<const uint4*>(fc_x + m * a.K + k);
      acc[m] = __dp4a((int)xv.x, (int)wv.x, acc[m]);
      acc[m] = __dp4a((int)xv.y, (int)wv.y, acc[m]);
      acc[m] = __dp4a((int)xv.z, (int)wv.z, acc[m]);
      acc[m] = __dp4a((int)xv.w, (int)wv.w, acc[m]);
    }
  }
#pragma unroll
  for (int m = 0; m < MR; m++)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
  if (lane == 0) {
    const ChanParams cp = a.chan[n];
#pragma unroll
    for (int m = 0; m < MR; m++)
      if (m < a.M) {
        int q = a.hi_shift ? requant_cp<true>(acc[m] + cp.bias, cp, a.out_zp, a.clamp_min, a.clamp_max)
                           : requant_cp<false>(acc[m] + cp.bias, cp, a.out_zp, a.clamp_min, a.clamp_max);
        if (a.lut) q = __ldg(a.lut + q + 128);
        a.out[(size_t)m * a.N + n] = (int8_t)q;
      }
  }
}

// Conv2D i16 x i8 (TB200_OP_CONV2D_I16): one thread per output; consecutive threads take consecutive output channels
// of a pixel, so the pixel's input window is read by the whole group and the weights stream per thread. 64-bit
// accumulation (TOSA's 48-bit accumulator never leaves it), then apply_scale_16:
// (acc * multiplier + 2^(shift-1)) >> shift, + out_zp, clamp, int16.
__global__ void __launch_bounds__(256) conv2d_i16_kernel(ConvI16Args a) {
  const long long total = (long long)a.N * a.OH * a.OW * a.OC;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int oc = (int)(idx % a.OC);
  long long p = idx / a.OC;
  const int ow = (int)(p % a.OW);
  p /= a.OW;
  const int oh = (int)(p % a.OH);
  const int n = (int)(p / a.OH);
  long long acc = a.bias[oc];
  const int8_t* wrow = a.w + (size_t)oc * a.KH * a.KW * a.IC;
  for (int kh = 0; kh < a.KH; kh++) {
    const int ih = oh * a.stride_h - a.pad_t + kh * a.dil_h;
    if (ih < 0 || ih >= a.H) continue;
    for (int kw = 0; kw < a.KW; kw++) {
      const int iw = ow * a.stride_w - a.pad_l + kw * a.dil_w;
      if (iw < 0 || iw >= a.W) continue;
      const int16_t* px = a.x + (((size_t)n * a.H + ih) * a.W + iw) * a.IC;
      const int8_t* wt = wrow + ((size_t)kh * a.KW + kw) * a.IC;
      int part = 0;  // |(x - zp) * (w - wzp)| < 2^16 * 2^8: 64 terms fit in 31 bits
      for (int c = 0; c < a.IC; c++) {
        part += ((int)px[c] - a.input_zp) * ((int)wt[c] - a.weight_zp);
        if ((c & 63) == 63) {
          acc += part;
          part = 0;
        }
      }
      acc += part;
    }
  }
  const int sh = a.shift[oc];
  long long r = ((acc * (long long)a.mult[oc] + (1ll << (sh - 1))) >> sh) + a.out_zp;
  r = r < a.clamp_min ? a.clamp_min : (r > a.clamp_max ? a.clamp_max : r);
  a.out[idx] = (int16_t)r;
}

}  // namespace

static bool conv_c16_applies(const ConvArgs& a) {
  const int taps = a.KH * a.KW;
  return a.IC == 16 && a.weight_zp == 0 && a.OC <= 256 && (taps == 9 || taps == 1 || taps == 25);
}

// the 3x3x3 stem with 32-bit epilogue records, output channels in whole 16-byte groups
static bool conv_stem333_shape(const ConvArgs& a) {
  return a.IC == 3 && a.KH == 3 && a.KW == 3 && a.dil_h == 1 && a.dil_w == 1 && a.weight_zp == 0 && a.epi != 0 &&
         (a.OC & 15) == 0 && a.OC <= 256;
}
static bool conv_stem333_applies(const ConvArgs& a) {
  return conv_stem333_shape(a) && a.q4 && ((uintptr_t)a.x & 3) == 0 && ((uintptr_t)a.out & 15) == 0;
}

const char* conv2d_simt_kernel_name(const ConvArgs& a) {
  if (conv_c16_applies(a)) return "conv2d_c16_dp4a";
  if (conv_stem333_shape(a)) return "conv2d_stem333_dp4a";
  return (a.IC <= 4 && a.K <= 64 && a.OC <= 256 && a.weight_zp == 0) ? "conv2d_smallic_dp4a" : "conv2d_simt";
}

void launch_conv2d_simt(const ConvArgs& a, cudaStream_t stream) {
  long long P = (long long)a.N * a.OH * a.OW;
  if (conv_c16_applies(a)) {
    const unsigned blocks = (unsigned)((P + 127) / 128);
    const int taps = a.KH * a.KW;
    const size_t smem = (size_t)a.OC * taps * 16;
    if (taps == 9) {
      launch_dependent(conv2d_c16_kernel<9>, dim3(blocks), dim3(128), smem, stream, a);
    } else if (taps == 1) {
      launch_dependent(conv2d_c16_kernel<1>, dim3(blocks), dim3(128), smem, stream, a);
    } else {
      static std::atomic<unsigned long long> attr{0};  // function attributes are per device
      if (first_use_on_device(attr)) {
        cudaFuncSetAttribute(conv2d_c16_kernel<25>, cudaFuncAttributeMaxDynamicSharedMemorySize, 256 * 25 * 16);
        mark_used_on_device(attr);
      }
      launch_dependent(conv2d_c16_kernel<25>, dim3(blocks), dim3(128), smem, stream, a);
    }
    return;
  }
  if (conv_stem333_applies(a)) {
    const unsigned blocks = (unsigned)((P + 128 * kStemPix - 1) / (128 * kStemPix));
    const size_t smem = (size_t)a.OC * (32 + 16) + 256;
    if (a.lut) {
      if (a.epi == 1) launch_dependent(conv2d_stem333_kernel<1, true>, dim3(blocks), dim3(128), smem, stream, a);
      else launch_dependent(conv2d_stem333_kernel<2, true>, dim3(blocks), dim3(128), smem, stream, a);
    } else {
      if (a.epi == 1) launch_dependent(conv2d_stem333_kernel<1, false>, dim3(blocks), dim3(128), smem, stream, a);
      else launch_dependent(conv2d_stem333_kernel<2, false>, dim3(blocks), dim3(128), smem, stream, a);
    }
    return;
  }
  if (a.IC <= 4 && a.K <= 64 && a.OC <= 256 && a.weight_zp == 0) {
    const unsigned blocks = (unsigned)((P + 128 * kPix - 1) / (128 * kPix));
    const int kwords = (a.K + 3) / 4;
    if (a.IC == 3 && a.KH == 3 && a.KW == 3)
      conv2d_smallic_kernel<7, true><<<blocks, 128, (size_t)a.OC * 7 * 4, stream>>>(a);
    else if (kwords <= 3) conv2d_smallic_kernel<3, false><<<blocks, 128, (size_t)a.OC * 3 * 4, stream>>>(a);
    else if (kwords <= 7) conv2d_smallic_kernel<7, false><<<blocks, 128, (size_t)a.OC * 7 * 4, stream>>>(a);
    else if (kwords <= 9) conv2d_smallic_kernel<9, false><<<blocks, 128, (size_t)a.OC * 9 * 4, stream>>>(a);
    else conv2d_smallic_kernel<16, false><<<blocks, 128, (size_t)a.OC * 16 * 4, stream>>>(a);
    return;
  }
  dim3 grid((unsigned)((P + BM - 1) / BM), (unsigned)((a.OC + BN - 1) / BN));
  if ((a.IC & 3) == 0)
    conv2d_simt_kernel<true><<<grid, 256, 0, stream>>>(a);
  else
    conv2d_simt_kernel<false><<<grid, 256, 0, stream>>>(a);
}

void launch_fc_rows(const FcRowsArgs& a, cudaStream_t stream) {
  const unsigned blocks = (unsigned)((a.N + 7) / 8);
  if (a.M <= 1) fc_rows_kernel<1><<<blocks, 256, (size_t)a.K, stream>>>(a);
  else if (a.M <= 2) fc_rows_kernel<2><<<blocks, 256, (size_t)2 * a.K, stream>>>(a);
  else fc_rows_kernel<4><<<blocks, 256, (size_t)4 * a.K, stream>>>(a);
}

void launch_conv2d_i16(const ConvI16Args& a, cudaStream_t stream) {
  const long long total = (long long)a.N * a.OH * a.OW * a.OC;
  conv2d_i16_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(a);
}

void launch_matmul_int(const void* a, const void* b, void* out, bool in_i16, bool out_i16, int M, int K, int N, int a_zp,
                       int b_zp, cudaStream_t stream) {
  const dim3 grid((N + 63) / 64, (M + 63) / 64);
  if (!in_i16 && !out_i16)
    matmul_int_kernel<int8_t, int32_t><<<grid, 256, 0, stream>>>((const int8_t*)a, (const int8_t*)b, (int32_t*)out, M, K, N, a_zp, b_zp);
  else if (!in_i16)
    matmul_int_kernel<int8_t, int16_t><<<grid, 256, 0, stream>>>((const int8_t*)a, (const int8_t*)b, (int16_t*)out, M, K, N, a_zp, b_zp);
  else if (!out_i16)
    matmul_int_kernel<int16_t, int32_t><<<grid, 256, 0, stream>>>((const int16_t*)a, (const int16_t*)b, (int32_t*)out, M, K, N, a_zp, b_zp);
  else
    matmul_int_kernel<int16_t, int16_t><<<grid, 256, 0, stream>>>((const int16_t*)a, (const int16_t*)b, (int16_t*)out, M, K, N, a_zp, b_zp);
}

}  // namespace tb200
