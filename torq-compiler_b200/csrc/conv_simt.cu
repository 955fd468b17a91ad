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
    else cp[j] = ChanParams{0, 0, 2, 0};
  }
  const bool dr = a.double_round != 0;
  const bool vec_ok = ((a.OC & 3) == 0) && (oc0 + 3 < a.OC);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    long long p = p_base + tx + 16 * i;
    if (p >= P) continue;
    int q[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int v = acc[i][j] - a.weight_zp * xsum[i] + cp[j].bias;
      q[j] = requant(v, cp[j].mult, cp[j].shift, dr, a.out_zp, a.clamp_min, a.clamp_max);
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

// Depthwise: one thread per (output pixel, VEC consecutive channels).
// torq_hl.depthwise_conv2d (Conv2DPattern.cpp:627-637), weights [KH,KW,C,M].
// Taps outside the image are skipped (they would contribute (izp - izp) * w).
template <int VEC>
__global__ void __launch_bounds__(256) depthwise_kernel(DwArgs a) {
  const int OC = a.C * a.M;
  const int groups = (VEC == 4) ? (a.C >> 2) : OC;
  const long long total = (long long)a.N * a.OH * a.OW * groups;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  int g = (int)(idx % groups);
  long long p = idx / groups;
  int ow = (int)(p % a.OW);
  long long t = p / a.OW;
  int oh = (int)(t % a.OH);
  int n = (int)(t / a.OH);
  const int ih0 = oh * a.stride_h - a.pad_t;
  const int iw0 = ow * a.stride_w - a.pad_l;
  const int8_t* xin = a.x + (size_t)n * a.H * a.W * a.C;
  const bool dr = a.double_round != 0;

  if (VEC == 4) {
    const int c = g * 4;
    int acc[4] = {0, 0, 0, 0};
    for (int kh = 0; kh < a.KH; kh++) {
      int ih = ih0 + kh * a.dil_h;
      if (ih < 0 || ih >= a.H) continue;
      for (int kw = 0; kw < a.KW; kw++) {
        int iw = iw0 + kw * a.dil_w;
        if (iw < 0 || iw >= a.W) continue;
        uint32_t xv = *reinterpret_cast<const uint32_t*>(xin + ((size_t)ih * a.W + iw) * a.C + c);
        uint32_t wv = *reinterpret_cast<const uint32_t*>(a.w + ((size_t)kh * a.KW + kw) * a.C + c);
#pragma unroll
        for (int j = 0; j < 4; j++) acc[j] += (sx8(xv, j) - a.input_zp) * (sx8(wv, j) - a.weight_zp);
      }
    }
    int q[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      ChanParams cp = a.chan[c + j];
      q[j] = requant(acc[j] + cp.bias, cp.mult, cp.shift, dr, a.out_zp, a.clamp_min, a.clamp_max);
    }
    *reinterpret_cast<uint32_t*>(a.out + (size_t)p * OC + c) = pack4(q[0], q[1], q[2], q[3]);
  } else {
    const int oc = g;
    const int c = oc / a.M;
    const int m = oc - c * a.M;
    int acc = 0;
    for (int kh = 0; kh < a.KH; kh++) {
      int ih = ih0 + kh * a.dil_h;
      if (ih < 0 || ih >= a.H) continue;
      for (int kw = 0; kw < a.KW; kw++) {
        int iw = iw0 + kw * a.dil_w;
        if (iw < 0 || iw >= a.W) continue;
        int xv = xin[((size_t)ih * a.W + iw) * a.C + c];
        int wv = a.w[(((size_t)kh * a.KW + kw) * a.C + c) * a.M + m];
        acc += (xv - a.input_zp) * (wv - a.weight_zp);
      }
    }
    ChanParams cp = a.chan[oc];
    a.out[(size_t)p * OC + oc] =
        (int8_t)requant(acc + cp.bias, cp.mult, cp.shift, dr, a.out_zp, a.clamp_min, a.clamp_max);
  }
}

// raw torq_hl.matmul, int32 result (tests/testdata/tosa_ops/matmul-in-int8-out-int32.mlir).
__global__ void __launch_bounds__(256) matmul_i32_kernel(const int8_t* __restrict__ a,
                                                         const int8_t* __restrict__ b,
                                                         int32_t* __restrict__ out, int M, int K, int N,
                                                         int a_zp, int b_zp) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)M * N) return;
  int n = (int)(idx % N);
  int m = (int)(idx / N);
  int acc = 0;
  for (int k = 0; k < K; k++) acc += ((int)a[(size_t)m * K + k] - a_zp) * ((int)b[(size_t)k * N + n] - b_zp);
  out[idx] = acc;
}

}  // namespace

void launch_conv2d_simt(const ConvArgs& a, cudaStream_t stream) {
  long long P = (long long)a.N * a.OH * a.OW;
  dim3 grid((unsigned)((P + BM - 1) / BM), (unsigned)((a.OC + BN - 1) / BN));
  if ((a.IC & 3) == 0)
    conv2d_simt_kernel<true><<<grid, 256, 0, stream>>>(a);
  else
    conv2d_simt_kernel<false><<<grid, 256, 0, stream>>>(a);
}

void launch_depthwise(const DwArgs& a, cudaStream_t stream) {
  if (a.M == 1 && (a.C & 3) == 0) {
    long long total = (long long)a.N * a.OH * a.OW * (a.C >> 2);
    depthwise_kernel<4><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(a);
  } else {
    long long total = (long long)a.N * a.OH * a.OW * a.C * a.M;
    depthwise_kernel<1><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(a);
  }
}

void launch_matmul_i32(const int8_t* a, const int8_t* b, int32_t* out, int M, int K, int N, int a_zp,
                       int b_zp, cudaStream_t stream) {
  long long total = (long long)M * N;
  matmul_i32_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(a, b, out, M, K, N, a_zp, b_zp);
}

}  // namespace tb200
