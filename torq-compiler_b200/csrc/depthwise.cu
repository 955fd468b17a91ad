// Depthwise convolution (torq_hl.depthwise_conv2d,
// compiler/torq/Conversions/LinalgToTorqHL/Conv2DPattern.cpp:627-637; TOSA weights [KH,KW,C,M]).
//
// Two kernels with identical results:
//  * dw3x3_kernel: the 3x3 / stride 1-2 / M == 1 / C % 4 == 0 case that MobileNet-style
//    networks spend their depthwise time in. Each thread owns 4 channels and a column
//    strip; per input row it loads 4 (stride 1) or 3 (stride 2) neighbouring pixels,
//    transposes the 4x4 byte block with PRMT so that a register holds one channel's
//    horizontal taps, and feeds dp4a with weights packed (w0,w1,w2,0) / (0,w0,w1,w2):
//    one transposed register serves two adjacent outputs. Rows roll through a 3-row
//    register window, so every input row is loaded and transposed once per strip.
//    Taps outside the image are staged as izp, i.e. (izp - izp) * w = 0, and
//    -izp * sum(w) sits folded in ChanParams::bias.
//  * depthwise_generic_kernel: any window, stride, dilation, channel multiplier and
//    weight zero point; taps outside the image are skipped.
#include "kernels.h"

namespace tb200 {

namespace {

constexpr int kRows = 8;  // output rows per thread in the 3x3 kernel

// out[c] = bytes (p0.c, p1.c, p2.c, p3.c)
__device__ __forceinline__ void transpose4x4(uint32_t p0, uint32_t p1, uint32_t p2, uint32_t p3, uint32_t (&t)[4]) {
  uint32_t a = __byte_perm(p0, p1, 0x5140), b = __byte_perm(p0, p1, 0x7362);
  uint32_t c = __byte_perm(p2, p3, 0x5140), d = __byte_perm(p2, p3, 0x7362);
  t[0] = __byte_perm(a, c, 0x5410);
  t[1] = __byte_perm(a, c, 0x7632);
  t[2] = __byte_perm(b, d, 0x5410);
  t[3] = __byte_perm(b, d, 0x7632);
}

// HI33: every rescale shift of the op is >= 33 (compact constants, see gemm_tcgen05.cu).
template <int STRIDE, bool HI33>
__global__ void __launch_bounds__(128, 5) dw3x3_kernel(DwArgs a) {
  constexpr int TW = STRIDE == 1 ? 2 : 1;    // outputs per thread along W
  constexpr int NCOL = STRIDE == 1 ? 4 : 3;  // input columns per row load
  const int groups = a.C >> 2;
  const int owt = (a.OW + TW - 1) / TW;
  const int ohb = (a.OH + kRows - 1) / kRows;
  const long long total = (long long)a.N * ohb * owt * groups;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int g = (int)(idx % groups);
  long long r0 = idx / groups;
  const int j = (int)(r0 % owt);
  r0 /= owt;
  const int rb = (int)(r0 % ohb);
  const int n = (int)(r0 / ohb);
  const int c = g * 4;
  const int ow0 = j * TW;
  const int iw0 = ow0 * STRIDE - a.pad_l;
  const int oh_begin = rb * kRows;
  const int oh_end = min(a.OH, oh_begin + kRows);
  const int8_t* xin = a.x + (size_t)n * a.H * a.W * a.C + c;
  const uint32_t zpw = (uint32_t)(a.input_zp & 0xff) * 0x01010101u;
  const uint32_t lo2 = (uint32_t)(a.clamp_min & 0xffff) * 0x10001u;
  const uint32_t hi2 = (uint32_t)(a.clamp_max & 0xffff) * 0x10001u;

  // weights: [3 rows][TW variants][C] words, this thread's 4 channels
  uint32_t wq[3][TW][4];
#pragma unroll
  for (int kh = 0; kh < 3; kh++)
#pragma unroll
    for (int v = 0; v < TW; v++) {
      uint4 w = *reinterpret_cast<const uint4*>(a.wq + ((size_t)(kh * TW + v) * a.C + c));
      wq[kh][v][0] = w.x; wq[kh][v][1] = w.y; wq[kh][v][2] = w.z; wq[kh][v][3] = w.w;
    }
  // per-channel constants: {bias, mult, high word of rnd, shift - 32} (HI33) or the full record
  int4 cq[4];
  ChanParams cp[HI33 ? 1 : 4];
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const ChanParams t = a.chan[c + k];
    if (HI33) cq[k] = make_int4(t.bias, t.mult, (int)(t.rnd >> 32), t.hshift);
    else cp[k] = t;
  }

  // raw pixel words of one input row (izp for anything outside the image)
  auto fetch_row = [&](int ih, uint32_t (&p)[4]) {
    const bool row_in = ih >= 0 && ih < a.H;
    const int8_t* row = xin + (size_t)(row_in ? ih : 0) * a.W * a.C;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int iw = iw0 + k;
      p[k] = (k < NCOL && row_in && iw >= 0 && iw < a.W) ? *reinterpret_cast<const uint32_t*>(row + (size_t)iw * a.C) : zpw;
    }
  };

  uint32_t win[3][4];
  uint32_t pend[2][4];  // rows fetched ahead of their use (1 for stride 1, 2 for stride 2)
  {
    uint32_t p[4];
    if (STRIDE == 1) {
      fetch_row(oh_begin - a.pad_t, p);
      transpose4x4(p[0], p[1], p[2], p[3], win[0]);
      fetch_row(oh_begin - a.pad_t + 1, p);
      transpose4x4(p[0], p[1], p[2], p[3], win[1]);
      fetch_row(oh_begin - a.pad_t + 2, pend[0]);
    } else {
      fetch_row(oh_begin * 2 - a.pad_t, p);
      transpose4x4(p[0], p[1], p[2], p[3], win[0]);
      fetch_row(oh_begin * 2 - a.pad_t + 1, pend[0]);
      fetch_row(oh_begin * 2 - a.pad_t + 2, pend[1]);
    }
  }
  for (int oh = oh_begin; oh < oh_end; oh++) {
    const int ih0 = oh * STRIDE - a.pad_t;
    // consume the rows fetched during the previous iteration, then fetch the next ones
    if (STRIDE == 1) {
      transpose4x4(pend[0][0], pend[0][1], pend[0][2], pend[0][3], win[2]);
      if (oh + 1 < oh_end) fetch_row(ih0 + 3, pend[0]);
    } else {
      transpose4x4(pend[0][0], pend[0][1], pend[0][2], pend[0][3], win[1]);
      transpose4x4(pend[1][0], pend[1][1], pend[1][2], pend[1][3], win[2]);
      if (oh + 1 < oh_end) {
        fetch_row(ih0 + 3, pend[0]);
        fetch_row(ih0 + 4, pend[1]);
      }
    }
    int8_t* orow = a.out + (((size_t)n * a.OH + oh) * a.OW + ow0) * a.C + c;
#pragma unroll
    for (int v = 0; v < TW; v++) {
      if (ow0 + v >= a.OW) break;
      int q[4];
#pragma unroll
      for (int k = 0; k < 4; k++) {
        int acc = HI33 ? cq[k].x : cp[k].bias;
#pragma unroll
        for (int kh = 0; kh < 3; kh++) acc = __dp4a((int)win[kh][k], (int)wq[kh][v][k], acc);
        if (HI33) {
          long long tt = (long long)acc * (long long)cq[k].y + (((long long)cq[k].z << 32) | (long long)(uint32_t)a.rnd_lo);
          tt += (long long)(int32_t)((uint32_t)acc >> 31) * (long long)a.dmul;
          q[k] = ((int32_t)(tt >> 32) >> cq[k].w) + a.out_zp;
        } else {
          q[k] = scale_cp<false>(acc, cp[k]) + a.out_zp;
        }
      }
      *reinterpret_cast<uint32_t*>(orow + (size_t)v * a.C) = clamp_pack4(q[0], q[1], q[2], q[3], lo2, hi2);
    }
    // roll the window
    if (STRIDE == 1) {
#pragma unroll
      for (int k = 0; k < 4; k++) {
        win[0][k] = win[1][k];
        win[1][k] = win[2][k];
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; k++) win[0][k] = win[2][k];
    }
  }
}

// One thread per (output pixel, VEC consecutive channels); taps outside the image are skipped.
template <int VEC>
__global__ void __launch_bounds__(256) depthwise_generic_kernel(DwArgs a) {
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
  const bool hi = a.hi_shift != 0;

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
      q[j] = hi ? requant_cp<true>(acc[j] + cp.bias, cp, a.out_zp, a.clamp_min, a.clamp_max)
                : requant_cp<false>(acc[j] + cp.bias, cp, a.out_zp, a.clamp_min, a.clamp_max);
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
    a.out[(size_t)p * OC + oc] = (int8_t)(hi ? requant_cp<true>(acc + cp.bias, cp, a.out_zp, a.clamp_min, a.clamp_max)
                                             : requant_cp<false>(acc + cp.bias, cp, a.out_zp, a.clamp_min, a.clamp_max));
  }
}

}  // namespace

bool depthwise3x3_supported(const DwArgs& a) {
  return a.KH == 3 && a.KW == 3 && a.M == 1 && (a.C & 3) == 0 && a.dil_h == 1 && a.dil_w == 1 &&
         a.stride_h == a.stride_w && (a.stride_h == 1 || a.stride_h == 2) && a.weight_zp == 0;
}

size_t depthwise3x3_pack(const int8_t* w, int C, int stride, uint32_t* out) {
  const int variants = stride == 1 ? 2 : 1;
  for (int kh = 0; kh < 3; kh++)
    for (int v = 0; v < variants; v++)
      for (int c = 0; c < C; c++) {
        uint32_t b[4] = {0, 0, 0, 0};
        for (int kw = 0; kw < 3; kw++) b[kw + v] = (uint8_t)w[((size_t)kh * 3 + kw) * C + c];
        out[((size_t)(kh * variants + v)) * C + c] = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
      }
  return (size_t)3 * variants * C;
}

void launch_depthwise(const DwArgs& a, cudaStream_t stream) {
  if (a.wq && depthwise3x3_supported(a)) {
    const int tw = a.stride_h == 1 ? 2 : 1;
    long long total = (long long)a.N * ((a.OH + kRows - 1) / kRows) * ((a.OW + tw - 1) / tw) * (a.C >> 2);
    unsigned blocks = (unsigned)((total + 127) / 128);
    if (a.stride_h == 1) {
      if (a.hi33) dw3x3_kernel<1, true><<<blocks, 128, 0, stream>>>(a);
      else dw3x3_kernel<1, false><<<blocks, 128, 0, stream>>>(a);
    } else {
      if (a.hi33) dw3x3_kernel<2, true><<<blocks, 128, 0, stream>>>(a);
      else dw3x3_kernel<2, false><<<blocks, 128, 0, stream>>>(a);
    }
  } else if (a.M == 1 && (a.C & 3) == 0) {
    long long total = (long long)a.N * a.OH * a.OW * (a.C >> 2);
    depthwise_generic_kernel<4><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(a);
  } else {
    long long total = (long long)a.N * a.OH * a.OW * a.C * a.M;
    depthwise_generic_kernel<1><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(a);
  }
}

}  // namespace tb200
