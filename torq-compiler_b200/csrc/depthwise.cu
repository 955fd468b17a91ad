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
//    register window (fully unrolled, so the roll is register renaming); all rows of a strip
//    are requested up front with cp.async into per-thread shared-memory slots, so every
//    input row is loaded and transposed once per strip with its latency hidden.
//    Taps outside the image are staged as izp, i.e. (izp - izp) * w = 0, and
//    -izp * sum(w) sits folded in ChanParams::bias.
//  * depthwise_generic_kernel: any window, stride, dilation, channel multiplier and
//    weight zero point; taps outside the image are skipped.
#include <cstdlib>

#include "kernels.h"
#include "dependent_launch.cuh"

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

// cp.async.wait_group takes an immediate; in the unrolled loops the argument is a constant
// and the switch folds to a single instruction.
__device__ __forceinline__ void cp_async_wait(int n) {
  switch (n) {
#define TB200_CASE(N) case N: asm volatile("cp.async.wait_group " #N ";" ::: "memory"); break;
    TB200_CASE(0) TB200_CASE(1) TB200_CASE(2) TB200_CASE(3) TB200_CASE(4) TB200_CASE(5) TB200_CASE(6)
    TB200_CASE(7) TB200_CASE(8) TB200_CASE(9) TB200_CASE(10) TB200_CASE(11) TB200_CASE(12) TB200_CASE(13)
    TB200_CASE(14) TB200_CASE(15) TB200_CASE(16)
#undef TB200_CASE
    default: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
  }
}

// EPI: 0 = rescale from the full ChanParams record; 1 / 2 = compact Q4 records with / without the sign term
// (common.cuh), four of them held in registers per thread.
// All addressing is 32-bit element offsets from the tensor bases (the launcher checks that
// both tensors are below 2 GiB), so a load costs one add and a predicated LDG.
template <int STRIDE, int EPI>
__global__ void __launch_bounds__(128, 4) dw3x3_kernel(DwArgs a) {
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
  const int n_rows = min(a.OH - oh_begin, kRows);
  const uint32_t zpw = (uint32_t)(a.input_zp & 0xff) * 0x01010101u;
  const uint32_t lo2 = (uint32_t)(a.clamp_min & 0xffff) * 0x10001u;
  const uint32_t hi2 = (uint32_t)(a.clamp_max & 0xffff) * 0x10001u;
  const uint32_t* __restrict__ x32 = reinterpret_cast<const uint32_t*>(a.x);
  uint32_t* __restrict__ o32 = reinterpret_cast<uint32_t*>(a.out);
  const int Cw = a.C >> 2;  // words per pixel

  // weights: [3 rows][TW variants][C] words, this thread's 4 channels
  uint32_t wq[3][TW][4];
#pragma unroll
  for (int kh = 0; kh < 3; kh++)
#pragma unroll
    for (int v = 0; v < TW; v++) {
      uint4 w = *reinterpret_cast<const uint4*>(a.wq + ((size_t)(kh * TW + v) * a.C + c));
      wq[kh][v][0] = w.x; wq[kh][v][1] = w.y; wq[kh][v][2] = w.z; wq[kh][v][3] = w.w;
    }
  // per-channel constants: the Q4 record or the full record
  int4 cq[4];
  ChanParams cp[EPI != 0 ? 1 : 4];
#pragma unroll
  for (int k = 0; k < 4; k++) {
    if (EPI != 0) cq[k] = __ldg(a.q4 + c + k);
    else cp[k] = a.chan[c + k];
  }

  // column word offsets and validity of the NCOL input columns this strip touches
  int col_off[4];
  bool col_ok[4];
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const int iw = iw0 + k;
    col_ok[k] = k < NCOL && iw >= 0 && iw < a.W;
    col_off[k] = iw * Cw + g;
  }
  const int img_off = n * a.H * a.W * Cw;  // word offset of image n
  const int row_words = a.W * Cw;

  // The strip's input rows R[0..NR): output row r reads R[S*r], R[S*r+1], R[S*r+2]. Every row
  // is requested up front with cp.async into this thread's own shared-memory slots (one
  // commit group per row), so all of a strip's bytes are in flight at once; the loop over
  // output rows is fully unrolled and waits for just the rows it needs.
  constexpr int NR = (kRows - 1) * STRIDE + 3;
  extern __shared__ uint32_t stage[];  // [NR][4][128]
  const uint32_t stage_addr = (uint32_t)__cvta_generic_to_shared(stage) + threadIdx.x * 4;
  const int ih_base = oh_begin * STRIDE - a.pad_t;
  const int nr_live = (n_rows - 1) * STRIDE + 3;  // rows this strip really needs
#pragma unroll
  for (int i = 0; i < NR; i++) {
    const int ih = ih_base + i;
    const bool row_in = i < nr_live && ih >= 0 && ih < a.H;
    const int roff = img_off + ih * row_words;
#pragma unroll
    for (int k = 0; k < NCOL; k++) {
      if (row_in && col_ok[k]) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(stage_addr + (i * 4 + k) * 512),
                     "l"(x32 + (uint32_t)(roff + col_off[k]))
                     : "memory");
      } else {
        stage[(i * 4 + k) * 128 + threadIdx.x] = zpw;
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  auto take_row = [&](int i, uint32_t (&t)[4]) {
    const uint32_t p0 = stage[(i * 4 + 0) * 128 + threadIdx.x], p1 = stage[(i * 4 + 1) * 128 + threadIdx.x],
                   p2 = stage[(i * 4 + 2) * 128 + threadIdx.x];
    const uint32_t p3 = NCOL == 4 ? stage[(i * 4 + 3) * 128 + threadIdx.x] : zpw;
    transpose4x4(p0, p1, p2, p3, t);
  };
  uint32_t win[NR][4];
  int out_off = ((n * a.OH + oh_begin) * a.OW + ow0) * Cw + g;  // word offset of the first output
  const int out_row_words = a.OW * Cw;
  const bool second = TW == 2 && ow0 + 1 < a.OW;
#pragma unroll
  for (int r = 0; r < kRows; r++) {
    if (r < n_rows) {
      // wait for this output row's newest input row (groups complete in order), then transpose
      cp_async_wait(NR - 1 - (STRIDE * r + 2));
      if (r == 0) {
        take_row(0, win[0]);
        take_row(1, win[1]);
        take_row(2, win[2]);
      } else {
#pragma unroll
        for (int i = 0; i < STRIDE; i++) take_row(STRIDE * r + 2 - i, win[STRIDE * r + 2 - i]);
      }
#pragma unroll
      for (int v = 0; v < TW; v++) {
        int q[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
          int acc = EPI != 0 ? 0 : cp[k].bias;
#pragma unroll
          for (int kh = 0; kh < 3; kh++) acc = __dp4a((int)win[STRIDE * r + kh][k], (int)wq[kh][v][k], acc);
          if (EPI == 1) q[k] = scale_q4_sign(acc, cq[k]);
          else if (EPI == 2) q[k] = scale_q4(acc, cq[k]);
          else q[k] = scale_cp<false>(acc, cp[k]) + a.out_zp;
        }
        const uint32_t word = clamp_pack4(q[0], q[1], q[2], q[3], lo2, hi2);
        if (v == 0 || second) o32[(uint32_t)(out_off + v * Cw)] = word;
      }
      out_off += out_row_words;
    }
  }
}

// The same arithmetic with the block's input tile loaded cooperatively (C % 16 == 0): a block is
// CG channel groups (4 channels each, CG*4 a multiple of 16) x SW column strips = 128 threads and owns
// kRows output rows x SW*TW output columns x CG*4 channels. Its input tile [NR rows][IWT columns][CG*4
// bytes] is fetched with 16-byte cp.async by whichever thread the piece falls to (about one piece per
// thread and row instead of four 4-byte copies per thread and row, and no 64-bit index arithmetic per
// thread); pieces outside the image are stored as the input zero point. After one barrier every thread
// reads its own 4 channels of its 3 or 4 columns from the tile and proceeds exactly as dw3x3_kernel.
// ROWS: output rows per thread: 8, or 14 where the frame height is a multiple of 14 (112, 56, 28, 14): the two halo
// rows, the weights and the per-channel records are then paid once per 14 rows instead of once per 8.
template <int STRIDE, int EPI, int ROWS>
__global__ void __launch_bounds__(128, STRIDE == 1 ? 6 : 8) dw3x3_tile_kernel(DwArgs a, int cg_log2, int cchunks) {
  grid_dependency_release();
  grid_dependency_wait();
  constexpr int TW = STRIDE == 1 ? 2 : 1;
  constexpr int NCOL = STRIDE == 1 ? 4 : 3;
  constexpr int NR = (ROWS - 1) * STRIDE + 3;
  extern __shared__ __align__(16) uint32_t tile[];  // [NR][IWT][CG] words
  const int CG = 1 << cg_log2, SW = 128 >> cg_log2;
  const int IWT = (SW * TW - 1) * STRIDE + 3;  // input columns of the tile
  const int gl = threadIdx.x & (CG - 1), strip = threadIdx.x >> cg_log2;
  const int wt = blockIdx.x / cchunks, cc = blockIdx.x - wt * cchunks;
  const int rb = blockIdx.y, n = blockIdx.z;
  const int c0 = cc << (cg_log2 + 2);        // first channel of the block
  const int ow_tile = wt * SW * TW;          // first output column of the block
  const int iw_tile = ow_tile * STRIDE - a.pad_l;
  const int oh_begin = rb * ROWS;
  const int n_rows = min(a.OH - oh_begin, ROWS);
  const int nr_live = (n_rows - 1) * STRIDE + 3;
  const int ih_base = oh_begin * STRIDE - a.pad_t;
  const uint32_t zpw = (uint32_t)(a.input_zp & 0xff) * 0x01010101u;

  // ---- cooperative tile load: pieces of 16 bytes, index q = column * (CG/4) + piece ----
  {
    const int p16_log2 = cg_log2 - 2;  // 16-byte pieces per column
    const int per_row = IWT << p16_log2;
    const uint32_t tile_addr = (uint32_t)__cvta_generic_to_shared(tile);
    const int8_t* img = a.x + (size_t)n * a.H * a.W * a.C + c0;
    for (int q = threadIdx.x; q < per_row; q += 128) {
      const int col = q >> p16_log2, piece = q & ((1 << p16_log2) - 1);
      const int iw = iw_tile + col;
      const bool col_in = iw >= 0 && iw < a.W;
      const int8_t* src = img + (size_t)iw * a.C + piece * 16;
#pragma unroll
      for (int i = 0; i < NR; i++) {
        const int ih = ih_base + i;
        const uint32_t dst = tile_addr + (uint32_t)((i * per_row + q) * 16);
        if (i < nr_live) {
          if (col_in && ih >= 0 && ih < a.H) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src + (size_t)ih * a.W * a.C) : "memory");
          } else {
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(zpw) : "memory");
          }
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }

  const int c = c0 + gl * 4;
  const int ow0 = ow_tile + strip * TW;
  const bool live = ow0 < a.OW;
  // weights and per-channel constants of this thread's 4 channels (requested before the wait)
  uint32_t wq[3][TW][4];
#pragma unroll
  for (int kh = 0; kh < 3; kh++)
#pragma unroll
    for (int v = 0; v < TW; v++) {
      const uint4 w = __ldg(reinterpret_cast<const uint4*>(a.wq + ((size_t)(kh * TW + v) * a.C + c)));
      wq[kh][v][0] = w.x; wq[kh][v][1] = w.y; wq[kh][v][2] = w.z; wq[kh][v][3] = w.w;
    }
  int4 cq[4];
  ChanParams cp[EPI != 0 ? 1 : 4];
#pragma unroll
  for (int k = 0; k < 4; k++) {
    if (EPI != 0) cq[k] = __ldg(a.q4 + c + k);
    else cp[k] = a.chan[c + k];
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  if (!live) return;

  const uint32_t lo2 = (uint32_t)(a.clamp_min & 0xffff) * 0x10001u;
  const uint32_t hi2 = (uint32_t)(a.clamp_max & 0xffff) * 0x10001u;
  const int col_words = CG;                       // words per tile column
  const int row_words_t = IWT << cg_log2;         // words per tile row
  const uint32_t* mine = tile + strip * TW * STRIDE * col_words + gl;
  auto take_row = [&](int i, uint32_t (&t)[4]) {
    const uint32_t* r = mine + i * row_words_t;
    const uint32_t p0 = r[0], p1 = r[col_words], p2 = r[2 * col_words];
    const uint32_t p3 = NCOL == 4 ? r[3 * col_words] : zpw;
    transpose4x4(p0, p1, p2, p3, t);
  };
  uint32_t* __restrict__ o32 = reinterpret_cast<uint32_t*>(a.out);
  const int Cw = a.C >> 2;
  uint32_t win[NR][4];
  int out_off = ((n * a.OH + oh_begin) * a.OW + ow0) * Cw + (c >> 2);
  const int out_row_words = a.OW * Cw;
  const bool second = TW == 2 && ow0 + 1 < a.OW;
#pragma unroll
  for (int r = 0; r < ROWS; r++) {
    if (r < n_rows) {
      // keep the tile reads of later rows behind this row's arithmetic: hoisted to the top they cost
      // 30-40 registers and two resident blocks per SM
      asm volatile("" ::: "memory");
      if (r == 0) {
        take_row(0, win[0]);
        take_row(1, win[1]);
        take_row(2, win[2]);
      } else {
#pragma unroll
        for (int i = 0; i < STRIDE; i++) take_row(STRIDE * r + 2 - i, win[STRIDE * r + 2 - i]);
      }
#pragma unroll
      for (int v = 0; v < TW; v++) {
        int q[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
          int acc = EPI != 0 ? 0 : cp[k].bias;
#pragma unroll
          for (int kh = 0; kh < 3; kh++) acc = __dp4a((int)win[STRIDE * r + kh][k], (int)wq[kh][v][k], acc);
          if (EPI == 1) q[k] = scale_q4_sign(acc, cq[k]);
          else if (EPI == 2) q[k] = scale_q4(acc, cq[k]);
          else q[k] = scale_cp<false>(acc, cp[k]) + a.out_zp;
        }
        const uint32_t word = clamp_pack4(q[0], q[1], q[2], q[3], lo2, hi2);
        if (v == 0 || second) o32[(uint32_t)(out_off + v * Cw)] = word;
      }
      out_off += out_row_words;
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
  const long long in_bytes = (long long)a.N * a.H * a.W * a.C, out_bytes = (long long)a.N * a.OH * a.OW * a.C;
  if (in_bytes >= (1ll << 31) || out_bytes >= (1ll << 31)) return false;  // 32-bit offsets inside the kernel
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

// Block shape of dw3x3_tile_kernel: the widest channel chunk (16..128 channels) that divides C among those
// that waste the fewest threads on the columns beyond OW.
static bool dw_tile_shape(const DwArgs& a, int& cg_log2, int& tiles, int& cchunks) {
  static const bool no_tile = getenv("TB200_DW_NO_TILE") != nullptr;  // A/B switch: the per-thread-copy kernel
  if ((a.C & 15) != 0 || a.N > 65535 || no_tile) return false;
  const int tw = a.stride_h == 1 ? 2 : 1;
  const int owt = (a.OW + tw - 1) / tw;
  int best = -1, best_threads = 0;
  for (int l = 2; l <= 5; l++) {
    const int ch = 4 << l;
    if (a.C % ch) continue;
    const int sw = 128 >> l;
    const int threads = ((owt + sw - 1) / sw) * sw;
    if (best < 0 || threads <= best_threads) { best = l; best_threads = threads; }
  }
  if (best < 0) return false;
  cg_log2 = best;
  tiles = best_threads / (128 >> best);
  cchunks = a.C / (4 << best);
  return true;
}

void launch_depthwise(const DwArgs& a, cudaStream_t stream) {
  int cg_log2 = 0, tiles = 0, cchunks = 0;
  if (a.wq && depthwise3x3_supported(a) && dw_tile_shape(a, cg_log2, tiles, cchunks)) {
    const int S = a.stride_h, tw = S == 1 ? 2 : 1, sw = 128 >> cg_log2;
    static const bool rows8 = getenv("TB200_DW_ROWS8") != nullptr;  // A/B switch
    // 14 rows per thread only while that still leaves a few blocks per SM (a batch-1 frame wants the parallelism)
    const long long blocks14 = (long long)tiles * cchunks * ((a.OH + 13) / 14) * a.N;
    const int rows = (a.OH % 14 == 0 && !rows8 && blocks14 >= 148 * 16) ? 14 : kRows;
    const int nr = (rows - 1) * S + 3, iwt = (sw * tw - 1) * S + 3;
    const size_t smem = (size_t)nr * iwt * (4 << cg_log2);
    const dim3 grid((unsigned)(tiles * cchunks), (unsigned)((a.OH + rows - 1) / rows), (unsigned)a.N);
    auto go = [&](auto kern) { launch_dependent(kern, grid, dim3(128), smem, stream, a, cg_log2, cchunks); };
    if (rows == 14) {
      if (S == 1) {
        if (a.epi == 1) go(dw3x3_tile_kernel<1, 1, 14>);
        else if (a.epi == 2) go(dw3x3_tile_kernel<1, 2, 14>);
        else go(dw3x3_tile_kernel<1, 0, 14>);
      } else {
        if (a.epi == 1) go(dw3x3_tile_kernel<2, 1, 14>);
        else if (a.epi == 2) go(dw3x3_tile_kernel<2, 2, 14>);
        else go(dw3x3_tile_kernel<2, 0, 14>);
      }
    } else if (S == 1) {
      if (a.epi == 1) go(dw3x3_tile_kernel<1, 1, kRows>);
      else if (a.epi == 2) go(dw3x3_tile_kernel<1, 2, kRows>);
      else go(dw3x3_tile_kernel<1, 0, kRows>);
    } else {
      if (a.epi == 1) go(dw3x3_tile_kernel<2, 1, kRows>);
      else if (a.epi == 2) go(dw3x3_tile_kernel<2, 2, kRows>);
      else go(dw3x3_tile_kernel<2, 0, kRows>);
    }
  } else if (a.wq && depthwise3x3_supported(a)) {
    const int tw = a.stride_h == 1 ? 2 : 1;
    long long total = (long long)a.N * ((a.OH + kRows - 1) / kRows) * ((a.OW + tw - 1) / tw) * (a.C >> 2);
    unsigned blocks = (unsigned)((total + 127) / 128);
    const size_t smem1 = (size_t)((kRows - 1) * 1 + 3) * 4 * 128 * 4, smem2 = (size_t)((kRows - 1) * 2 + 3) * 4 * 128 * 4;
    if (a.stride_h == 1) {
      if (a.epi == 1) dw3x3_kernel<1, 1><<<blocks, 128, smem1, stream>>>(a);
      else if (a.epi == 2) dw3x3_kernel<1, 2><<<blocks, 128, smem1, stream>>>(a);
      else dw3x3_kernel<1, 0><<<blocks, 128, smem1, stream>>>(a);
    } else {
      if (a.epi == 1) dw3x3_kernel<2, 1><<<blocks, 128, smem2, stream>>>(a);
      else if (a.epi == 2) dw3x3_kernel<2, 2><<<blocks, 128, smem2, stream>>>(a);
      else dw3x3_kernel<2, 0><<<blocks, 128, smem2, stream>>>(a);
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
