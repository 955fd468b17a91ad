/*
 * TEST INFRASTRUCTURE ONLY (see tosa_oracle.h). PARITY UNPINNED (see there).
 *
 * Every function states the reference location whose arithmetic it restates.
 * The integer rescale itself lives in MLIR's TosaToArith lowering of
 * tosa.apply_scale, pinned by the IREE v3.10 fork the reference submodules
 * (third_party/iree, absent); its published definition is TOSA 1.0.1
 * apply_scale_32, which is what is written here.
 */
#include "tosa_oracle.h"

#include <math.h>
#include <stddef.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static int g_threads = 0;
int tq_num_threads(void) {
#ifdef _OPENMP
  return g_threads > 0 ? g_threads : omp_get_max_threads();
#else
  return 1;
#endif
}
void tq_set_num_threads(int n) {
  g_threads = n;
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#endif
}

/* int32 arithmetic wraps, it does not saturate
 * (compiler/torq/Utils/ConversionUtils.cpp:40-45). */
static inline int32_t wadd(int32_t a, int32_t b) { return (int32_t)((uint32_t)a + (uint32_t)b); }
static inline int32_t wsub(int32_t a, int32_t b) { return (int32_t)((uint32_t)a - (uint32_t)b); }
static inline int32_t wmul(int32_t a, int32_t b) { return (int32_t)((uint32_t)a * (uint32_t)b); }

/* TOSA 1.0.1 apply_scale_32. Op order as the reference matches it:
 * apply_scale -> addi(zp) -> maxsi -> minsi -> trunci
 * (compiler/torq/Conversions/LinalgToTorqHL/PatternUtils.cpp:3441-3451). */
int32_t tq_apply_scale_32(int32_t value, int32_t multiplier, int32_t shift, int32_t double_round) {
  int64_t round = (int64_t)1 << (shift - 1);
  if (double_round && shift > 31) {
    round += (value >= 0) ? ((int64_t)1 << 30) : -((int64_t)1 << 30);
  }
  int64_t r = (int64_t)value * (int64_t)multiplier + round;
  r = r >> shift; /* arithmetic */
  return (int32_t)(uint32_t)(uint64_t)r;
}

/* compiler/torq/Conversions/TosaToTorqHL/Patterns.cpp:776-805 (the tree's copy of
 * the TOSA spec helper). */
void tq_reciprocal_scale(uint32_t count, int32_t* multiplier, int32_t* shift) {
  uint32_t v = count - 1;
  int k = 0;
  while (v) {
    k++;
    v >>= 1;
  } /* k = 32 - clz(count - 1) */
  int64_t numerator = (((int64_t)1 << 30) + 1) << k;
  *multiplier = (int32_t)(numerator / (int64_t)count);
  *shift = 30 + k;
}

/* The TFLite/TOSA "quantize multiplier" rule with scale32: real = M * 2^-S,
 * M in [2^30, 2^31). Used to derive the integers the seeded workloads record. */
void tq_quantize_multiplier(double real, int32_t* multiplier, int32_t* shift) {
  if (real == 0.0) {
    *multiplier = 0;
    *shift = 2;
    return;
  }
  int e;
  double q = frexp(real, &e);
  int64_t m = (int64_t)llround(q * (double)((int64_t)1 << 31));
  if (m == ((int64_t)1 << 31)) {
    m /= 2;
    e++;
  }
  int s = 31 - e;
  if (s > 62) { /* too small to represent: shift the multiplier down */
    m >>= (s - 62);
    s = 62;
  }
  *multiplier = (int32_t)m;
  *shift = s;
}

/* Requantise one accumulator (bias already added for mode A; mode B adds it
 * itself in the reference pseudocode, same sum). Mode B:
 * compiler/torq/Utils/Kernel.h:607-635 with scale[c] = M[c] >> (S[c]-min S)
 * (compiler/torq/Conversions/LinalgToTorqHL/PatternUtils.cpp:3536-3549). */
typedef struct {
  int32_t min_shift;
} rq_ctx_t;

static rq_ctx_t rq_prepare(const tq_requant_t* rq, int oc) {
  rq_ctx_t c;
  c.min_shift = rq->shift[0];
  if (rq->per_channel)
    for (int i = 1; i < oc; i++)
      if (rq->shift[i] < c.min_shift) c.min_shift = rq->shift[i];
  return c;
}

static inline int8_t rq_apply(const tq_requant_t* rq, const rq_ctx_t* ctx, int32_t acc, int c) {
  int idx = rq->per_channel ? c : 0;
  int32_t r;
  if (rq->mode == 0) {
    r = tq_apply_scale_32(acc, rq->multiplier[idx], rq->shift[idx], rq->double_round);
  } else {
    int sh = ctx->min_shift;
    int32_t scale = rq->multiplier[idx] >> (rq->shift[idx] - sh);
    int64_t t = (int64_t)acc * (int64_t)scale;
    t = (t + ((int64_t)1 << (sh - 1))) >> sh;
    r = (int32_t)(uint32_t)(uint64_t)t;
  }
  r = wadd(r, rq->out_zp);
  if (r < rq->clamp_min) r = rq->clamp_min;
  if (r > rq->clamp_max) r = rq->clamp_max;
  return (int8_t)r;
}

/* torq_hl.conv2d semantics: compiler/torq/Conversions/LinalgToTorqHL/Conv2DPattern.cpp:478-654.
 * Padded taps hold input_zp, i.e. contribute (zp - zp) * w = 0 (:630,642). */
void tq_conv2d(const int8_t* x, int N, int H, int W, int IC, const int8_t* w, int OC, int KH, int KW,
               const int32_t* bias, int bias_len, int stride_h, int stride_w, int dil_h, int dil_w,
               int pad_t, int pad_b, int pad_l, int pad_r, int input_zp, int weight_zp,
               const tq_requant_t* rq, int8_t* out, int OH, int OW) {
  (void)pad_b;
  (void)pad_r;
  rq_ctx_t ctx = rq_prepare(rq, OC);
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < N; n++) {
    for (int oh = 0; oh < OH; oh++) {
      for (int ow = 0; ow < OW; ow++) {
        int8_t* o = out + (((size_t)n * OH + oh) * OW + ow) * OC;
        for (int oc = 0; oc < OC; oc++) {
          int32_t acc = 0;
          const int8_t* wk = w + (size_t)oc * KH * KW * IC;
          for (int kh = 0; kh < KH; kh++) {
            int ih = oh * stride_h - pad_t + kh * dil_h;
            if (ih < 0 || ih >= H) continue;
            for (int kw = 0; kw < KW; kw++) {
              int iw = ow * stride_w - pad_l + kw * dil_w;
              if (iw < 0 || iw >= W) continue;
              const int8_t* xp = x + (((size_t)n * H + ih) * W + iw) * IC;
              const int8_t* wp = wk + ((size_t)kh * KW + kw) * IC;
              int32_t s = 0;
              if (input_zp == 0 && weight_zp == 0) {
                for (int ic = 0; ic < IC; ic++) s += (int32_t)xp[ic] * (int32_t)wp[ic];
              } else {
                for (int ic = 0; ic < IC; ic++)
                  s += ((int32_t)xp[ic] - input_zp) * ((int32_t)wp[ic] - weight_zp);
              }
              acc = wadd(acc, s);
            }
          }
          acc = wadd(acc, bias[bias_len == 1 ? 0 : oc]);
          o[oc] = rq_apply(rq, &ctx, acc, oc);
        }
      }
    }
  }
}

/* torq_hl.depthwise_conv2d: Conv2DPattern.cpp:627-637; TOSA weights [KH,KW,C,M],
 * output channel = c * M + m (tests/testdata/tosa_ops/dw_peeling.mlir). */
void tq_depthwise(const int8_t* x, int N, int H, int W, int C, const int8_t* w, int M, int KH, int KW,
                  const int32_t* bias, int bias_len, int stride_h, int stride_w, int dil_h, int dil_w,
                  int pad_t, int pad_b, int pad_l, int pad_r, int input_zp, int weight_zp,
                  const tq_requant_t* rq, int8_t* out, int OH, int OW) {
  (void)pad_b;
  (void)pad_r;
  int OC = C * M;
  rq_ctx_t ctx = rq_prepare(rq, OC);
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < N; n++) {
    for (int oh = 0; oh < OH; oh++) {
      for (int ow = 0; ow < OW; ow++) {
        int8_t* o = out + (((size_t)n * OH + oh) * OW + ow) * OC;
        for (int c = 0; c < C; c++) {
          for (int m = 0; m < M; m++) {
            int32_t acc = 0;
            for (int kh = 0; kh < KH; kh++) {
              int ih = oh * stride_h - pad_t + kh * dil_h;
              if (ih < 0 || ih >= H) continue;
              for (int kw = 0; kw < KW; kw++) {
                int iw = ow * stride_w - pad_l + kw * dil_w;
                if (iw < 0 || iw >= W) continue;
                int32_t xv = (int32_t)x[(((size_t)n * H + ih) * W + iw) * C + c] - input_zp;
                int32_t wv = (int32_t)w[(((size_t)kh * KW + kw) * C + c) * M + m] - weight_zp;
                acc = wadd(acc, xv * wv);
              }
            }
            int oc = c * M + m;
            acc = wadd(acc, bias[bias_len == 1 ? 0 : oc]);
            o[oc] = rq_apply(rq, &ctx, acc, oc);
          }
        }
      }
    }
  }
}

/* torq_hl.fully_connected: weights canonicalised to [O, I]
 * (compiler/torq/Conversions/LinalgToTorqHL/Conv2DMatmulPattern.cpp:121-138). */
void tq_fully_connected(const int8_t* a, int M, int K, const int8_t* w, int N, const int32_t* bias,
                        int bias_len, int input_zp, int weight_zp, const tq_requant_t* rq, int8_t* out) {
  rq_ctx_t ctx = rq_prepare(rq, N);
#pragma omp parallel for collapse(2) schedule(static)
  for (int m = 0; m < M; m++) {
    for (int n = 0; n < N; n++) {
      const int8_t* ap = a + (size_t)m * K;
      const int8_t* wp = w + (size_t)n * K;
      int32_t acc = 0;
      if (input_zp == 0 && weight_zp == 0) {
        for (int k = 0; k < K; k++) acc += (int32_t)ap[k] * (int32_t)wp[k];
      } else {
        for (int k = 0; k < K; k++)
          acc = wadd(acc, ((int32_t)ap[k] - input_zp) * ((int32_t)wp[k] - weight_zp));
      }
      acc = wadd(acc, bias[bias_len == 1 ? 0 : n]);
      out[(size_t)m * N + n] = rq_apply(rq, &ctx, acc, n);
    }
  }
}

/* raw torq_hl.matmul (compiler/torq/Conversions/LinalgToTorqHL/MatmulPattern.cpp:917-995;
 * tests/testdata/tosa_ops/matmul-in-int8-out-int32.mlir). */
void tq_matmul_i32(const int8_t* a, int M, int K, const int8_t* b, int N, int a_zp, int b_zp,
                   int32_t* out) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; m++) {
    int32_t* o = out + (size_t)m * N;
    for (int n = 0; n < N; n++) o[n] = 0;
    for (int k = 0; k < K; k++) {
      int32_t av = (int32_t)a[(size_t)m * K + k] - a_zp;
      const int8_t* bp = b + (size_t)k * N;
      for (int n = 0; n < N; n++) o[n] = wadd(o[n], av * ((int32_t)bp[n] - b_zp));
    }
  }
}

/* torq_hl.maxpool2d: compiler/torq/Conversions/LinalgToTorqHL/PoolingPattern.cpp:128-258;
 * padding comes from a folded tosa.pad with an explicit constant (:160). */
void tq_maxpool(const int8_t* x, int N, int H, int W, int C, int KH, int KW, int stride_h,
                int stride_w, int pad_t, int pad_b, int pad_l, int pad_r, int pad_value, int8_t* out,
                int OH, int OW) {
  (void)pad_b;
  (void)pad_r;
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < N; n++) {
    for (int oh = 0; oh < OH; oh++) {
      for (int ow = 0; ow < OW; ow++) {
        int8_t* o = out + (((size_t)n * OH + oh) * OW + ow) * C;
        for (int c = 0; c < C; c++) {
          int32_t best = -128;
          for (int kh = 0; kh < KH; kh++) {
            int ih = oh * stride_h - pad_t + kh;
            for (int kw = 0; kw < KW; kw++) {
              int iw = ow * stride_w - pad_l + kw;
              int32_t v = (ih < 0 || ih >= H || iw < 0 || iw >= W)
                              ? pad_value
                              : (int32_t)x[(((size_t)n * H + ih) * W + iw) * C + c];
              if (v > best) best = v;
            }
          }
          o[c] = (int8_t)best;
        }
      }
    }
  }
}

/* The same on int16 tensors (tests/testdata/tosa_ops/maxpool2d_i16_s2_k3x3_32x32x4.mlir,
 * doc/user-manual/ops.md: MaxPool2D i16 -> i16). */
void tq_maxpool_i16(const int16_t* x, int N, int H, int W, int C, int KH, int KW, int stride_h, int stride_w,
                    int pad_t, int pad_l, int pad_value, int16_t* out, int OH, int OW) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < N; n++) {
    for (int oh = 0; oh < OH; oh++) {
      for (int ow = 0; ow < OW; ow++) {
        int16_t* o = out + (((size_t)n * OH + oh) * OW + ow) * C;
        for (int c = 0; c < C; c++) {
          int32_t best = -32768;
          for (int kh = 0; kh < KH; kh++) {
            int ih = oh * stride_h - pad_t + kh;
            for (int kw = 0; kw < KW; kw++) {
              int iw = ow * stride_w - pad_l + kw;
              int32_t v = (ih < 0 || ih >= H || iw < 0 || iw >= W)
                              ? pad_value
                              : (int32_t)x[(((size_t)n * H + ih) * W + iw) * C + c];
              if (v > best) best = v;
            }
          }
          o[c] = (int16_t)best;
        }
      }
    }
  }
}

/* tosa.avg_pool2d {acc_type = i32} (tests/testdata/tosa_ops/avgpool2d.mlir);
 * count excludes padding, scale = reciprocal_scale(count), single rounding
 * (compiler/torq/Conversions/LinalgToTorqHL/PoolingPattern.cpp:263-355 for the
 * whole-frame case). */
void tq_avgpool(const int8_t* x, int N, int H, int W, int C, int KH, int KW, int stride_h,
                int stride_w, int pad_t, int pad_b, int pad_l, int pad_r, int input_zp, int output_zp,
                int8_t* out, int OH, int OW) {
  (void)pad_b;
  (void)pad_r;
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < N; n++) {
    for (int oh = 0; oh < OH; oh++) {
      for (int ow = 0; ow < OW; ow++) {
        int8_t* o = out + (((size_t)n * OH + oh) * OW + ow) * C;
        for (int c = 0; c < C; c++) {
          int32_t acc = 0;
          uint32_t count = 0;
          for (int kh = 0; kh < KH; kh++) {
            int ih = oh * stride_h - pad_t + kh;
            if (ih < 0 || ih >= H) continue;
            for (int kw = 0; kw < KW; kw++) {
              int iw = ow * stride_w - pad_l + kw;
              if (iw < 0 || iw >= W) continue;
              count++;
              acc = wadd(acc, (int32_t)x[(((size_t)n * H + ih) * W + iw) * C + c] - input_zp);
            }
          }
          int32_t mult, sh;
          tq_reciprocal_scale(count ? count : 1, &mult, &sh);
          int32_t r = tq_apply_scale_32(acc, mult, sh, 0);
          r = wadd(r, output_zp);
          if (r < -128) r = -128;
          if (r > 127) r = 127;
          o[c] = (int8_t)r;
        }
      }
    }
  }
}

/* torq_hl.add / sub / mul in their TOSA form: rescale(i8->i32) x2 -> op -> rescale
 * (tests/testdata/tosa_ops/add-single-rescale.mlir, yolov8_block_mul_rescale.mlir;
 * compiler/torq/Conversions/LinalgToTorqHL/ElementWiseBinaryPattern.cpp:385-570,
 * MulPattern.cpp:229-238). */
void tq_binary(int kind, const int8_t* a, const int8_t* b, int64_t n, int a_zp, int a_mult, int a_shift,
               int b_zp, int b_mult, int b_shift, int out_mult, int out_shift, int out_zp,
               int double_round, int clamp_min, int clamp_max, int8_t* out) {
  tq_binary_pre(kind, a, b, n, a_zp, 0, a_mult, a_shift, b_zp, 0, b_mult, b_shift, out_mult, out_shift, out_zp,
                double_round, clamp_min, clamp_max, out);
}

/* The same with the two-stage input rescale of the TFLite-derived fixtures
 * (tests/testdata/tosa_ops/add-56x56x256.mlir, sub-56x56x256xi8.mlir): the first tosa.rescale
 * (multiplier 2^30, shift s <= 30, i8 -> i32) is an exact left shift by 30 - s, the second
 * (i32 -> i32) is the real scaling. x_lshift is that left shift (0: single-stage form). */
void tq_binary_pre(int kind, const int8_t* a, const int8_t* b, int64_t n, int a_zp, int a_lshift, int a_mult, int a_shift,
                   int b_zp, int b_lshift, int b_mult, int b_shift, int out_mult, int out_shift, int out_zp,
                   int double_round, int clamp_min, int clamp_max, int8_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) {
    int32_t ra = tq_apply_scale_32(((int32_t)a[i] - a_zp) * (1 << a_lshift), a_mult, a_shift, double_round);
    int32_t rb = tq_apply_scale_32(((int32_t)b[i] - b_zp) * (1 << b_lshift), b_mult, b_shift, double_round);
    int32_t v = kind == 0 ? wadd(ra, rb) : kind == 1 ? wsub(ra, rb) : wmul(ra, rb);
    int32_t r = tq_apply_scale_32(v, out_mult, out_shift, double_round);
    r = wadd(r, out_zp);
    if (r < clamp_min) r = clamp_min;
    if (r > clamp_max) r = clamp_max;
    out[i] = (int8_t)r;
  }
}

/* torq_hl.table: out = table[x + 128]
 * (compiler/torq/Conversions/LinalgToTorqHL/ExtractPattern.cpp:97-135). */
void tq_table(const int8_t* x, int64_t n, const int8_t* table, int8_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) out[i] = table[(int)x[i] + 128];
}

/* standalone tosa.rescale i8 -> i8: extsi -> subi(izp) -> apply_scale -> addi(ozp)
 * -> clamp -> trunci (PatternUtils.cpp:426-435,3441-3451). */
void tq_rescale(const int8_t* x, int64_t rows, int C, int input_zp, const tq_requant_t* rq, int8_t* out) {
  rq_ctx_t ctx = rq_prepare(rq, C);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; r++)
    for (int c = 0; c < C; c++)
      out[r * C + c] = rq_apply(rq, &ctx, (int32_t)x[r * C + c] - input_zp, c);
}

/* tosa.resize NEAREST_NEIGHBOR scale 2: out[y,x] = in[y/2, x/2]
 * (PatternUtils.cpp:489-491; tests/testdata/tosa_ops/resize-8x8x32xi8.mlir). */
void tq_resize_nn2x(const int8_t* x, int N, int H, int W, int C, int8_t* out) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < N; n++)
    for (int oh = 0; oh < 2 * H; oh++)
      for (int ow = 0; ow < 2 * W; ow++)
        memcpy(out + (((size_t)n * 2 * H + oh) * 2 * W + ow) * C,
               x + (((size_t)n * H + oh / 2) * W + ow / 2) * C, (size_t)C);
}

/* rescaled concat along channels = two input rescales feeding tosa.concat
 * (tests/testdata/tosa_ops/concat-a.mlir for the plain copy form). */
void tq_concat2(const int8_t* a, int Ca, const int8_t* b, int Cb, int64_t rows, int a_zp, int a_mult,
                int a_shift, int b_zp, int b_mult, int b_shift, int out_zp, int double_round,
                int8_t* out) {
  int C = Ca + Cb;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; r++) {
    for (int c = 0; c < Ca; c++) {
      int32_t v = wadd(tq_apply_scale_32((int32_t)a[r * Ca + c] - a_zp, a_mult, a_shift, double_round),
                       out_zp);
      out[r * C + c] = (int8_t)(v < -128 ? -128 : v > 127 ? 127 : v);
    }
    for (int c = 0; c < Cb; c++) {
      int32_t v = wadd(tq_apply_scale_32((int32_t)b[r * Cb + c] - b_zp, b_mult, b_shift, double_round),
                       out_zp);
      out[r * C + Ca + c] = (int8_t)(v < -128 ? -128 : v > 127 ? 127 : v);
    }
  }
}
