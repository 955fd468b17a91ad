/*
 * TEST INFRASTRUCTURE ONLY - never linked into, imported by or called from the
 * product library. CPU restatement of the reference's host ("llvm-cpu")
 * arithmetic for the quantized layer ops.
 *
 * PARITY UNPINNED: the reference holds no golden output vectors for this path
 * (its tests compare engines at +-1 LSB, python/torq/testing/comparison.py:42-49)
 * and neither IREE nor the NPU C-model can be built or run beside this file.
 * What IS pinned: op forms, attribute values and constants of the reference's
 * TOSA fixtures (tests/testdata/tosa_ops, tests/testdata/gen_ops), and the
 * arithmetic order documented in
 * compiler/torq/Conversions/LinalgToTorqHL/PatternUtils.cpp:426-451,3441-3451.
 * Two independent restatements (this C file and oracle_np.py) must agree
 * bit-for-bit before any GPU kernel is trusted.
 */
#ifndef TOSA_ORACLE_H_
#define TOSA_ORACLE_H_
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* Requantisation parameters shared by every op that ends in a tosa.rescale. */
typedef struct tq_requant {
  const int32_t* multiplier; /* [OC] if per_channel else [1] */
  const int8_t* shift;       /* [OC] if per_channel else [1] */
  int32_t per_channel;
  int32_t double_round;
  int32_t mode;      /* 0 = TOSA apply_scale_32 (A), 1 = NPU common-shift (B) */
  int32_t out_zp;
  int32_t clamp_min; /* quantised-domain clamp (ReLU/ReLU6 folded) */
  int32_t clamp_max;
} tq_requant_t;

int32_t tq_apply_scale_32(int32_t value, int32_t multiplier, int32_t shift, int32_t double_round);
void tq_reciprocal_scale(uint32_t count, int32_t* multiplier, int32_t* shift);
void tq_quantize_multiplier(double real, int32_t* multiplier, int32_t* shift);
int tq_num_threads(void);
void tq_set_num_threads(int n);

void tq_conv2d(const int8_t* x, int N, int H, int W, int IC, const int8_t* w, int OC, int KH, int KW,
               const int32_t* bias, int bias_len, int stride_h, int stride_w, int dil_h, int dil_w,
               int pad_t, int pad_b, int pad_l, int pad_r, int input_zp, int weight_zp,
               const tq_requant_t* rq, int8_t* out, int OH, int OW);

void tq_depthwise(const int8_t* x, int N, int H, int W, int C, const int8_t* w, int M, int KH, int KW,
                  const int32_t* bias, int bias_len, int stride_h, int stride_w, int dil_h, int dil_w,
                  int pad_t, int pad_b, int pad_l, int pad_r, int input_zp, int weight_zp,
                  const tq_requant_t* rq, int8_t* out, int OH, int OW);

/* a [M,K] row-major, w [N,K] row-major ("[O,I]"), out int8 [M,N] */
void tq_fully_connected(const int8_t* a, int M, int K, const int8_t* w, int N, const int32_t* bias,
                        int bias_len, int input_zp, int weight_zp, const tq_requant_t* rq, int8_t* out);
/* raw matmul: a [M,K], b [K,N] row-major, out int32 [M,N] */
void tq_matmul_i32(const int8_t* a, int M, int K, const int8_t* b, int N, int a_zp, int b_zp,
                   int32_t* out);

void tq_maxpool(const int8_t* x, int N, int H, int W, int C, int KH, int KW, int stride_h,
                int stride_w, int pad_t, int pad_b, int pad_l, int pad_r, int pad_value, int8_t* out,
                int OH, int OW);
void tq_maxpool_i16(const int16_t* x, int N, int H, int W, int C, int KH, int KW, int stride_h, int stride_w,
                    int pad_t, int pad_l, int pad_value, int16_t* out, int OH, int OW);
void tq_avgpool(const int8_t* x, int N, int H, int W, int C, int KH, int KW, int stride_h,
                int stride_w, int pad_t, int pad_b, int pad_l, int pad_r, int input_zp, int output_zp,
                int8_t* out, int OH, int OW);

/* kind: 0 add, 1 sub, 2 mul */
void tq_binary(int kind, const int8_t* a, const int8_t* b, int64_t n, int a_zp, int a_mult, int a_shift,
               int b_zp, int b_mult, int b_shift, int out_mult, int out_shift, int out_zp,
               int double_round, int clamp_min, int clamp_max, int8_t* out);
void tq_binary_pre(int kind, const int8_t* a, const int8_t* b, int64_t n, int a_zp, int a_lshift, int a_mult, int a_shift,
                   int b_zp, int b_lshift, int b_mult, int b_shift, int out_mult, int out_shift, int out_zp,
                   int double_round, int clamp_min, int clamp_max, int8_t* out);
void tq_table(const int8_t* x, int64_t n, const int8_t* table, int8_t* out);
void tq_rescale(const int8_t* x, int64_t rows, int C, int input_zp, const tq_requant_t* rq, int8_t* out);
void tq_resize_nn2x(const int8_t* x, int N, int H, int W, int C, int8_t* out);
void tq_concat2(const int8_t* a, int Ca, const int8_t* b, int Cb, int64_t rows, int a_zp, int a_mult,
                int a_shift, int b_zp, int b_mult, int b_shift, int out_zp, int double_round,
                int8_t* out);

#ifdef __cplusplus
}
#endif
#endif
