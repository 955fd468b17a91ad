// Host-callable launchers of the layer kernels. Every launcher only enqueues
// work on `stream`; none allocates or synchronises.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "common.cuh"

namespace tb200 {

// ---- per-device facts (device_util.cu) ----
int current_device();
int current_sm_count();  // SMs of the current device
// One-time set-up that is per device (function attributes): first_use_on_device is true until
// mark_used_on_device has been called with the same flag while the same device was current.
bool first_use_on_device(std::atomic<unsigned long long>& done);
void mark_used_on_device(std::atomic<unsigned long long>& done);
// Limit of every bounded wait inside the kernels, from TB200_WAIT_LIMIT_MS (default 2000 ms).
unsigned long long wait_limit_ns();

struct ConvArgs {
  const int8_t* x;        // NHWC
  const int8_t* w;        // packed [OC][Kpad], K order (kh, kw, ic), zero padded
  const ChanParams* chan; // [OC]
  int8_t* out;            // NHWC
  int N, H, W, IC, OC, KH, KW, OH, OW;
  int stride_h, stride_w, dil_h, dil_w, pad_t, pad_l;
  int K, Kpad;            // KH*KW*IC and its padded row length
  int input_zp, weight_zp, out_zp, clamp_min, clamp_max;
  int double_round;
  int hi_shift;           // every rescale shift of the op is >= 32
  const int8_t* lut;      // 256-entry table applied to the int8 result (out = lut[q + 128]), or null
  int epi;                // 0 = ChanParams arithmetic; 1 / 2 = compact Q4 records with / without the sign term (stem kernel)
  const int4* q4;         // [OC] Q4 records (epi != 0); the output zero point rides in them
  long long x_bytes;      // size of the input tensor: the stem kernel reads it in aligned words
};
void launch_conv2d_simt(const ConvArgs& a, cudaStream_t stream);

// FullyConnected / 1x1 convolution on at most 4 rows (a classifier at batch 1, GEMV-shaped calls): the weights are
// streamed once at HBM rate by one warp per output channel (dp4a), instead of through 128-row tensor-core tiles.
struct FcRowsArgs {
  const int8_t* x;         // [M, K]
  const int8_t* w;         // [N, K]
  const ChanParams* chan;  // [N]
  int8_t* out;             // [M, N]
  int M, N, K;             // M <= 4, K a multiple of 16
  int out_zp, clamp_min, clamp_max, hi_shift;
  const int8_t* lut;       // fused table or null
};
void launch_fc_rows(const FcRowsArgs& a, cudaStream_t stream);

// Conv2D on int16 activations with int8 weights and the 16-bit rescale that follows it (TB200_OP_CONV2D_I16).
struct ConvI16Args {
  const int16_t* x;         // NHWC
  const int8_t* w;          // OHWI
  const long long* bias;    // [OC] (already broadcast)
  const int32_t* mult;      // [OC] 16-bit multipliers
  const int32_t* shift;     // [OC]
  int16_t* out;             // NHWC
  int N, H, W, IC, OC, KH, KW, OH, OW;
  int stride_h, stride_w, dil_h, dil_w, pad_t, pad_l;
  int input_zp, weight_zp, out_zp, clamp_min, clamp_max;
};
void launch_conv2d_i16(const ConvI16Args& a, cudaStream_t stream);
const char* conv2d_simt_kernel_name(const ConvArgs& a);  // which CUDA-core kernel the launcher picks

struct DwArgs {
  const int8_t* x;        // NHWC
  const int8_t* w;        // [KH][KW][C][M]
  const ChanParams* chan; // [C*M], bias unmodified (taps outside the image are skipped)
  int8_t* out;
  int N, H, W, C, M, KH, KW, OH, OW;
  int stride_h, stride_w, dil_h, dil_w, pad_t, pad_l;
  int input_zp, weight_zp, out_zp, clamp_min, clamp_max;
  int double_round;
  int hi_shift;           // every rescale shift of the op is >= 32
  int epi;                // 3x3 fast path: 0 = ChanParams arithmetic, 1 / 2 = compact Q4 records with / without the sign term
  const int4* q4;         // [C] Q4 records (epi != 0); the output zero point rides in them
  const uint32_t* wq;     // 3x3 fast path: weights packed per row for dp4a (see depthwise.cu), else null
};
void launch_depthwise(const DwArgs& a, cudaStream_t stream);
// 3x3, M == 1, C % 4 == 0, no dilation, stride 1 or 2, symmetric weights: the dp4a kernel applies;
// its ChanParams::bias must have the input zero point folded (bias - izp * sum of the 9 taps).
bool depthwise3x3_supported(const DwArgs& a);
// Packs [3][3][C] weights into [3 rows][variants][C] words; returns the word count written.
size_t depthwise3x3_pack(const int8_t* w, int C, int stride, uint32_t* out);

// raw int8 x int8 -> int32 matmul, b is [K][N]
void launch_matmul_int(const void* a, const void* b, void* out, bool in_i16, bool out_i16, int M, int K, int N, int a_zp,
                       int b_zp, cudaStream_t stream);

struct PoolArgs {
  const int8_t* x;
  int8_t* out;
  int N, H, W, C, KH, KW, OH, OW, stride_h, stride_w, pad_t, pad_l;
  int pad_value;            // max pool
  int input_zp, output_zp;  // avg pool
  int elem16;               // max pool on int16 tensors (x and out then point to int16 data)
};
void launch_maxpool(const PoolArgs& a, cudaStream_t stream);
void launch_avgpool(const PoolArgs& a, cudaStream_t stream);

struct BinaryArgs {
  const int8_t* a;
  const int8_t* b;
  int8_t* out;
  long long n;
  int kind;  // 0 add, 1 sub, 2 mul
  int a_zp, a_mult, a_shift, b_zp, b_mult, b_shift, out_mult, out_shift, out_zp;
  int double_round, clamp_min, clamp_max;
  int a_lshift, b_lshift;  // (x - zp) << lshift before the input rescale (two-stage input rescale), 0..22
  int epi;                 // output rescale: 0 = 64-bit arithmetic, 1 / 2 = the compact 32-bit record q4 with / without the sign term
  int4 q4;
};
void launch_binary(const BinaryArgs& a, cudaStream_t stream);

void launch_table(const int8_t* x, const int8_t* table, int8_t* out, long long n, cudaStream_t stream);

struct RescaleArgs {
  const int8_t* x;
  int8_t* out;
  const ChanParams* chan;  // [C] or [1]
  long long rows;
  int C, per_channel, input_zp, out_zp, clamp_min, clamp_max, double_round;
  int out_row_stride, out_col_offset;  // lets a concat write into a wider row
  int identity;  // the rescale passes values through unchanged (set by the planner): a strided copy
};
void launch_rescale(const RescaleArgs& a, cudaStream_t stream);

// ---- tensor-core GEMM (gemm_tcgen05.cu) ----
struct GemmTcGeometry {
  int row_bytes;  // bytes of K per shared-memory row: 32, 64 or 128
  int k_blocks;   // K blocks of row_bytes
  int Kpad;       // k_blocks * row_bytes: row length of the packed weights
  int BN;         // columns per N tile: a multiple of 16 up to 128, or a multiple of 32 up to 256 (gpt == 2)
  int n_tiles;
  int gpt;        // epilogue groups that share one accumulator tile (1, or 2 for the wide tiles)
};
GemmTcGeometry gemm_tc_geometry(int N, int K, long long M);  // M rows: few rows keep the narrow tiles
struct GemmTcArgs {
  const int8_t* a;        // [M, K] int8, row pitch lda bytes (multiple of 16)
  long long lda;
  const int8_t* w;        // packed [n_tiles * BN][Kpad] per gemm_tc_geometry(N, K, M), zero padded
  const ChanParams* chan; // [n_tiles * BN]
  int8_t* out;            // [M, N] int8, row pitch ldc bytes
  long long ldc;
  long long M;
  int N, K;
  int out_zp, clamp_min, clamp_max;
  int epi;                // 0 = ChanParams arithmetic (any shift), 1 / 2 = compact Q4 records with / without the sign term
  const int4* q4;         // [n_tiles * BN] Q4 records when epi != 0 (common.cuh); the output zero point rides in them
  int* status;            // device status word: a kernel whose bounded wait expires writes a code here
  const int8_t* lut;      // 256-entry table applied to the int8 result, or null
  // A rescaled add fused behind the product (a residual connection): out = rescale(t_self[product] + t_other[res]),
  // the operand-side rescales as tables exactly as binary_kernel builds them. res has the layout of out.
  const int8_t* res;      // the other operand of the add, or null
  BinaryArgs add;         // its parameters (kind 0, epi 1 or 2); a_* belong to the product when add_self_is_a
  int add_self_is_a;
};
struct GemmTcState;       // cached tensor maps of one GEMM step
GemmTcState* gemm_tc_state_new();
void gemm_tc_state_free(GemmTcState* s);
bool gemm_tc_supported(long long M, int N, int K, long long lda);
cudaError_t launch_gemm_i8_tc(const GemmTcArgs& a, GemmTcState* st, cudaStream_t stream);

// KH x KW convolution (stride 1 or 2, no dilation, symmetric weights, IC % 16 == 0, OC % 16 == 0)
// as implicit GEMM on the same kernel: see gemm_tcgen05.cu.
int read_gemm_trace(unsigned long long* out, int n);  // debugging aid, see gemm_tcgen05.cu
struct ConvTcGeometry {
  int row_bytes, icb_per_tap, k_blocks, Kpad;  // K = (kh, kw, ic): the OHWI row of a filter
  int BN, n_tiles, gpt;
  int TW, TH, tiles_w, tiles_h;                // output patch of a tile (TW * TH = 128)
  int khs;                                     // kernel rows served by one load of TH + khs - 1 input rows (1 = a load per tap)
  int halo;                                    // 1: one load per tile and channel block serves every tap (TWv valid columns of TW = 16)
  int TWv;                                     // output columns a tile produces (TW unless halo)
  int s2;                                      // 1: stride-2 3x3 over one patch of pixel pairs per tile (16 x 8 outputs)
};
ConvTcGeometry conv_tc_geometry(int N, int OH, int OW, int IC, int OC, int KH, int KW, int stride);
// The geometry the launch uses: as above, plus the stride-2 pixel-pair form, which depends on the input width and the left pad.
ConvTcGeometry conv_tc_geometry_padded(int N, int OH, int OW, int W, int IC, int OC, int KH, int KW, int stride, int pad_l);
bool conv_tc_supported(int N, int H, int W, int IC, int OC, int KH, int KW, int stride_h, int stride_w, int dil_h, int dil_w,
                       int OH, int OW);
struct ConvTcArgs {
  const int8_t* x;        // [N, H, W, IC]
  const int8_t* w;        // [n_tiles * BN][Kpad]: per tap IC weights padded to whole channel blocks; rows beyond OC zero
  const ChanParams* chan; // [n_tiles * BN], bias already holds bias - izp * sum of all taps
  int8_t* out;            // [N, OH, OW, OC]
  int N, H, W, IC, OC, KH, KW, OH, OW, stride, pad_t, pad_l;
  int out_zp, clamp_min, clamp_max;
  int epi;                // as GemmTcArgs::epi
  const int4* q4;
  // border classes: pixel (oh, ow) has class rcls[oh] * ncc + ccls[ow]; corr[class][n_tiles * BN] =
  // izp * (sum of the weights of the taps that fall outside the frame for that class)
  const int32_t* corr;
  const uint8_t* rcls;
  const uint8_t* ccls;
  const uint8_t* cls_nonzero;
  int ncc;
  int* status;
  const int8_t* lut;      // 256-entry table applied to the int8 result, or null
};
cudaError_t launch_conv_i8_tc(const ConvTcArgs& a, GemmTcState* st, cudaStream_t stream);

// ---- decoder kernels (decoder.cu): bf16 tensors are passed as uint16_t bit patterns ----
void launch_embed(const int32_t* tok, const int8_t* table, const uint16_t* scale, uint16_t* out, int B, int H, int V,
                  float mult, cudaStream_t stream);
void launch_rmsnorm(const uint16_t* x, const uint16_t* res, const uint16_t* w, uint16_t* out, int rows, int H, float eps,
                    cudaStream_t stream);
int gemv_w8_splits(int B, int N, int K);
size_t gemv_w8_scratch_bytes(int B, int N, int splits);
// false when a caller-chosen slice count leaves K slices the tensor-core kernel cannot stage in shared memory
bool gemv_w8_splits_fit(int B, int N, int K, int splits);
// y bf16, or fp32 when y_f32. finalize == false with more than one K slice in use leaves the per-slice
// sums in scratch ([slice][B][N] fp32) for a consumer kernel that takes a GemvPartials.
void launch_gemv_w8(const uint16_t* x, const int8_t* W, const uint16_t* scale, void* y, int y_f32, float* scratch, int B,
                    int N, int K, int splits, cudaStream_t stream, bool finalize = true);
int gemv_w8_used_splits(int B, int N, int K, int splits);  // K slices that launch_gemv_w8 really launches
// A bf16 [B, N] operand that is still the per-slice partial sums of a split-K product: the consumer adds
// the slices in order, applies the row scale and rounds to bf16, exactly as the finalize kernel would.
// splits == 0: the operand is an ordinary bf16 tensor.
struct GemvPartials {
  const float* partial;
  const uint16_t* scale;
  int splits;
};
// First norm as launch_rmsnorm (x may be partial sums); with w2 a second norm without residual of the
// first result goes to out2 in the same launch. H * 4 bytes of shared memory: H <= 8192.
void launch_rmsnorm_fused(const uint16_t* x, GemvPartials gp, const uint16_t* res, const uint16_t* w, uint16_t* out,
                          const uint16_t* w2, uint16_t* out2, int rows, int H, float eps, float eps2,
                          cudaStream_t stream);
void launch_rope_kv(const uint16_t* qkv, const int32_t* pos, const uint16_t* qw, const uint16_t* kw, uint16_t* q_out,
                    uint16_t* kcache, uint16_t* vcache, int B, int n_q, int n_kv, int D, int T, float theta, float eps,
                    cudaStream_t stream, GemvPartials gp = GemvPartials{nullptr, nullptr, 0});
int attn_decode_splits(int B);
size_t attn_decode_scratch_bytes(int B, int n_q, int splits);
void launch_attn_decode(const uint16_t* q, const int32_t* pos, const uint16_t* kcache, const uint16_t* vcache,
                        uint16_t* out, float* scratch, int B, int n_q, int T, int window, float scale, int splits,
                        cudaStream_t stream);
void launch_geglu(const uint16_t* gu, uint16_t* out, int B, int I, cudaStream_t stream,
                  GemvPartials gp = GemvPartials{nullptr, nullptr, 0});
// block-quantised GEMV: W [N, K] int8, scale bf16 and zp int8 (or null) [N, K / bs], bs a multiple of 16, batch <= 8
void launch_gemv_q8b(const uint16_t* x, const int8_t* W, const uint16_t* scale, const int8_t* zp, uint16_t* y, int B, int N,
                     int K, int bs, cudaStream_t stream);
void launch_act_bf16(const uint16_t* x, uint16_t* out, long long n, int fn, cudaStream_t stream);  // fn: see TB200_OP_ACT_BF16
size_t argmax_scratch_bytes(int B);
void launch_argmax(const void* logits, int is_f32, int32_t* out, void* scratch, int B, int V, cudaStream_t stream);

// ---- whole decode step as one persistent kernel (decode_step.cu) ----
// Byte offsets: weights and norm vectors into the constant image, caches into the arena.
struct DecodeLayerDesc {
  unsigned long long w_qkv, s_qkv, w_o, s_o, w_gu, s_gu, w_down, s_down;
  unsigned long long in_norm, post_attn_norm, pre_ffn_norm, post_ffn_norm, q_norm, k_norm;
  unsigned long long kcache, vcache;
  float theta;
  int window;
  int rope_table;  // which of DecodeStepArgs::theta this layer rotates with
  int pad_;
};
struct DecodeStepArgs {
  const char* consts;
  char* arena;
  char* scratch;
  const int32_t* tokens;  // [B]
  const int32_t* pos;     // [1]
  int32_t* out_ids;       // [B]
  float* logits;          // [B, V] or null
  int* status;            // device status word
  unsigned long long layers_off, embed_w, embed_s, lm_w, lm_s, final_norm;  // constant-image offsets
  unsigned long long counter_off, qkv_off, o_off, act_off, d_off, attn_ml_off, attn_part_off, attn_out_off, amax_off;  // scratch offsets
  unsigned long long trace_off;  // scratch offset of the stage timestamps, 0 = tracing off
  int trace_len;
  int n_layers, B, H, n_q, I, V, V_embed, T;  // V: rows of the LM head (this GPU's shard), V_embed: of the embedding table
  int attn_slices, nslots, xin_stride, xin_bytes, grid;
  float eps, attn_scale, embed_mult;
  float theta[2];  // the (at most two) RoPE bases of the layers
  // tensor parallelism: this GPU's rank, the group size, every member's scratch area as mapped
  // into this process (peer_scratch[rank] == scratch), the inboxes of the K-split projections
  // (scratch offsets, fp32 [tp][B][H]) and the first vocabulary row of this GPU's LM-head shard
  int tp, rank, vocab_offset;
  int o_k, o_k_offset;  // K of the o projection and where its slice starts in the local attention output
  unsigned long long inbox_o_off, inbox_d_off;
  char* peer_scratch[8];
  unsigned long long wait_ns;  // limit of every bounded wait inside the kernel (filled by the launcher)
};
bool decode_step_supported(int B, int H, int n_q, int n_kv, int D, int I, int V);
// fills the scratch offsets and the slice count of `offsets`; returns the scratch size
size_t decode_step_scratch_bytes(int B, int H, int n_q, int I, int n_layers, int sm_count, int tp, DecodeStepArgs* offsets);
cudaError_t launch_decode_step(DecodeStepArgs a, cudaStream_t stream);

// ---- tensor ops outside the layer set (generic_ops.cu); dtypes are enum tb200_dtype values ----
struct EwArgs {
  const void* a;
  const void* b;   // null for a unary function
  void* out;
  long long n;     // output elements
  int fn, arg;     // enum tb200_ew_fn and its argument
  int a_dtype, b_dtype, out_dtype;
  int in_zp, out_zp, clamp_min, clamp_max;
  float fmin, fmax;
  int bool_result;
  int contiguous;  // both operands have the output's shape: element i of each meets element i of the result
  int dims[4];     // output extents (leading dimensions padded with 1)
  int a_str[4], b_str[4];  // element strides of the operands per output dimension, 0 where they broadcast
};
void launch_ew(const EwArgs& a, cudaStream_t stream);
struct RescaleGenericArgs {
  const void* x;
  void* out;
  const int32_t* mult;
  const int8_t* shift;
  long long n;
  int C, per_channel, in_dtype, out_dtype, input_unsigned;
  int in_zp, out_zp, double_round;
  long long clamp_min, clamp_max;
};
void launch_rescale_generic(const RescaleGenericArgs& a, cudaStream_t stream);
struct StridedCopyArgs {
  const void* in;
  void* out;
  long long n;            // elements visited = product of dims
  int elem_bytes;         // bytes moved per index: 1, 2 or 4 (the element), or 8 / 16 after widen_strided_copy
  int pad_elem_bytes;     // the tensor's element size (pad_value is one such element)
  int dims[6];            // extents of the index space (of the output region written); slot 5 is the innermost, unused leading slots are 1
  int lo[6], in_dims[6];  // input coordinate = index - lo, valid inside [0, in_dims)
  long long in_str[6], out_str[6], in_offset, out_offset;  // in elements
  int pad_value;
};
void launch_strided_copy(const StridedCopyArgs& a, cudaStream_t stream);
// Regroups the innermost dimension into 16-, 8- or 4-byte pieces when it is dense on both sides and every
// extent, offset and stride allows it (host side, plan time).
void widen_strided_copy(StridedCopyArgs& a);
struct ReduceArgs {
  const void* x;
  void* out;
  int outer, axis, inner;  // x viewed as [outer, axis, inner]
  int fn;                  // 0 sum, 1 max, 2 min, 3 argmax, 4 mean (floats)
  int in_dtype, out_dtype;
};
void launch_reduce(const ReduceArgs& a, cudaStream_t stream);
// tosa.gather / tosa.scatter rows of `row_bytes` bytes: gather out[n, w] = values[n, idx[n, w]]; scatter out[n, idx[n, w]] = updates[n, w]
// (the caller has copied values to out first). Indices outside [0, K) give zero rows / are skipped.
void launch_gather_rows(const void* values, const int32_t* idx, void* out, int N, int K, int W, int row_bytes, cudaStream_t stream);
void launch_scatter_rows(const void* updates, const int32_t* idx, void* out, int N, int K, int W, int row_bytes, cudaStream_t stream);
void launch_matmul_f(const void* a, const void* b, void* out, int M, int K, int N, int in_dtype, int out_dtype, cudaStream_t stream);
struct DepthwiseFArgs {
  const void* x;     // [N, H, W, C]
  const void* w;     // [KH, KW, C, M]
  const void* bias;  // [C * M]
  void* out;         // [N, OH, OW, C * M]
  int dtype;         // TB200_BF16 or TB200_F32, all four tensors
  int N, H, W, C, M, KH, KW, OH, OW, stride_h, stride_w, dil_h, dil_w, pad_t, pad_l;
};
void launch_depthwise_f(const DepthwiseFArgs& a, cudaStream_t stream);
void launch_softmax(const void* x, void* out, long long rows, int cols, int dtype, cudaStream_t stream);
void launch_table16(const int16_t* x, const int16_t* table, int32_t* out, long long n, cudaStream_t stream);

void launch_resize_nn2x(const int8_t* x, int8_t* out, int N, int H, int W, int C, cudaStream_t stream);

}  // namespace tb200
