/*
 * "torq-b200-ops": the per-dispatch executable format of the B200 backend.
 *
 * It is the sibling of the reference's `torq-fb` flatbuffer
 * (runtime/schemas/torq_executable_def.fbs:11,99-197). Where `torq-fb` carries
 * NPU bit-streams, XRAM segments and host actions, this format carries one
 * record per TorqHL-level layer op, with the operand/attribute lists of
 * compiler/torq/Dialect/TorqHL/TorqHLOps.td (conv2d :119-143, depthwise :145-170,
 * fully_connected :172-190, avg_pool2d :192-208, add :48-69, mul :101-117,
 * table :311-327, maxpool2d :435-453, resize NN :959-968) PLUS the TOSA
 * multiplier[]/shift[] arrays of the tosa.rescale that followed the op, so that
 * the exact host arithmetic (requant mode A) is representable.
 *
 * Layout of a blob (little endian, every section 16-byte aligned):
 *   tb200_ops_header_t
 *   tb200_tensor_t  tensors[n_tensors]
 *   tb200_op_t      ops[n_ops]
 *   int32_t         input_tensor_ids[n_inputs]
 *   int32_t         output_tensor_ids[n_outputs]
 *   uint8_t         constants[const_bytes]      (tensor.const_offset indexes here)
 *
 * Activations are NHWC (rank-4) or [rows, cols] (rank-2); conv weights are OHWI,
 * depthwise weights are [KH, KW, C, 1] exactly as the TOSA fixtures of the
 * reference have them (tests/testdata/tosa_ops/dw_peeling.mlir).
 */
#ifndef TORQ_B200_OPS_H_
#define TORQ_B200_OPS_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TB200_OPS_MAGIC 0x4f323042u /* "B02O" */
#define TB200_OPS_VERSION 1u
#define TB200_OPS_FORMAT_STRING "torq-b200-ops"

/* Element types; numbering follows runtime/schemas/torq_executable_def.fbs:63-75
 * for the types both formats name. */
enum tb200_dtype {
  TB200_I8 = 0,
  TB200_I16 = 1,
  TB200_I32 = 2,
  TB200_F32 = 3,
  TB200_BF16 = 4,
  TB200_I64 = 5,
};

enum tb200_tensor_kind {
  TB200_TENSOR_ACTIVATION = 0, /* intermediate, lives in the executable's arena */
  TB200_TENSOR_INPUT = 1,      /* bound by the caller at dispatch */
  TB200_TENSOR_OUTPUT = 2,     /* bound by the caller at dispatch */
  TB200_TENSOR_CONSTANT = 3,   /* bytes in the constants section */
  TB200_TENSOR_STATE = 4,      /* persistent across dispatches (KV cache); zeroed at create */
};

enum tb200_op_kind {
  TB200_OP_CONV2D = 1,        /* torq_hl.conv2d            */
  TB200_OP_DEPTHWISE = 2,     /* torq_hl.depthwise_conv2d  */
  TB200_OP_FC = 3,            /* torq_hl.fully_connected / torq_hl.matmul with constant B */
  TB200_OP_MAXPOOL = 4,       /* torq_hl.maxpool2d: int8, or int16 in and out (doc/user-manual/ops.md MaxPool2D i16) */
  TB200_OP_AVGPOOL = 5,       /* torq_hl.avg_pool2d (any window; whole-frame = global) */
  TB200_OP_ADD = 6,           /* torq_hl.add : rescale,rescale -> add -> rescale */
  TB200_OP_MUL = 7,           /* torq_hl.mul : rescale,rescale -> mul -> rescale */
  TB200_OP_TABLE = 8,         /* torq_hl.table : out = table[x + 128] */
  TB200_OP_RESCALE = 9,       /* standalone tosa.rescale (torq_hl.fma form): i8 -> i8 on the layer path; any of i8 / i16 / i32 in and
                               * out (TosaToTorqHL/Patterns.cpp:1735-1947) on the generic one, clamped to the result type's range */
  TB200_OP_RESIZE_NN2X = 10,  /* torq_hl.resize_nearest_neighbor, 2x replicate */
  TB200_OP_CONCAT = 11,       /* channel concat of in0,in1 with per-input rescale */
  TB200_OP_SUB = 12,          /* as ADD with in1 negated after its rescale */
  TB200_OP_MATMUL_I32 = 13,   /* raw torq_hl.matmul: int8 [M,K] x int8 [K,N] -> int32, no rescale; B is the constant
                               * `weights`, or (weights = -1) the runtime tensor in1 as in tosa.matmul */
  TB200_OP_RESHAPE = 14,      /* tosa.reshape / tosa.identity: out0 is a view of in0 (no launch); a device copy when out0 is a graph output */
  /* decoder (bf16 activations, int8 per-output-channel weights) */
  TB200_OP_EMBED = 32,        /* gather rows of an int8 table, dequant, * f0 */
  TB200_OP_RMSNORM = 33,      /* y = x * rsqrt(mean(x^2) + f0) * (1 + w)  (bf16) */
  TB200_OP_GEMV_W8 = 34,      /* y[b,n] = (sum_k x[b,k] * W[n,k]) * scale[n]  (fp32 acc) */
  TB200_OP_ROPE_KV = 35,      /* q/k per-head RMSNorm + rotary, append k,v to cache */
  TB200_OP_ATTN_DECODE = 36,  /* single-query GQA attention over the cache */
  TB200_OP_GEGLU = 37,        /* y = gelu_tanh(gate) * up */
  TB200_OP_ADD_BF16 = 38,     /* residual add */
  TB200_OP_ARGMAX = 39,       /* greedy token id from logits; i1 >= 2: over the shards of a tensor-parallel
                               * group of i1 GPUs, this shard's ids offset by i0 */
  TB200_OP_ACT_BF16 = 41,     /* elementwise bf16 activation, i0: 0 sigmoid, 1 tanh-GELU, 2 exp, 3 tanh, 4 SiLU
                               * (SigmoidPattern.cpp:25-232, GeluPattern.cpp:25-283, ExpOpPattern, TrigOpPattern);
                               * computed in fp32 and rounded once, like the reference's host path */
  TB200_OP_GEMV_Q8B = 42,     /* y = x . bf16((W - zp) * scale) with block-wise scales and zero points along K
                               * (ONNX DequantizeLinear(axis=0, block_size=i0) + MatMul, the reference's Gemma form:
                               * tests/testdata/torch_ops/matmul_dql_q8_0.mlir, ExpandWeightsPattern.cpp:350-376);
                               * weights int8 [K, N], bias slot = scales bf16 [K/i0, N], multiplier slot = zero
                               * points int8 [K/i0, N] or -1 */
  /* tensor ops outside the layer set: what the reference's fixtures exercise around the layers
   * (tests/testdata/tosa_ops: cast-*, Elementwise_*, rescale-*, transpose-*, pad_*, identity-stride-offset-*,
   * reduce-*, argmax-*). Dense row-major tensors of rank <= 4, element types i8 / i16 / i32 / f32 / bf16;
   * a boolean (i1) tensor is an i8 tensor holding 0 or 1. */
  TB200_OP_EW = 48,           /* elementwise, i0 = enum tb200_ew_fn, i1 = its argument (tosa.mul shift, tosa.arithmetic_right_shift
                               * round). Unary (in1 = -1) or binary; both operands and the result have the same rank and an
                               * extent-1 dimension of an operand is broadcast. Integers are computed in int32 (wrapping) and
                               * truncated to the result type, floats in fp32 and rounded once (nearest even). NEGATE uses
                               * in0_zp / out_zp, CLAMP uses clamp_min / clamp_max (integers) or f0 / f1 (floats). */
  TB200_OP_TRANSPOSE = 49,    /* tosa.transpose: out dimension d is in dimension i<d> (i0..i3) */
  TB200_OP_SLICE = 50,        /* tosa.slice / tensor.extract_slice with unit strides: i0..i3 = first index per dimension */
  TB200_OP_PAD = 51,          /* tosa.pad: i0..i3 = leading padding per dimension, pad_value = the constant */
  TB200_OP_CONCAT_AXIS = 52,  /* tosa.concat of in0, in1 along axis i0 (plain copy, any element type) */
  TB200_OP_REDUCE = 53,       /* tosa.reduce_sum / reduce_max / reduce_min / argmax along axis i1: i0 = 0 sum, 1 max, 2 min,
                               * 3 argmax, 4 mean (floats). The result's shape is whatever the op record's output tensor says (the axis kept
                               * with extent 1, or dropped): only its element count matters. Integer sums wrap in int32; float sums and means (ReduceMeanPattern.cpp:37-466) add in fp32 in index order;
                               * argmax gives the first index of the maximum as i32 */
  TB200_OP_TABLE16 = 54,      /* tosa.table on int16: 513-entry int16 table, linear interpolation over the low 7 bits, int32 result
                               * (base << 7) + (next - base) * fraction; the reference's i16 table op is ExtractPattern.cpp:439-545 */
  TB200_OP_SOFTMAX = 55,      /* softmax over the last axis of a bf16 / f32 tensor: subtract the row maximum, exp, sum, multiply by the
                               * reciprocal (the order of SoftmaxPattern.cpp:23-333); fp32 inside, one rounding to the result type */
  TB200_OP_CONV2D_I16 = 56,   /* Conv2D on int16 activations with int8 weights (doc/user-manual/ops.md: "Conv2D i16 i8 -> i32, TOSA specifies
                               * i48 output"; fixture tests/testdata/gen_ops/conv2d_64x64_i16.mlir) fused with the tosa.rescale
                               * {scale32 = false} that follows it: 64-bit accumulator + bias (i64[OC] or i64[1]), TOSA apply_scale_16
                               * (acc * multiplier + 2^(shift-1)) >> shift with a 16-bit multiplier, single rounding, + out_zp, clamp,
                               * int16 result. Attributes as CONV2D. */
  TB200_OP_PERMUTE = 57,      /* a transpose of more than four dimensions (depth-to-space and the like: tosa.reshape -> tosa.transpose ->
                               * tosa.reshape): the input, whatever its stored shape, is viewed as a dense tensor of rank r <= 6 with extents
                               * i0 = d0 | d1 << 16, i1 = d2 | d3 << 16, i2 = d4 | d5 << 16, permuted by i3 = p0 | p1 << 4 | ... | r << 24 and
                               * stored densely; the output tensor only needs the same element count */
  TB200_OP_GATHER = 58,       /* tosa.gather: in0 values [N, K, C], in1 indices [N, W] (i32) -> [N, W, C]; out[n, w, :] = values[n, indices[n, w], :]
                               * (doc/user-manual/ops.md: Gather i8 / i16 / i32). An index outside [0, K) reads as zero. */
  TB200_OP_SCATTER = 59,      /* tosa.scatter: a copy of in0 values [N, K, C] in which row indices[n, w] (in1, i32 [N, W]) is replaced by in2
                               * updates[n, w, :]; indices of one n are distinct (TOSA), an index outside [0, K) is skipped */
  TB200_OP_MATMUL_F = 60,     /* tosa.matmul on floats (doc/user-manual/ops.md: MatMul bf16 x bf16 -> f32): in0 [M, K] x in1 [K, N], bf16 or f32
                               * operands, products and sums in fp32, each rounded, added in index order of k; result f32 or bf16 */
  TB200_OP_DEPTHWISE_F = 61,  /* tosa.depthwise_conv2d on floats (doc/user-manual/ops.md: DepthwiseConv2D bf16): in0 [N, H, W, C], in1 weights
                               * [KH, KW, C, M], in2 bias [C * M], all bf16 or all f32 -> [N, OH, OW, C * M]; fp32 products, each rounded,
                               * added tap by tap in (kh, kw) order (taps outside the frame skipped), the bias last; kh, kw, stride, pad, dil as for depthwise */
  TB200_OP_ALLREDUCE = 40,    /* sum of the fp32 partial results of the i0 GPUs of a tensor-parallel group
                               * (this one is rank i1), rounded to bf16; only inside the fused decode step */
};

enum tb200_ew_fn {
  /* unary */
  TB200_EW_CAST = 0, TB200_EW_ABS = 1, TB200_EW_NEGATE = 2, TB200_EW_BITWISE_NOT = 3, TB200_EW_LOGICAL_NOT = 4,
  TB200_EW_CLZ = 5, TB200_EW_CLAMP = 6, TB200_EW_CEIL = 7, TB200_EW_FLOOR = 8,
  /* unary, floats only, evaluated in fp32 (tolerance class: the function's last bits differ between math libraries) */
  TB200_EW_EXP = 9, TB200_EW_LOG = 10, TB200_EW_RECIPROCAL = 11, TB200_EW_RSQRT = 12, TB200_EW_TANH = 13,
  TB200_EW_SIGMOID = 14, TB200_EW_ERF = 15,
  /* binary */
  TB200_EW_ADD = 16, TB200_EW_SUB = 17, TB200_EW_MUL = 18, TB200_EW_MAX = 19, TB200_EW_MIN = 20,
  TB200_EW_AND = 21, TB200_EW_OR = 22, TB200_EW_XOR = 23, TB200_EW_LSL = 24, TB200_EW_ASR = 25,
  TB200_EW_EQ = 26, TB200_EW_GT = 27, TB200_EW_GE = 28, TB200_EW_LOGICAL_AND = 29, TB200_EW_LOGICAL_OR = 30,
  TB200_EW_LOGICAL_XOR = 31,
};

/* tb200_op_t::flags of TB200_OP_RESCALE and TB200_OP_EW (CAST) */
#define TB200_FLAG_INPUT_UNSIGNED 1u  /* tosa.rescale input_unsigned: the input bytes are uint8 / uint16 */
#define TB200_FLAG_OUTPUT_UNSIGNED 2u /* tosa.rescale output_unsigned */
#define TB200_FLAG_BOOL_RESULT 4u     /* the result is a boolean (0 / 1 in an i8 tensor): CAST writes x != 0 */

enum tb200_requant_mode {
  TB200_REQUANT_TOSA = 0, /* (A) TOSA apply_scale_32, the host/llvm-cpu arithmetic */
  TB200_REQUANT_NPU = 1,  /* (B) common shift, round-to-nearest ties to +inf
                             (compiler/torq/Utils/Kernel.h:607-635) */
};

typedef struct tb200_ops_header {
  uint32_t magic;
  uint32_t version;
  uint32_t n_tensors;
  uint32_t n_ops;
  uint32_t n_inputs;
  uint32_t n_outputs;
  uint64_t tensors_offset;
  uint64_t ops_offset;
  uint64_t inputs_offset;
  uint64_t outputs_offset;
  uint64_t const_offset;
  uint64_t const_bytes;
  uint64_t total_bytes;
} tb200_ops_header_t;

typedef struct tb200_tensor {
  uint32_t dtype;
  uint32_t kind;
  uint32_t rank;        /* 1..4 */
  int32_t shape[4];     /* unused trailing dims are 1 */
  uint32_t reserved;
  uint64_t const_offset; /* TB200_TENSOR_CONSTANT only */
  uint64_t const_bytes;
} tb200_tensor_t;

typedef struct tb200_op {
  uint32_t kind;
  uint32_t flags;
  int32_t in0, in1, in2;  /* tensor ids, -1 = unused */
  int32_t out0, out1;
  int32_t weights;        /* constant tensor ids, -1 = none */
  int32_t bias;           /* i32[OC] or i32[1] */
  int32_t multiplier;     /* i32[OC] or i32[1] */
  int32_t shift;          /* i8[OC] or i8[1] */
  int32_t table;          /* i8[256] */
  int32_t kh, kw, stride_h, stride_w, dil_h, dil_w;
  int32_t pad_t, pad_b, pad_l, pad_r; /* TOSA order top,bottom,left,right */
  int32_t in0_zp, in1_zp, weight_zp, out_zp;
  int32_t clamp_min, clamp_max;
  int32_t per_channel;    /* multiplier/shift have OC entries */
  int32_t double_round;   /* tosa.rescale rounding_mode == DOUBLE_ROUND */
  int32_t requant_mode;   /* enum tb200_requant_mode */
  int32_t in0_mult, in0_shift; /* input-side rescale of ADD/MUL/CONCAT (scalar) */
  int32_t in1_mult, in1_shift;
  int32_t out_mult, out_shift; /* output rescale of elementwise ops (scalar) */
  int32_t pad_value;      /* MAXPOOL: constant of the folded tosa.pad */
  int32_t i0, i1, i2, i3; /* op-specific (decoder: heads, kv heads, head_dim, window; ADD/SUB/MUL: i0, i1 =
                             left shift of (in0 - zp), (in1 - zp) before the input-side rescale, 0..22) */
  float f0, f1, f2, f3;   /* op-specific (eps, rope theta, scale) */
} tb200_op_t;

#ifdef __cplusplus
}
#endif
#endif /* TORQ_B200_OPS_H_ */
