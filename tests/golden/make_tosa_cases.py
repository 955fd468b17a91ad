"""Generates tests/golden/tosa_*.b200ops / tosa_*.npz from the reference's own TOSA fixtures.

Run where the reference tree is available:  python tests/golden/make_tosa_cases.py <path of the reference tree>

For each chosen fixture the TOSA text is read by torq_b200.tosa_frontend (so the constants -
weights, multipliers, shifts, zero points, pad values - are the reference's own), serialized
to a torq-b200-ops blob, and run through BOTH oracle restatements on the reference harness's
seeded input (numpy default_rng(1234), integers in [-40, 40),
python/torq/testing/iree.py:1256-1285). The two must agree; the blob, the input and the
agreed output are stored. The reference holds no expected outputs of its own (it compares
engines), so these files pin the constants and the op forms, and freeze the oracle's answer.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
for p in (ROOT, os.path.join(ROOT, "torq-compiler_b200"), os.path.join(ROOT, "tests")):
    sys.path.insert(0, p)

from oracle import oracle_np as onp  # noqa: E402
from oracle_exec import outputs_match, run_graph, uses_float_functions  # noqa: E402
from torq_b200 import tosa_frontend  # noqa: E402
from torq_b200.oplist import NP_DTYPE  # noqa: E402

# every fixture of tests/testdata/{tosa_ops,gen_ops} that the front end reads and every engine here runs, with at
# most 1.3 M input + output elements (the larger ones are left out)
CASES = [
    "tosa_ops/add", "tosa_ops/add-rank2", "tosa_ops/add-single-rescale", "tosa_ops/add_dense_8x8x24xi8",
    "tosa_ops/add_strided_7x7x24xi8", "tosa_ops/avgpool2d", "tosa_ops/clamp-int8", "tosa_ops/conv_5x5_odd_frame_stride2",
    "tosa_ops/disable-avgpool", "tosa_ops/disable-resize-nearest-neighbor-10x10x512xi8",
    "tosa_ops/disable-resize-nearest-neighbor-20x20x256xi8", "tosa_ops/disable-sub",
    "tosa_ops/dw_21x21_odd_frame_stride2", "tosa_ops/dw_4x4_stride2", "tosa_ops/dw_peeling",
    "tosa_ops/efficientnet-sigmoid-rescale-mul", "tosa_ops/identity-4x16x16", "tosa_ops/identity-56-i8",
    "tosa_ops/identity-64-i8", "tosa_ops/matmul-in-int8-out-int32", "tosa_ops/matmul-in-int8-out-int32-1",
    "tosa_ops/matmul-in-int8-out-int32-2", "tosa_ops/matmul-in-int8-out-int32-3",
    "tosa_ops/matmul-in-int8-out-int32-noalign", "tosa_ops/maxpool-seg-tile", "tosa_ops/maxpool-seg-tile-1",
    "tosa_ops/maxpool1d_i16_stride4_k4x1_256x16x32", "tosa_ops/maxpool1d_i8_stride4_k4x1_256x16x32",
    "tosa_ops/maxpool2d-stride1-k3x3-32x32x4", "tosa_ops/maxpool2d-stride1-k3x3-32x32x4-i16",
    "tosa_ops/maxpool2d-stride2-k2x2-32x32x4", "tosa_ops/maxpool2d-stride2-k2x2-8x8x1",
    "tosa_ops/maxpool2d-stride2-k2x2-8x8x32", "tosa_ops/maxpool2d-stride2-k2x2-8x8x4",
    "tosa_ops/maxpool2d-stride2-k3x3-32x32x4", "tosa_ops/maxpool2d-stride2-k3x3-8x8x4",
    "tosa_ops/maxpool2d-stride2-k3x3-bottom-right-pad", "tosa_ops/maxpool2d-stride2-k3x3-pad-112x112x64",
    "tosa_ops/maxpool2d-stride2-k3x3-pad-32x32x64", "tosa_ops/maxpool2d-stride2-k3x3-top-left-pad",
    "tosa_ops/maxpool2d_i16_s2_k3x3_32x32x4", "tosa_ops/maxpool2d_i16_s2_k7x7_10x10x4",
    "tosa_ops/maxpool2d_int8_batch1_2x2_stride2x2_32x16x4", "tosa_ops/maxpool_f5_15x20x384", "tosa_ops/maxpool_f5_8x8x4",
    "tosa_ops/maxpool_f5_s2_10x10x4", "tosa_ops/maxpool_f5_s2_top_left_pad_10x10x4", "tosa_ops/maxpool_f7_8x8x4",
    "tosa_ops/maxpool_f7_s2_10x10x4", "tosa_ops/maxpool_f7_s2_top_left_pad_10x10x4",
    "tosa_ops/maxpool_int16_batch1_3x3_stride1x1_16x4", "tosa_ops/maxpool_int8_batch1_3x3_stride1x1_16x4",
    "tosa_ops/reshape", "tosa_ops/resize-31x31x33xi8", "tosa_ops/resize-4x4x32xi8", "tosa_ops/resize-8x8x32xi8",
    "tosa_ops/sub-1input-56x56x24xi8", "tosa_ops/sub-1input-strided-7x7x24xi8", "tosa_ops/yolov8_block_mul_rescale",
    "gen_ops/add_8x8", "gen_ops/add_8x8_i8", "gen_ops/conv2d_64x64", "gen_ops/conv2d_8x8", "gen_ops/maxpool2d_8x8",
]


# the tensor ops outside the layer set (casts, elementwise integer / float ops, rescales between integer types,
# transposes, slices, pads, reductions): every further fixture the front end reads with at most 150 k elements
GENERIC_CASES = [
    "tosa_ops/dw_16x16-bf16", "tosa_ops/dw_f5_16x16-bf16",  # bf16 depthwise convolutions, fp32 accumulation
    "tosa_ops/conv2d_1x1_size1_bias_matmul_as_conv-i8",      # a 1x1 convolution of two runtime tensors (a matmul)
    "tosa_ops/multioutput",                                  # one result returned twice
    # functions with a dynamic leading extent, specialised to 1 as the reference's harness draws them
    "gen_ops/abs_1x65x3x6xi32", "gen_ops/abs_1x65x4x3x6xf32", "gen_ops/abs_1x65xi32", "gen_ops/abs_65x6xi16", "gen_ops/abs_65xi32",
    "tosa_ops/mbv2-softmax-i8",  # the decomposed int8 softmax: 42 integer ops incl. four interpolated int16 tables
    "tosa_ops/Elementwise_add-i32", "tosa_ops/Elementwise_bitwise_and-i16-scalar",
    "tosa_ops/Elementwise_bitwise_and-i16", "tosa_ops/Elementwise_bitwise_and-i32",
    "tosa_ops/Elementwise_bitwise_and-i8", "tosa_ops/Elementwise_bitwise_not-i16",
    "tosa_ops/Elementwise_bitwise_not-i32", "tosa_ops/Elementwise_bitwise_not-i8",
    "tosa_ops/Elementwise_bitwise_or-i16", "tosa_ops/Elementwise_bitwise_or-i32",
    "tosa_ops/Elementwise_bitwise_or-i8", "tosa_ops/Elementwise_bitwise_xor-i16",
    "tosa_ops/Elementwise_bitwise_xor-i32", "tosa_ops/Elementwise_bitwise_xor-i8", "tosa_ops/Elementwise_eq-bf16",
    "tosa_ops/Elementwise_eq-i32", "tosa_ops/Elementwise_gt-bf16", "tosa_ops/Elementwise_gt-i32",
    "tosa_ops/Elementwise_gteq-bf16", "tosa_ops/Elementwise_gteq-i32", "tosa_ops/Elementwise_logical_and",
    "tosa_ops/Elementwise_logical_not", "tosa_ops/Elementwise_logical_or", "tosa_ops/Elementwise_logical_xor",
    "tosa_ops/Elementwise_max-bf16", "tosa_ops/Elementwise_max-i32", "tosa_ops/Elementwise_min-bf16",
    "tosa_ops/Elementwise_min-i32", "tosa_ops/Elementwise_sub-i32", "tosa_ops/abs-bf16", "tosa_ops/abs-fp32",
    "tosa_ops/abs-int32-4", "tosa_ops/abs-int32", "tosa_ops/add-16x16x128xi16", "tosa_ops/add-broadcast",
    "tosa_ops/add-constant", "tosa_ops/add-i32-3d", "tosa_ops/add-rank6", "tosa_ops/add-rescale-reshape-padding-i8",
    "tosa_ops/add-rescaled-bias-broadcast-i8", "tosa_ops/add-strided-scalar-i32", "tosa_ops/argmax-1x128x7-2axis",
    "tosa_ops/argmax-1x256x50-2axis", "tosa_ops/argmax-1x4x64-1axis", "tosa_ops/argmax-1x50x256-1axis",
    "tosa_ops/argmax-1x64x4-2axis", "tosa_ops/argmax-1x64x8-2axis", "tosa_ops/argmax-1x7x128-1axis",
    "tosa_ops/argmax-1x8x64-1axis", "tosa_ops/asr-1x21x1024xi32", "tosa_ops/cast-bf16-to-f32",
    "tosa_ops/cast-bf16-to-i16", "tosa_ops/cast-bf16-to-i32", "tosa_ops/cast-bf16-to-i8",
    "tosa_ops/cast-f32-to-bf16", "tosa_ops/cast-f32-to-i16", "tosa_ops/cast-f32-to-i32", "tosa_ops/cast-f32-to-i8",
    "tosa_ops/cast-i1-to-i16", "tosa_ops/cast-i16-to-bf16", "tosa_ops/cast-i16-to-f32", "tosa_ops/cast-i16-to-i32",
    "tosa_ops/cast-i16-to-i8", "tosa_ops/cast-i32-to-bf16", "tosa_ops/cast-i32-to-f32", "tosa_ops/cast-i32-to-i16",
    "tosa_ops/cast-i32-to-i8", "tosa_ops/cast-i8-to-bf16", "tosa_ops/cast-i8-to-f32", "tosa_ops/cast-i8-to-i16",
    "tosa_ops/cast-i8-to-i32", "tosa_ops/ceil-bf16", "tosa_ops/ceil-fp32", "tosa_ops/clamp-fp32",
    "tosa_ops/clamp-int16", "tosa_ops/clz-int32", "tosa_ops/concat-a",
    "tosa_ops/disable-mul-1hwc-rescale-in-int8-out-int32-nonalign",
    "tosa_ops/disable-mul-1hwc-rescale-in-int8-out-int32", "tosa_ops/disable-mul-i32", "tosa_ops/floor-bf16",
    "tosa_ops/floor-fp32", "tosa_ops/identity-4x16x16-i16", "tosa_ops/identity-4x16x16-i32",
    "tosa_ops/identity-64-i16", "tosa_ops/identity-64-i32", "tosa_ops/identity-stride-offset-123x120xi8",
    "tosa_ops/identity-stride-offset-6x15x5xi8", "tosa_ops/identity-stride-offset-6x15x70xi8",
    "tosa_ops/identity-stride-offset-6x6xi8", "tosa_ops/matmul-in-int8-out-int16",
    "tosa_ops/matmul-in-int16-out-int16", "tosa_ops/matmul-in-int16-out-int32",
    "tosa_ops/matmul-in-int8-out-int16-64x128x2048", "gen_ops/conv2d_64x64_i16",
    # transposes of five and six dimensions (depth-to-space, space-to-depth), gather / scatter, and fixtures that only
    # needed a collapsed view or a larger size limit
    "tosa_ops/Elementwise_max_broadcast_clip-i8", "tosa_ops/Elementwise_min_broadcast_clip-i8", "tosa_ops/add-32x32x128xi16",
    "tosa_ops/add-56x56x256", "tosa_ops/add-bf16", "tosa_ops/add-i32",
    "tosa_ops/clamp-bf16", "tosa_ops/css_scalar", "tosa_ops/d2s_16x16x128xi16_crd",
    "tosa_ops/d2s_16x16x128xi16_dcr", "tosa_ops/d2s_16x16x128xi8_crd", "tosa_ops/d2s_16x16x128xi8_dcr",
    "tosa_ops/d2s_8x8x128xi16_crd", "tosa_ops/d2s_8x8x128xi16_dcr", "tosa_ops/d2s_8x8x128xi8_crd",
    "tosa_ops/d2s_8x8x128xi8_dcr", "tosa_ops/d2s_8x8x4xi16", "tosa_ops/d2s_8x8x4xi8",
    "tosa_ops/d2s_9x9x128xi16_dcr", "tosa_ops/disable-maxpool-tile", "tosa_ops/gather-i16",
    "tosa_ops/gather-i32", "tosa_ops/gather", "tosa_ops/identity-2x5x2x16x8x2-i16",
    "tosa_ops/identity-2x5x2x16x8x2-i32", "tosa_ops/identity-2x5x2x16x8x2-i8", "tosa_ops/identity-stride-offset-3x4x2x70xi8",
    "tosa_ops/matmul-in-int8-out-int16-1024x128x1024", "tosa_ops/matmul-notile", "tosa_ops/s2d_16x16x1xi8",
    "tosa_ops/scatter-single-channel", "tosa_ops/scatter", "tosa_ops/scatter_1",
    "tosa_ops/sub-56x56x256xi8", "tosa_ops/sub-bf16", "tosa_ops/sub-i32",
    "tosa_ops/sub-rescale-scalar-bis", "tosa_ops/sub-rescale-scalar", "tosa_ops/transpose-5dim",
    "tosa_ops/transpose-5dim_1", "tosa_ops/transpose-5dim_2", "tosa_ops/transpose-5dim_3",
    "tosa_ops/add-scalar", "tosa_ops/concat-b", "tosa_ops/sub-rescale-tensor-int8",
    # float matmul (fp32 products and sums in index order: bit-exact) and the float functions (tolerance class)
    "tosa_ops/disable-matmul-bf16", "tosa_ops/disable-matmul-in-bf16-out-bf16_207x207", "tosa_ops/matmul-fp32",
    "tosa_ops/matmul-in-bf16-out-fp32_207x207", "tosa_ops/matmul-in-bf16-out-fp32_2x2", "tosa_ops/softmax-1x1000xi8",
    "tosa_ops/mul-1hw1-in-int8-out-int32", "tosa_ops/mul-1hwc-in-int16-out-int32",
    "tosa_ops/mul-1hwc-in-int8-out-int32-1", "tosa_ops/mul-1hwc-in-int8-out-int32-2dim",
    "tosa_ops/mul-1hwc-in-int8-out-int32-3dim", "tosa_ops/mul-1hwc-in-int8-out-int32", "tosa_ops/mul-bf16",
    "tosa_ops/mul-broadcast-i16", "tosa_ops/mul-broadcast", "tosa_ops/mul-scalar", "tosa_ops/negate-bf16",
    "tosa_ops/negate-fp32", "tosa_ops/negate-int16", "tosa_ops/negate-int32", "tosa_ops/negate",
    "tosa_ops/pad_TL_4x8x8", "tosa_ops/pad_TL_8x8x4", "tosa_ops/reduce-max-f32", "tosa_ops/reduce-max-i32",
    "tosa_ops/reducesum-avgpool", "tosa_ops/rescale-const-input-output-zp", "tosa_ops/rescale-i16-i32",
    "tosa_ops/rescale-i32-i16", "tosa_ops/rescale-i32-i32", "tosa_ops/rescale-i32-i8", "tosa_ops/rescale-i8-i32",
    "tosa_ops/rescale-in-int16-out-int8", "tosa_ops/rescale-in-int32-out-int8", "tosa_ops/rescale-in-int8-out-int16",
    "tosa_ops/rescale-in-int8-out-int32-2dim-nonalign", "tosa_ops/rescale-in-int8-out-int32-2dim",
    "tosa_ops/rescale-in-int8-out-int32-3dim-nonalign", "tosa_ops/rescale-in-int8-out-int32-3dim",
    "tosa_ops/rescale-in-int8-out-int32", "tosa_ops/rescale-in-int8-out-uint8", "tosa_ops/rescale-in-uint8-out-int8",
    "tosa_ops/rescale-rank1", "tosa_ops/rescale-scalar", "tosa_ops/sub-broadcast-1", "tosa_ops/sub-broadcast",
    "tosa_ops/sub-constant-1", "tosa_ops/sub-constant-bf16", "tosa_ops/sub-constant-tensor", "tosa_ops/sub-constant",
    "tosa_ops/sub-css", "tosa_ops/sub-scalar-tensor-bf16", "tosa_ops/transpose-2dim-aligned",
    "tosa_ops/transpose-2dim", "tosa_ops/transpose-3dim", "tosa_ops/transpose-3dim_1", "tosa_ops/transpose-3dim_2",
    "tosa_ops/transpose-64x64xi8", "tosa_ops/transpose-95x159xbf16", "tosa_ops/transpose-95x159xi8",
    "tosa_ops/transpose-96x160xi16", "tosa_ops/transpose-96x160xi8", "tosa_ops/transpose",
    
]


def numpy_replay(g, inputs):
    """The same graph through the numpy restatement (only the op kinds the cases use)."""
    vals = {t.id: t.data for t in g.tensors if t.kind == 3 and t.data is not None}
    vals.update({t.id: a for t, a in zip(g.inputs, inputs)})
    for op in g.ops:
        a, x = op.attrs, vals[op.inputs[0].id]
        k = op.kind
        if k in ("conv2d", "depthwise"):
            fn = onp.conv2d if k == "conv2d" else onp.depthwise
            y = fn(x, op.consts["weights"].data, op.consts["bias"].data, op.consts["multiplier"].data,
                   op.consts["shift"].data, a["out_zp"], a["clamp_min"], a["clamp_max"], (a["stride_h"], a["stride_w"]),
                   (a["dil_h"], a["dil_w"]), (a["pad_t"], a["pad_b"], a["pad_l"], a["pad_r"]), a["in0_zp"], a["weight_zp"],
                   bool(a["double_round"]))
        elif k == "maxpool":
            y = onp.maxpool(x, (a["kh"], a["kw"]), (a["stride_h"], a["stride_w"]), (a["pad_t"], a["pad_b"], a["pad_l"], a["pad_r"]),
                            a["pad_value"])
        elif k == "avgpool":
            y = onp.avgpool(x, (a["kh"], a["kw"]), (a["stride_h"], a["stride_w"]), (a["pad_t"], a["pad_b"], a["pad_l"], a["pad_r"]),
                            a["in0_zp"], a["out_zp"])
        elif k in ("add", "sub", "mul"):
            y = onp.binary(k, x, vals[op.inputs[1].id], a["in0_zp"], a["in0_mult"], a["in0_shift"], a["in1_zp"], a["in1_mult"],
                           a["in1_shift"], a["out_mult"], a["out_shift"], a["out_zp"], bool(a["double_round"]), a["clamp_min"],
                           a["clamp_max"], a_lshift=a["i0"], b_lshift=a["i1"])
        elif k == "table":
            y = onp.table(x, op.consts["table"].data)
        elif k == "rescale" and (op.inputs[0].dtype, op.outputs[0].dtype, a.get("flags", 0)) != ("i8", "i8", 0):
            y = onp.rescale_elementwise(x, op.inputs[0].dtype, op.outputs[0].dtype, op.consts["multiplier"].data,
                                        op.consts["shift"].data, a["in0_zp"], a["out_zp"], (a["clamp_min"], a["clamp_max"]),
                                        per_channel=bool(a["per_channel"]), double_round=bool(a["double_round"]),
                                        input_unsigned=bool(a.get("flags", 0) & 1))
        elif k == "ew":
            from oracle.generic_ops import EW_NAMES
            second = vals[op.inputs[1].id] if len(op.inputs) > 1 else None
            y = onp.ew_elementwise(EW_NAMES[a["i0"]], x, op.inputs[0].dtype, second, op.inputs[1].dtype if second is not None else None,
                                   op.outputs[0].dtype, op.outputs[0].shape, arg=a["i1"], in_zp=a["in0_zp"], out_zp=a["out_zp"],
                                   clamp=(a["clamp_min"], a["clamp_max"]), fclamp=(a["f0"], a["f1"]), bool_result=bool(a.get("flags", 0) & 4))
        elif k == "matmul_f":  # one output at a time, numpy float32 scalars: every product and every sum rounded
            bmat = vals[op.inputs[1].id]
            to_f = (lambda v: (v.astype(np.uint32) << 16).view(np.float32)) if op.inputs[0].dtype == "bf16" else (lambda v: v.astype(np.float32))
            xa, xb = to_f(x), to_f(bmat)
            acc = np.zeros((xa.shape[0], xb.shape[1]), np.float32)
            for m_ in range(xa.shape[0]):
                for n_ in range(xb.shape[1]):
                    s_ = np.float32(0)
                    col = xb[:, n_]
                    row = xa[m_]
                    for k_ in range(row.size):
                        s_ = np.float32(s_ + np.float32(row[k_] * col[k_]))
                    acc[m_, n_] = s_
            y = tosa_frontend._to_bf16_bits(acc) if op.outputs[0].dtype == "bf16" else acc
        elif k == "depthwise_f":  # one output at a time, numpy float32 scalars, taps in (kh, kw) order, the bias last
            to_f = (lambda v: (v.astype(np.uint32) << 16).view(np.float32)) if op.inputs[0].dtype == "bf16" else (lambda v: v.astype(np.float32))
            xa, wa, ba = to_f(x), to_f(vals[op.inputs[1].id]), to_f(vals[op.inputs[2].id]).reshape(-1)
            N_, H_, W_, C_ = xa.shape
            KH_, KW_, _, M_ = wa.shape
            _, OH_, OW_, _ = op.outputs[0].shape
            acc = np.zeros(op.outputs[0].shape, np.float32)
            for n_ in range(N_):
                for oh_ in range(OH_):
                    for ow_ in range(OW_):
                        for c_ in range(C_):
                            for m_ in range(M_):
                                s_ = np.float32(0)
                                for kh_ in range(KH_):
                                    ih_ = oh_ * a["stride_h"] - a["pad_t"] + kh_ * a["dil_h"]
                                    for kw_ in range(KW_):
                                        iw_ = ow_ * a["stride_w"] - a["pad_l"] + kw_ * a["dil_w"]
                                        if 0 <= ih_ < H_ and 0 <= iw_ < W_:
                                            s_ = np.float32(s_ + np.float32(xa[n_, ih_, iw_, c_] * wa[kh_, kw_, c_, m_]))
                                acc[n_, oh_, ow_, c_ * M_ + m_] = np.float32(s_ + ba[c_ * M_ + m_])
            y = tosa_frontend._to_bf16_bits(acc) if op.outputs[0].dtype == "bf16" else acc
        elif k == "gather":
            idx = vals[op.inputs[1].id]
            y = np.empty(op.outputs[0].shape, x.dtype)
            for n_ in range(idx.shape[0]):
                for w_ in range(idx.shape[1]):
                    y[n_, w_, :] = x[n_, int(idx[n_, w_]), :]
        elif k == "scatter":
            idx, upd = vals[op.inputs[1].id], vals[op.inputs[2].id]
            y = x.copy()
            for n_ in range(idx.shape[0]):
                for w_ in range(idx.shape[1]):
                    y[n_, int(idx[n_, w_]), :] = upd[n_, w_, :]
        elif k == "permute":  # element by element through flat indices
            r = (a["i3"] >> 24) & 15
            d6 = [a["i0"] & 0xffff, a["i0"] >> 16, a["i1"] & 0xffff, a["i1"] >> 16, a["i2"] & 0xffff, a["i2"] >> 16][:r]
            perm = [(a["i3"] >> (4 * i)) & 15 for i in range(r)]
            in_str = [int(np.prod(d6[i + 1:])) for i in range(r)]
            flat_in = x.reshape(-1)
            flat_out = np.empty(flat_in.size, x.dtype)
            out_dims = [d6[pd] for pd in perm]
            for o, idx in enumerate(np.ndindex(*out_dims)):
                flat_out[o] = flat_in[sum(idx[d] * in_str[perm[d]] for d in range(r))]
            y = flat_out.reshape(op.outputs[0].shape)
        elif k == "transpose":
            perm = [a["i0"], a["i1"], a["i2"], a["i3"]][:x.ndim]
            y = np.empty(op.outputs[0].shape, x.dtype)
            for idx in np.ndindex(*y.shape):  # out[idx] = in[idx permuted back]
                src = [0] * x.ndim
                for d, pd in enumerate(perm):
                    src[pd] = idx[d]
                y[idx] = x[tuple(src)]
        elif k == "slice":
            start = [a["i0"], a["i1"], a["i2"], a["i3"]][:x.ndim]
            y = np.array([x[tuple(s + i for s, i in zip(start, idx))] for idx in np.ndindex(*op.outputs[0].shape)], x.dtype)
        elif k == "pad":
            before = [a["i0"], a["i1"], a["i2"], a["i3"]][:x.ndim]
            y = np.full(op.outputs[0].shape, np.array(a["pad_value"]).astype(x.dtype), x.dtype)
            y[tuple(slice(b0, b0 + d) for b0, d in zip(before, x.shape))] = x
        elif k == "table16":
            y = onp.table16_elementwise(x, op.consts["table"].data)
        elif k == "concat_axis":
            y = np.concatenate([x, vals[op.inputs[1].id]], axis=a["i0"])
        elif k == "reduce":
            moved = np.moveaxis(x, a["i1"], -1).reshape(-1, x.shape[a["i1"]])
            if op.inputs[0].dtype == "bf16":
                moved = (moved.astype(np.uint32) << 16).view(np.float32)
            if a["i0"] in (0, 4) and moved.dtype == np.float32:  # one element at a time in fp32, every sum rounded
                sums = []
                for row in moved:
                    s_ = np.float32(0)
                    for v in row:
                        s_ = np.float32(s_ + v)
                    sums.append(np.float32(s_ / np.float32(row.size)) if a["i0"] == 4 else s_)
                y = np.array(sums, np.float32)
            elif a["i0"] == 0:
                y = np.array([int(sum(int(v) for v in row)) & 0xFFFFFFFF for row in moved], np.uint32).view(np.int32)
            elif a["i0"] == 3:
                y = np.array([int(np.argmax(row)) for row in moved], np.int32)
            else:
                pick = max if a["i0"] == 1 else min
                y = np.array([pick(row.tolist()) for row in moved])
            if op.outputs[0].dtype == "bf16":
                y = (np.asarray(y, np.float32).view(np.uint32) >> 16).astype(np.uint16)  # a max / min of bf16 values is one of them
            y = np.asarray(y).astype(NP_DTYPE[op.outputs[0].dtype])
        elif k == "rescale":
            y = onp.rescale(x, op.consts["multiplier"].data, op.consts["shift"].data, a["in0_zp"], a["out_zp"], a["clamp_min"],
                            a["clamp_max"], bool(a["double_round"]), a["requant_mode"])
        elif k == "conv2d_i16":
            y = onp.conv2d_i16_elementwise(x, op.consts["weights"].data, op.consts["bias"].data, op.consts["multiplier"].data,
                                           op.consts["shift"].data, (a["stride_h"], a["stride_w"]), (a["dil_h"], a["dil_w"]),
                                           (a["pad_t"], a["pad_b"], a["pad_l"], a["pad_r"]), a["in0_zp"], a["weight_zp"],
                                           a["out_zp"], a["clamp_min"], a["clamp_max"])
        elif k == "matmul_i32":
            y = onp.matmul_i32(x, vals[op.inputs[1].id], a["in0_zp"], a["weight_zp"]).astype(NP_DTYPE[op.outputs[0].dtype])
        elif k == "resize_nn2x":
            y = onp.resize_nn2x(x)
        elif k == "reshape":
            y = x.reshape(op.outputs[0].shape)
        else:
            raise NotImplementedError(k)
        vals[op.outputs[0].id] = np.asarray(y).reshape(op.outputs[0].shape)
    return [vals[t.id] for t in g.outputs]


def main(ref_root):
    out_dir = os.path.dirname(os.path.abspath(__file__))
    only = os.environ.get("TOSA_CASES_ONLY")  # "generic": only the second list; or a comma list of case names
    todo = GENERIC_CASES if only == "generic" else only.split(",") if only else CASES + GENERIC_CASES
    for case in todo:
        path = os.path.join(ref_root, "tests", "testdata", case + ".mlir")
        g = tosa_frontend.build_graph_from_file(path)
        rng = np.random.default_rng(1234)
        inputs = []
        with open(path) as f:
            declared, _, _ = tosa_frontend.parse_module(f.read())
        for v, t in zip(declared, g.inputs):  # the reference harness's draw per declared element type
            if v.dtype in ("f32", "bf16"):
                x = rng.uniform(-40, 40, v.shape).astype(np.float32)
                x = tosa_frontend._to_bf16_bits(x) if v.dtype == "bf16" else x
            elif v.dtype == "i1":
                x = rng.integers(0, 2, v.shape).astype(np.int8)
            elif v.dtype == "ui8":
                x = rng.integers(0, 80, v.shape, dtype=np.uint8).view(np.int8)
            else:
                x = rng.integers(-40, 40, v.shape, dtype=NP_DTYPE[t.dtype])
            inputs.append(np.ascontiguousarray(x).reshape(t.shape))
        want_c = run_graph(g, inputs)
        want_np = numpy_replay(g, inputs)
        tolerant = uses_float_functions(g)
        for a, b, t in zip(want_c, want_np, g.outputs):
            assert outputs_match(a, b, tolerant, t.dtype), case
        name = "tosa_" + os.path.basename(case).replace("-", "_")
        with open(os.path.join(out_dir, name + ".b200ops"), "wb") as f:
            f.write(g.serialize())
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **{f"in{i}": a for i, a in enumerate(inputs)},
                            **{f"out{i}": a for i, a in enumerate(want_c)})
        print(name, [op.kind for op in g.ops], [o.shape for o in want_c], "unique", [len(np.unique(o)) for o in want_c])


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_tosa_cases.py <path of the reference tree>")
    main(sys.argv[1])
