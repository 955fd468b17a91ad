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
from oracle_exec import run_graph  # noqa: E402
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


def numpy_replay(g, inputs):
    """The same graph through the numpy restatement (only the op kinds the cases use)."""
    vals = {t.id: a for t, a in zip(g.inputs, inputs)}
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
        elif k == "rescale":
            y = onp.rescale(x, op.consts["multiplier"].data, op.consts["shift"].data, a["in0_zp"], a["out_zp"], a["clamp_min"],
                            a["clamp_max"], bool(a["double_round"]), a["requant_mode"])
        elif k == "matmul_i32":
            y = onp.matmul_i32(x, vals[op.inputs[1].id], a["in0_zp"], a["weight_zp"])
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
    for case in CASES:
        g = tosa_frontend.build_graph_from_file(os.path.join(ref_root, "tests", "testdata", case + ".mlir"))
        rng = np.random.default_rng(1234)
        inputs = [rng.integers(-40, 40, t.shape, dtype=NP_DTYPE[t.dtype]) for t in g.inputs]
        want_c = run_graph(g, inputs)
        want_np = numpy_replay(g, inputs)
        for a, b in zip(want_c, want_np):
            assert a.shape == b.shape and (a == b).all(), case
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
