"""Replays a torq_b200 Graph through the CPU oracle, op by op (checker side only)."""
from __future__ import annotations

import numpy as np

from oracle import generic_ops as gops
from oracle import oracle as oc


def _rq(op, mode=None):
    a = op.attrs
    return oc.Requant(op.consts["multiplier"].data, op.consts["shift"].data, a.get("out_zp", 0),
                      a.get("clamp_min", -128), a.get("clamp_max", 127), per_channel=bool(a.get("per_channel", 0)),
                      double_round=bool(a.get("double_round", 1)), mode=a.get("requant_mode", 0) if mode is None else mode)


def run_graph(graph, inputs, keep_all=False):
    """inputs: list of numpy arrays in graph.inputs order. Returns outputs (and all tensors if keep_all)."""
    vals = {t.id: t.data for t in graph.tensors if t.kind == 3 and t.data is not None}  # constants used as operands
    vals.update({t.id: np.ascontiguousarray(a) for t, a in zip(graph.inputs, inputs)})
    for op in graph.ops:
        a = op.attrs
        x = vals[op.inputs[0].id]
        k = op.kind
        if k == "conv2d":
            y = oc.conv2d(x, op.consts["weights"].data, op.consts["bias"].data, _rq(op),
                          stride=(a["stride_h"], a["stride_w"]), dilation=(a["dil_h"], a["dil_w"]),
                          pad=(a["pad_t"], a["pad_b"], a["pad_l"], a["pad_r"]), input_zp=a["in0_zp"],
                          weight_zp=a["weight_zp"])
        elif k == "conv2d_i16":
            y = gops.conv2d_i16(x, op.consts["weights"].data, op.consts["bias"].data, op.consts["multiplier"].data,
                                op.consts["shift"].data, stride=(a["stride_h"], a["stride_w"]), dilation=(a["dil_h"], a["dil_w"]),
                                pad=(a["pad_t"], a["pad_b"], a["pad_l"], a["pad_r"]), input_zp=a["in0_zp"],
                                weight_zp=a["weight_zp"], out_zp=a["out_zp"], clamp=(a["clamp_min"], a["clamp_max"]))
        elif k == "depthwise":
            y = oc.depthwise(x, op.consts["weights"].data, op.consts["bias"].data, _rq(op),
                             stride=(a["stride_h"], a["stride_w"]), dilation=(a["dil_h"], a["dil_w"]),
                             pad=(a["pad_t"], a["pad_b"], a["pad_l"], a["pad_r"]), input_zp=a["in0_zp"],
                             weight_zp=a["weight_zp"])
        elif k == "fc":
            y = oc.fully_connected(x, op.consts["weights"].data, op.consts["bias"].data, _rq(op),
                                   input_zp=a["in0_zp"], weight_zp=a["weight_zp"])
        elif k == "matmul_i32":
            rhs = op.consts["weights"].data if "weights" in op.consts else vals[op.inputs[1].id]
            if op.inputs[0].dtype == "i16" or op.outputs[0].dtype == "i16":
                y = gops.matmul_int(x, rhs, a["in0_zp"], a["weight_zp"], op.outputs[0].dtype)
            else:
                y = oc.matmul_i32(x, rhs, a["in0_zp"], a["weight_zp"])
        elif k == "maxpool":
            y = oc.maxpool(x, (a["kh"], a["kw"]), (a["stride_h"], a["stride_w"]),
                           (a["pad_t"], a["pad_b"], a["pad_l"], a["pad_r"]), a["pad_value"])
        elif k == "avgpool":
            y = oc.avgpool(x, (a["kh"], a["kw"]), (a["stride_h"], a["stride_w"]),
                           (a["pad_t"], a["pad_b"], a["pad_l"], a["pad_r"]), a["in0_zp"], a["out_zp"])
        elif k in ("add", "sub", "mul"):
            y = oc.binary(k, x, vals[op.inputs[1].id], a["in0_zp"], a["in0_mult"], a["in0_shift"], a["in1_zp"],
                          a["in1_mult"], a["in1_shift"], a["out_mult"], a["out_shift"], a["out_zp"],
                          bool(a["double_round"]), a["clamp_min"], a["clamp_max"], a_lshift=a["i0"], b_lshift=a["i1"])
        elif k == "table":
            y = oc.table(x, op.consts["table"].data)
        elif k == "rescale" and (op.inputs[0].dtype, op.outputs[0].dtype, a.get("flags", 0)) != ("i8", "i8", 0):
            y = gops.rescale(x, op.inputs[0].dtype, op.outputs[0].dtype, op.consts["multiplier"].data, op.consts["shift"].data,
                             a["in0_zp"], a["out_zp"], (a["clamp_min"], a["clamp_max"]), per_channel=bool(a["per_channel"]),
                             double_round=bool(a["double_round"]), input_unsigned=bool(a.get("flags", 0) & 1),
                             output_unsigned=bool(a.get("flags", 0) & 2))
        elif k == "rescale":
            y = oc.rescale(x, _rq(op), a["in0_zp"])
        elif k == "ew":
            second = vals[op.inputs[1].id] if len(op.inputs) > 1 else None
            y = gops.ew(a["i0"], x, op.inputs[0].dtype, second, op.inputs[1].dtype if second is not None else None,
                        op.outputs[0].dtype, arg=a["i1"], in_zp=a["in0_zp"], out_zp=a["out_zp"],
                        clamp=(a["clamp_min"], a["clamp_max"]), fclamp=(a["f0"], a["f1"]), bool_result=bool(a.get("flags", 0) & 4))
            y = np.broadcast_to(y, op.outputs[0].shape) if y.shape != tuple(op.outputs[0].shape) else y
        elif k == "transpose":
            y = np.transpose(x, [a["i0"], a["i1"], a["i2"], a["i3"]][:x.ndim])
        elif k == "depthwise_f":
            a = op.attrs
            y = gops.depthwise_f(x, vals[op.inputs[1].id], vals[op.inputs[2].id], op.inputs[0].dtype, (a["stride_h"], a["stride_w"]),
                                 (a["dil_h"], a["dil_w"]), (a["pad_t"], a["pad_b"], a["pad_l"], a["pad_r"]))
        elif k == "matmul_f":
            y = gops.matmul_f(x, vals[op.inputs[1].id], op.inputs[0].dtype, op.outputs[0].dtype)
        elif k == "gather":
            y = gops.gather(x, vals[op.inputs[1].id])
        elif k == "scatter":
            y = gops.scatter(x, vals[op.inputs[1].id], vals[op.inputs[2].id])
        elif k == "permute":
            r = (a["i3"] >> 24) & 15
            d6 = [a["i0"] & 0xffff, a["i0"] >> 16, a["i1"] & 0xffff, a["i1"] >> 16, a["i2"] & 0xffff, a["i2"] >> 16]
            y = x.reshape(d6[:r]).transpose([(a["i3"] >> (4 * i)) & 15 for i in range(r)]).reshape(op.outputs[0].shape)
        elif k == "slice":
            start = [a["i0"], a["i1"], a["i2"], a["i3"]][:x.ndim]
            y = x[tuple(slice(s, s + n) for s, n in zip(start, op.outputs[0].shape))]
        elif k == "pad":
            before = [a["i0"], a["i1"], a["i2"], a["i3"]][:x.ndim]
            widths = [(b, o - b - d) for b, o, d in zip(before, op.outputs[0].shape, x.shape)]
            y = np.pad(x, widths, constant_values=np.array(a["pad_value"]).astype(x.dtype))
        elif k == "concat_axis":
            y = np.concatenate([x, vals[op.inputs[1].id]], axis=a["i0"])
        elif k == "softmax":
            y = gops.softmax(x, op.inputs[0].dtype)
        elif k == "table16":
            y = gops.table16(x, op.consts["table"].data)
        elif k == "reduce":
            y = gops.reduce(a["i0"], x, op.inputs[0].dtype, a["i1"], op.outputs[0].shape, op.outputs[0].dtype)
        elif k == "resize_nn2x":
            y = oc.resize_nn2x(x)
        elif k == "concat":
            y = oc.concat2(x, vals[op.inputs[1].id], a["in0_zp"], a["in0_mult"], a["in0_shift"], a["in1_zp"],
                           a["in1_mult"], a["in1_shift"], a["out_zp"], bool(a["double_round"]))
        elif k == "reshape":
            y = x.reshape(op.outputs[0].shape)
        else:
            raise NotImplementedError(k)
        assert tuple(y.shape) == tuple(op.outputs[0].shape), (k, y.shape, op.outputs[0].shape)
        vals[op.outputs[0].id] = np.ascontiguousarray(y)
    outs = [vals[t.id] for t in graph.outputs]
    return (outs, vals) if keep_all else outs


def uses_float_functions(graph) -> bool:
    """Graphs with exp / log / reciprocal / ... or softmax are tolerance-class: the last bits of those functions belong to
    the math library (the reference's own tests compare engines at +-1 LSB, python/torq/testing/comparison.py:42-49)."""
    return any((op.kind == "ew" and 9 <= op.attrs.get("i0", 0) <= 15) or op.kind == "softmax" for op in graph.ops)


def outputs_match(got, want, tolerant: bool, dtype: str = "") -> bool:
    """Bit-exact, or for tolerance-class graphs: integers within 1, bf16 within 2 ulp of the value, f32 within 1e-5 relative."""
    if got.shape != want.shape:
        return False
    if not tolerant:
        return bool((got.view(np.uint8) == want.view(np.uint8)).all()) if got.dtype == want.dtype else False
    if dtype == "bf16":
        a = (got.astype(np.uint32) << 16).view(np.float32)
        b = (want.astype(np.uint32) << 16).view(np.float32)
        return bool(np.all(np.abs(a - b) <= 2.0 ** -7 * np.maximum(np.abs(b), 1e-30)))
    if got.dtype.kind == "f":
        return bool(np.all(np.abs(got - want) <= 1e-5 * np.maximum(np.abs(want), 1e-30) + 1e-30))
    return bool(np.all(np.abs(got.astype(np.int64) - want.astype(np.int64)) <= 1))
