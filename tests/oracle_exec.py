"""Replays a torq_b200 Graph through the CPU oracle, op by op (checker side only)."""
from __future__ import annotations

import numpy as np

from oracle import oracle as oc


def _rq(op, mode=None):
    a = op.attrs
    return oc.Requant(op.consts["multiplier"].data, op.consts["shift"].data, a.get("out_zp", 0),
                      a.get("clamp_min", -128), a.get("clamp_max", 127), per_channel=bool(a.get("per_channel", 0)),
                      double_round=bool(a.get("double_round", 1)), mode=a.get("requant_mode", 0) if mode is None else mode)


def run_graph(graph, inputs, keep_all=False):
    """inputs: list of numpy arrays in graph.inputs order. Returns outputs (and all tensors if keep_all)."""
    vals = {t.id: np.ascontiguousarray(a) for t, a in zip(graph.inputs, inputs)}
    for op in graph.ops:
        a = op.attrs
        x = vals[op.inputs[0].id]
        k = op.kind
        if k == "conv2d":
            y = oc.conv2d(x, op.consts["weights"].data, op.consts["bias"].data, _rq(op),
                          stride=(a["stride_h"], a["stride_w"]), dilation=(a["dil_h"], a["dil_w"]),
                          pad=(a["pad_t"], a["pad_b"], a["pad_l"], a["pad_r"]), input_zp=a["in0_zp"],
                          weight_zp=a["weight_zp"])
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
        elif k == "rescale":
            y = oc.rescale(x, _rq(op), a["in0_zp"])
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
        vals[op.outputs[0].id] = y
    outs = [vals[t.id] for t in graph.outputs]
    return (outs, vals) if keep_all else outs
