"""Builder and serializer of `torq-b200-ops` executables (include/torq_b200_ops.h).

It stands where the reference's serializer stands
(compiler/torq/Serialization/Serialization.cpp:265-306 writes the `torq-fb`
flatbuffer per dispatch): one record per TorqHL-level op, constants in one blob.
The Graph also keeps every op as a plain Python record (`Graph.ops`) so that a
checker can replay the same graph through another engine.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Any

import numpy as np

MAGIC = 0x4F323042
VERSION = 1
FORMAT_STRING = "torq-b200-ops"

DTYPES = {"i8": 0, "i16": 1, "i32": 2, "f32": 3, "bf16": 4, "i64": 5}
DTYPE_SIZE = {"i8": 1, "i16": 2, "i32": 4, "f32": 4, "bf16": 2, "i64": 8}
NP_DTYPE = {"i8": np.int8, "i16": np.int16, "i32": np.int32, "f32": np.float32, "bf16": np.uint16, "i64": np.int64}

ACTIVATION, INPUT, OUTPUT, CONSTANT, STATE = 0, 1, 2, 3, 4

OP_KINDS = {
    "conv2d": 1, "depthwise": 2, "fc": 3, "maxpool": 4, "avgpool": 5, "add": 6, "mul": 7, "table": 8,
    "rescale": 9, "resize_nn2x": 10, "concat": 11, "sub": 12, "matmul_i32": 13, "reshape": 14,
    "embed": 32, "rmsnorm": 33, "gemv_w8": 34, "rope_kv": 35, "attn_decode": 36, "geglu": 37,
    "add_bf16": 38, "argmax": 39, "allreduce": 40, "act_bf16": 41, "gemv_q8b": 42,
    "ew": 48, "transpose": 49, "slice": 50, "pad": 51, "concat_axis": 52, "reduce": 53, "table16": 54, "softmax": 55, "conv2d_i16": 56, "permute": 57, "gather": 58, "scatter": 59, "matmul_f": 60, "depthwise_f": 61,
}

EW_FN = {"cast": 0, "abs": 1, "negate": 2, "bitwise_not": 3, "logical_not": 4, "clz": 5, "clamp": 6, "ceil": 7, "floor": 8,
         "exp": 9, "log": 10, "reciprocal": 11, "rsqrt": 12, "tanh": 13, "sigmoid": 14, "erf": 15,
         "add": 16, "sub": 17, "mul": 18, "maximum": 19, "minimum": 20, "bitwise_and": 21, "bitwise_or": 22,
         "bitwise_xor": 23, "logical_left_shift": 24, "arithmetic_right_shift": 25, "equal": 26, "greater": 27,
         "greater_equal": 28, "logical_and": 29, "logical_or": 30, "logical_xor": 31}
FLAG_INPUT_UNSIGNED, FLAG_OUTPUT_UNSIGNED, FLAG_BOOL_RESULT = 1, 2, 4
REDUCE_FN = {"sum": 0, "max": 1, "min": 2, "argmax": 3, "mean": 4}


class Header(C.Structure):
    _fields_ = [("magic", C.c_uint32), ("version", C.c_uint32), ("n_tensors", C.c_uint32), ("n_ops", C.c_uint32),
                ("n_inputs", C.c_uint32), ("n_outputs", C.c_uint32), ("tensors_offset", C.c_uint64),
                ("ops_offset", C.c_uint64), ("inputs_offset", C.c_uint64), ("outputs_offset", C.c_uint64),
                ("const_offset", C.c_uint64), ("const_bytes", C.c_uint64), ("total_bytes", C.c_uint64)]


class TensorRec(C.Structure):
    _fields_ = [("dtype", C.c_uint32), ("kind", C.c_uint32), ("rank", C.c_uint32), ("shape", C.c_int32 * 4),
                ("reserved", C.c_uint32), ("const_offset", C.c_uint64), ("const_bytes", C.c_uint64)]


_OP_INT_FIELDS = ["in0", "in1", "in2", "out0", "out1", "weights", "bias", "multiplier", "shift", "table",
                  "kh", "kw", "stride_h", "stride_w", "dil_h", "dil_w", "pad_t", "pad_b", "pad_l", "pad_r",
                  "in0_zp", "in1_zp", "weight_zp", "out_zp", "clamp_min", "clamp_max", "per_channel",
                  "double_round", "requant_mode", "in0_mult", "in0_shift", "in1_mult", "in1_shift", "out_mult",
                  "out_shift", "pad_value", "i0", "i1", "i2", "i3"]


class OpRec(C.Structure):
    _fields_ = ([("kind", C.c_uint32), ("flags", C.c_uint32)] + [(n, C.c_int32) for n in _OP_INT_FIELDS] +
                [("f0", C.c_float), ("f1", C.c_float), ("f2", C.c_float), ("f3", C.c_float)])


assert C.sizeof(Header) == 80 and C.sizeof(TensorRec) == 48 and C.sizeof(OpRec) == 184


@dataclass
class TensorRef:
    id: int
    shape: tuple
    dtype: str
    kind: int
    data: Any = None  # numpy array for constants

    @property
    def nbytes(self) -> int:
        return int(np.prod(self.shape)) * DTYPE_SIZE[self.dtype]


@dataclass
class Op:
    kind: str
    inputs: list
    outputs: list
    consts: dict = field(default_factory=dict)   # name -> TensorRef
    attrs: dict = field(default_factory=dict)    # C field name -> int/float


def _out_dim(i, k, s, d, p0, p1):
    return (i + p0 + p1 - d * (k - 1) - 1) // s + 1


class Graph:
    """A dispatch: tensors, ops in execution order, inputs and outputs."""

    def __init__(self):
        self.tensors: list[TensorRef] = []
        self.ops: list[Op] = []
        self.inputs: list[TensorRef] = []
        self.outputs: list[TensorRef] = []

    # ---- tensors -------------------------------------------------------
    def _tensor(self, shape, dtype, kind, data=None) -> TensorRef:
        shape = tuple(int(s) for s in shape)
        if not 1 <= len(shape) <= 4:
            raise ValueError(f"rank {len(shape)} not supported")
        t = TensorRef(len(self.tensors), shape, dtype, kind, data)
        self.tensors.append(t)
        return t

    def input(self, shape, dtype="i8") -> TensorRef:
        t = self._tensor(shape, dtype, INPUT)
        self.inputs.append(t)
        return t

    def state(self, shape, dtype) -> TensorRef:
        return self._tensor(shape, dtype, STATE)

    def const(self, array, dtype=None) -> TensorRef:
        a = np.ascontiguousarray(array)
        if dtype is None:
            dtype = {np.dtype(np.int8): "i8", np.dtype(np.int32): "i32", np.dtype(np.float32): "f32",
                     np.dtype(np.int16): "i16", np.dtype(np.uint16): "bf16", np.dtype(np.int64): "i64"}[a.dtype]
        a = a.astype(NP_DTYPE[dtype], copy=False)
        shape = a.shape if a.ndim else (1,)
        return self._tensor(shape, dtype, CONSTANT, a.reshape(shape))

    def output(self, t: TensorRef) -> TensorRef:
        if t.kind != ACTIVATION:
            raise ValueError("only an op result can be made an output")
        t.kind = OUTPUT
        self.outputs.append(t)
        return t

    def _emit(self, kind, inputs, out_shape, out_dtype="i8", consts=None, **attrs) -> TensorRef:
        out = self._tensor(out_shape, out_dtype, ACTIVATION)
        self.ops.append(Op(kind, list(inputs), [out], dict(consts or {}), attrs))
        return out

    # ---- requant helper --------------------------------------------------
    def _requant_consts(self, multiplier, shift, oc):
        m = np.atleast_1d(np.asarray(multiplier)).astype(np.int32)
        s = np.atleast_1d(np.asarray(shift)).astype(np.int8)
        if m.shape != s.shape or m.size not in (1, oc):
            raise ValueError("multiplier/shift must have 1 or OC entries")
        return self.const(m, "i32"), self.const(s, "i8"), int(m.size > 1)

    # ---- int8 layer ops ----------------------------------------------------
    def conv2d(self, x, weights, bias, multiplier, shift, *, stride=(1, 1), dilation=(1, 1), pad=(0, 0, 0, 0),
               input_zp=0, weight_zp=0, out_zp=0, clamp=(-128, 127), double_round=True, requant_mode=0):
        """torq_hl.conv2d: x NHWC int8, weights OHWI int8, pad = (top, bottom, left, right)."""
        w = np.asarray(weights, np.int8)
        N, H, W, IC = x.shape
        OC, KH, KW, IC2 = w.shape
        if IC != IC2:
            raise ValueError("weight IC mismatch")
        OH = _out_dim(H, KH, stride[0], dilation[0], pad[0], pad[1])
        OW = _out_dim(W, KW, stride[1], dilation[1], pad[2], pad[3])
        mt, st, pc = self._requant_consts(multiplier, shift, OC)
        consts = {"weights": self.const(w), "bias": self.const(np.atleast_1d(bias).astype(np.int32)),
                  "multiplier": mt, "shift": st}
        return self._emit("conv2d", [x], (N, OH, OW, OC), consts=consts, kh=KH, kw=KW, stride_h=stride[0],
                          stride_w=stride[1], dil_h=dilation[0], dil_w=dilation[1], pad_t=pad[0], pad_b=pad[1],
                          pad_l=pad[2], pad_r=pad[3], in0_zp=input_zp, weight_zp=weight_zp, out_zp=out_zp,
                          clamp_min=clamp[0], clamp_max=clamp[1], per_channel=pc, double_round=int(double_round),
                          requant_mode=requant_mode)

    def conv2d_i16(self, x, weights, bias, multiplier, shift, *, stride=(1, 1), dilation=(1, 1), pad=(0, 0, 0, 0),
                   input_zp=0, weight_zp=0, out_zp=0, clamp=(-32768, 32767)):
        """Conv2D on int16 activations (NHWC) with int8 weights (OHWI) and the 16-bit rescale that follows it:
        64-bit accumulation, (acc * multiplier + 2^(shift-1)) >> shift, + out_zp, clamp, int16."""
        w = np.asarray(weights, np.int8)
        N, H, W, IC = x.shape
        OC, KH, KW, IC2 = w.shape
        if IC != IC2 or x.dtype != "i16":
            raise ValueError("conv2d_i16 wants an int16 NHWC tensor and OHWI weights of the same channel count")
        OH = _out_dim(H, KH, stride[0], dilation[0], pad[0], pad[1])
        OW = _out_dim(W, KW, stride[1], dilation[1], pad[2], pad[3])
        mt, st, pc = self._requant_consts(multiplier, shift, OC)
        consts = {"weights": self.const(w), "bias": self.const(np.atleast_1d(bias).astype(np.int64)),
                  "multiplier": mt, "shift": st}
        return self._emit("conv2d_i16", [x], (N, OH, OW, OC), "i16", consts=consts, kh=KH, kw=KW, stride_h=stride[0],
                          stride_w=stride[1], dil_h=dilation[0], dil_w=dilation[1], pad_t=pad[0], pad_b=pad[1],
                          pad_l=pad[2], pad_r=pad[3], in0_zp=input_zp, weight_zp=weight_zp, out_zp=out_zp,
                          clamp_min=clamp[0], clamp_max=clamp[1], per_channel=pc, double_round=0)

    def depthwise_conv2d(self, x, weights, bias, multiplier, shift, *, stride=(1, 1), dilation=(1, 1),
                         pad=(0, 0, 0, 0), input_zp=0, weight_zp=0, out_zp=0, clamp=(-128, 127),
                         double_round=True, requant_mode=0):
        """torq_hl.depthwise_conv2d: weights [KH, KW, C, M]."""
        w = np.asarray(weights, np.int8)
        N, H, W, Cc = x.shape
        KH, KW, C2, M = w.shape
        if Cc != C2:
            raise ValueError("weight C mismatch")
        OH = _out_dim(H, KH, stride[0], dilation[0], pad[0], pad[1])
        OW = _out_dim(W, KW, stride[1], dilation[1], pad[2], pad[3])
        mt, st, pc = self._requant_consts(multiplier, shift, Cc * M)
        consts = {"weights": self.const(w), "bias": self.const(np.atleast_1d(bias).astype(np.int32)),
                  "multiplier": mt, "shift": st}
        return self._emit("depthwise", [x], (N, OH, OW, Cc * M), consts=consts, kh=KH, kw=KW, stride_h=stride[0],
                          stride_w=stride[1], dil_h=dilation[0], dil_w=dilation[1], pad_t=pad[0], pad_b=pad[1],
                          pad_l=pad[2], pad_r=pad[3], in0_zp=input_zp, weight_zp=weight_zp, out_zp=out_zp,
                          clamp_min=clamp[0], clamp_max=clamp[1], per_channel=pc, double_round=int(double_round),
                          requant_mode=requant_mode)

    def depthwise_conv2d_f(self, x, weights, bias, *, stride=(1, 1), dilation=(1, 1), pad=(0, 0, 0, 0)):
        """tosa.depthwise_conv2d on bf16 / f32: x [N, H, W, C], weights [KH, KW, C, M] and bias [C * M] tensors of x's type."""
        N, H, W, Cc = x.shape
        KH, KW, C2, M = weights.shape
        if Cc != C2 or int(np.prod(bias.shape)) != Cc * M or weights.dtype != x.dtype or bias.dtype != x.dtype or \
                x.dtype not in ("bf16", "f32"):
            raise ValueError("depthwise_conv2d_f wants bf16 or f32 x [N,H,W,C], weights [KH,KW,C,M], bias [C*M]")
        OH = _out_dim(H, KH, stride[0], dilation[0], pad[0], pad[1])
        OW = _out_dim(W, KW, stride[1], dilation[1], pad[2], pad[3])
        return self._emit("depthwise_f", [x, weights, bias], (N, OH, OW, Cc * M), x.dtype, kh=KH, kw=KW, stride_h=stride[0],
                          stride_w=stride[1], dil_h=dilation[0], dil_w=dilation[1], pad_t=pad[0], pad_b=pad[1],
                          pad_l=pad[2], pad_r=pad[3])

    def fully_connected(self, x, weights, bias, multiplier, shift, *, input_zp=0, weight_zp=0, out_zp=0,
                        clamp=(-128, 127), double_round=True, requant_mode=0):
        """torq_hl.fully_connected: x [M, K], weights [N, K] ("[O, I]")."""
        w = np.asarray(weights, np.int8)
        M, K = x.shape
        N, K2 = w.shape
        if K != K2:
            raise ValueError("weight K mismatch")
        mt, st, pc = self._requant_consts(multiplier, shift, N)
        consts = {"weights": self.const(w), "bias": self.const(np.atleast_1d(bias).astype(np.int32)),
                  "multiplier": mt, "shift": st}
        return self._emit("fc", [x], (M, N), consts=consts, in0_zp=input_zp, weight_zp=weight_zp, out_zp=out_zp,
                          clamp_min=clamp[0], clamp_max=clamp[1], per_channel=pc, double_round=int(double_round),
                          requant_mode=requant_mode)

    def matmul_i32(self, a, b, *, a_zp=0, b_zp=0, out_dtype="i32"):
        """raw torq_hl.matmul: a [M, K] x b [K, N], int32 accumulation with wrap-around. b is a constant int8 array
        or, as in the reference's tosa.matmul fixtures, a second runtime tensor; two runtime tensors may both be
        int16, and the result may be stored truncated to int16."""
        if isinstance(b, TensorRef):
            if len(a.shape) != 2 or len(b.shape) != 2 or a.shape[1] != b.shape[0]:
                raise ValueError("matmul wants [M, K] x [K, N]")
            if a.dtype not in ("i8", "i16") or b.dtype != a.dtype or out_dtype not in ("i32", "i16"):
                raise ValueError("matmul wants int8 x int8 or int16 x int16 -> int32 or int16")
            return self._emit("matmul_i32", [a, b], (a.shape[0], b.shape[1]), out_dtype, in0_zp=a_zp, weight_zp=b_zp)
        bw = np.asarray(b, np.int8)
        return self._emit("matmul_i32", [a], (a.shape[0], bw.shape[1]), "i32", consts={"weights": self.const(bw)},
                          in0_zp=a_zp, weight_zp=b_zp)

    def maxpool2d(self, x, kernel, stride, pad=(0, 0, 0, 0), pad_value=-128):
        N, H, W, Cc = x.shape
        OH = _out_dim(H, kernel[0], stride[0], 1, pad[0], pad[1])
        OW = _out_dim(W, kernel[1], stride[1], 1, pad[2], pad[3])
        return self._emit("maxpool", [x], (N, OH, OW, Cc), x.dtype if x.dtype == "i16" else "i8", kh=kernel[0], kw=kernel[1], stride_h=stride[0],
                          stride_w=stride[1], pad_t=pad[0], pad_b=pad[1], pad_l=pad[2], pad_r=pad[3],
                          pad_value=pad_value)

    def avg_pool2d(self, x, kernel, stride, pad=(0, 0, 0, 0), input_zp=0, output_zp=0):
        N, H, W, Cc = x.shape
        OH = _out_dim(H, kernel[0], stride[0], 1, pad[0], pad[1])
        OW = _out_dim(W, kernel[1], stride[1], 1, pad[2], pad[3])
        return self._emit("avgpool", [x], (N, OH, OW, Cc), kh=kernel[0], kw=kernel[1], stride_h=stride[0],
                          stride_w=stride[1], pad_t=pad[0], pad_b=pad[1], pad_l=pad[2], pad_r=pad[3],
                          in0_zp=input_zp, out_zp=output_zp)

    def _binary(self, kind, a, b, a_zp, a_ms, b_zp, b_ms, out_ms, out_zp, clamp, double_round, a_lshift=0, b_lshift=0):
        if a.shape != b.shape:
            raise ValueError("elementwise operands must have equal shapes")
        if not (0 <= a_lshift <= 22 and 0 <= b_lshift <= 22):
            raise ValueError("input left shift outside [0, 22]")
        return self._emit(kind, [a, b], a.shape, in0_zp=a_zp, in0_mult=a_ms[0], in0_shift=a_ms[1], in1_zp=b_zp,
                          in1_mult=b_ms[0], in1_shift=b_ms[1], out_mult=out_ms[0], out_shift=out_ms[1],
                          out_zp=out_zp, clamp_min=clamp[0], clamp_max=clamp[1], double_round=int(double_round),
                          i0=a_lshift, i1=b_lshift)

    def add(self, a, b, *, a_zp, a_ms, b_zp, b_ms, out_ms, out_zp, clamp=(-128, 127), double_round=True, a_lshift=0,
            b_lshift=0):
        """torq_hl.add in TOSA form; *_ms = (multiplier, shift). x_lshift: (x - zp) is shifted left by this
        before its rescale (the first stage of the two-stage input rescale TFLite-derived graphs carry)."""
        return self._binary("add", a, b, a_zp, a_ms, b_zp, b_ms, out_ms, out_zp, clamp, double_round, a_lshift, b_lshift)

    def sub(self, a, b, *, a_zp, a_ms, b_zp, b_ms, out_ms, out_zp, clamp=(-128, 127), double_round=True, a_lshift=0,
            b_lshift=0):
        return self._binary("sub", a, b, a_zp, a_ms, b_zp, b_ms, out_ms, out_zp, clamp, double_round, a_lshift, b_lshift)

    def mul(self, a, b, *, a_zp, a_ms, b_zp, b_ms, out_ms, out_zp, clamp=(-128, 127), double_round=True, a_lshift=0,
            b_lshift=0):
        return self._binary("mul", a, b, a_zp, a_ms, b_zp, b_ms, out_ms, out_zp, clamp, double_round, a_lshift, b_lshift)

    def table(self, x, table):
        t = np.asarray(table, np.int8)
        if t.size != 256:
            raise ValueError("table must have 256 entries")
        return self._emit("table", [x], x.shape, consts={"table": self.const(t)})

    def rescale(self, x, multiplier, shift, *, input_zp=0, out_zp=0, clamp=None, double_round=True,
                requant_mode=0, out_dtype="i8", input_unsigned=False, output_unsigned=False):
        """tosa.rescale. i8 -> i8 is the layer-path op; other integer types (i8 / i16 / i32 in and out, unsigned
        8/16-bit storage by flag) take the generic kernel. The clamp defaults to the result type's range."""
        mt, st, pc = self._requant_consts(multiplier, shift, x.shape[-1])
        if clamp is None:
            bits = {"i8": 8, "i16": 16, "i32": 32}[out_dtype]
            clamp = (0, (1 << bits) - 1) if output_unsigned else (-(1 << (bits - 1)), (1 << (bits - 1)) - 1)
        flags = (FLAG_INPUT_UNSIGNED if input_unsigned else 0) | (FLAG_OUTPUT_UNSIGNED if output_unsigned else 0)
        return self._emit("rescale", [x], x.shape, out_dtype, consts={"multiplier": mt, "shift": st}, in0_zp=input_zp,
                          out_zp=out_zp, clamp_min=clamp[0], clamp_max=min(clamp[1], (1 << 31) - 1), per_channel=pc,
                          double_round=int(double_round), requant_mode=requant_mode, flags=flags)

    # ---- tensor ops outside the layer set ---------------------------------------
    def ew(self, fn: str, a, b=None, *, out_dtype=None, arg: int = 0, in_zp: int = 0, out_zp: int = 0, clamp=(0, 0),
           fclamp=(0.0, 0.0), bool_result: bool = False):
        """Elementwise op `fn` (a key of EW_FN) on one or two tensors of equal rank; extent-1 dimensions broadcast."""
        if b is not None:
            if len(a.shape) != len(b.shape) or any(x != y and 1 not in (x, y) for x, y in zip(a.shape, b.shape)):
                raise ValueError("elementwise operands must have equal rank and broadcastable shapes")
            shape = tuple(max(x, y) for x, y in zip(a.shape, b.shape))
        else:
            shape = a.shape
        return self._emit("ew", [a] if b is None else [a, b], shape, out_dtype or a.dtype, i0=EW_FN[fn], i1=int(arg),
                          in0_zp=int(in_zp), out_zp=int(out_zp), clamp_min=int(clamp[0]), clamp_max=int(clamp[1]),
                          f0=float(fclamp[0]), f1=float(fclamp[1]), flags=FLAG_BOOL_RESULT if bool_result else 0)

    def softmax(self, x):
        """softmax over the last axis of a bf16 / f32 tensor."""
        if x.dtype not in ("bf16", "f32"):
            raise ValueError("softmax wants a bf16 or f32 tensor")
        return self._emit("softmax", [x], x.shape, x.dtype)

    def table16(self, x, table):
        """tosa.table on an int16 tensor: 513 int16 entries, interpolated; int32 result."""
        t = np.asarray(table, np.int16)
        if t.size != 513 or x.dtype != "i16":
            raise ValueError("table16 wants an i16 tensor and 513 entries")
        return self._emit("table16", [x], x.shape, "i32", consts={"table": self.const(t)})

    def transpose(self, x, perm):
        perm = [int(p) for p in perm]
        if sorted(perm) != list(range(len(x.shape))):
            raise ValueError("perm must be a permutation of the dimensions")
        p4 = perm + list(range(len(perm), 4))
        return self._emit("transpose", [x], tuple(x.shape[p] for p in perm), x.dtype, i0=p4[0], i1=p4[1], i2=p4[2], i3=p4[3])

    def matmul_f(self, a, b, out_dtype="f32"):
        """tosa.matmul on bf16 / f32 tensors: a [M, K] x b [K, N] -> f32 or bf16, fp32 products and sums in index order of k."""
        if len(a.shape) != 2 or len(b.shape) != 2 or a.shape[1] != b.shape[0] or a.dtype not in ("bf16", "f32") or \
                b.dtype != a.dtype or out_dtype not in ("bf16", "f32"):
            raise ValueError("matmul_f wants [M, K] x [K, N] of bf16 or f32")
        return self._emit("matmul_f", [a, b], (a.shape[0], b.shape[1]), out_dtype)

    def gather(self, values, indices):
        """tosa.gather: values [N, K, C], indices [N, W] (i32) -> [N, W, C], out[n, w] = values[n, indices[n, w]]."""
        if len(values.shape) != 3 or len(indices.shape) != 2 or indices.dtype != "i32" or indices.shape[0] != values.shape[0]:
            raise ValueError("gather wants values [N, K, C] and i32 indices [N, W]")
        return self._emit("gather", [values, indices], (values.shape[0], indices.shape[1], values.shape[2]), values.dtype)

    def scatter(self, values, indices, updates):
        """tosa.scatter: a copy of values [N, K, C] with rows indices[n, w] replaced by updates[n, w] ([N, W, C])."""
        if len(values.shape) != 3 or len(indices.shape) != 2 or indices.dtype != "i32" or updates.dtype != values.dtype or \
                tuple(updates.shape) != (values.shape[0], indices.shape[1], values.shape[2]):
            raise ValueError("scatter wants values [N, K, C], i32 indices [N, W] and updates [N, W, C]")
        return self._emit("scatter", [values, indices, updates], tuple(values.shape), values.dtype)

    def permute(self, x, view_shape, perm, out_shape):
        """Transpose of a view of up to six dimensions (x holds prod(view_shape) elements in any stored shape)."""
        view = [int(d) for d in view_shape]
        perm = [int(p) for p in perm]
        r = len(view)
        if r > 6 or sorted(perm) != list(range(r)) or any(d < 1 or d > 65535 for d in view):
            raise ValueError("permute wants at most six dimensions of at most 65535 and a permutation of them")
        if int(np.prod(view)) != int(np.prod(x.shape)) or int(np.prod(out_shape)) != int(np.prod(view)):
            raise ValueError("permute: element counts differ")
        d6 = view + [1] * (6 - r)
        packed = sum(p << (4 * i) for i, p in enumerate(perm)) | (r << 24)
        return self._emit("permute", [x], tuple(int(d) for d in out_shape), x.dtype, i0=d6[0] | d6[1] << 16,
                          i1=d6[2] | d6[3] << 16, i2=d6[4] | d6[5] << 16, i3=packed)

    def slice(self, x, start, size):
        if any(s < 0 or s + n > d for s, n, d in zip(start, size, x.shape)):
            raise ValueError("slice outside the tensor")
        s4 = [int(v) for v in start] + [0] * (4 - len(start))
        return self._emit("slice", [x], tuple(int(n) for n in size), x.dtype, i0=s4[0], i1=s4[1], i2=s4[2], i3=s4[3])

    def pad(self, x, before, after, value: int = 0):
        b4 = [int(v) for v in before] + [0] * (4 - len(before))
        shape = tuple(d + int(lo) + int(hi) for d, lo, hi in zip(x.shape, before, after))
        return self._emit("pad", [x], shape, x.dtype, i0=b4[0], i1=b4[1], i2=b4[2], i3=b4[3], pad_value=int(value))

    def concat_axis(self, a, b, axis: int):
        if a.dtype != b.dtype or len(a.shape) != len(b.shape) or any(
                x != y for i, (x, y) in enumerate(zip(a.shape, b.shape)) if i != axis):
            raise ValueError("concat operands differ outside the axis")
        shape = tuple(d + (b.shape[i] if i == axis else 0) for i, d in enumerate(a.shape))
        return self._emit("concat_axis", [a, b], shape, a.dtype, i0=int(axis))

    def reduce(self, fn: str, x, axis: int, *, keep_axis: bool = True, out_dtype=None):
        shape = tuple(1 if i == axis else d for i, d in enumerate(x.shape)) if keep_axis else \
            tuple(d for i, d in enumerate(x.shape) if i != axis) or (1,)
        return self._emit("reduce", [x], shape, out_dtype or ("i32" if fn == "argmax" else x.dtype), i0=REDUCE_FN[fn],
                          i1=int(axis))

    def resize_nearest_2x(self, x):
        N, H, W, Cc = x.shape
        return self._emit("resize_nn2x", [x], (N, 2 * H, 2 * W, Cc))

    def concat(self, a, b, *, a_zp, a_ms, b_zp, b_ms, out_zp, double_round=True):
        """channel concat with an i8->i8 rescale on each input."""
        if a.shape[:-1] != b.shape[:-1]:
            raise ValueError("concat operands differ outside the channel axis")
        return self._emit("concat", [a, b], a.shape[:-1] + (a.shape[-1] + b.shape[-1],), in0_zp=a_zp,
                          in0_mult=a_ms[0], in0_shift=a_ms[1], in1_zp=b_zp, in1_mult=b_ms[0], in1_shift=b_ms[1],
                          out_zp=out_zp, double_round=int(double_round))

    def reshape(self, x, shape):
        """tosa.reshape: the result is a view of the same bytes (no kernel runs)."""
        if int(np.prod(shape)) != int(np.prod(x.shape)):
            raise ValueError("reshape changes the element count")
        return self._emit("reshape", [x], shape, x.dtype)

    # ---- decoder ops (bf16 activations, int8 per-output-channel weights) ------
    def embed(self, tokens, table_i8, scales_bf16, mult: float):
        """x[b] = bf16(bf16(E[tok[b]] * scale[tok[b]]) * mult). table/scales may be TensorRefs
        (to share the tied LM-head table) or arrays."""
        tab = table_i8 if isinstance(table_i8, TensorRef) else self.const(np.asarray(table_i8, np.int8))
        sc = scales_bf16 if isinstance(scales_bf16, TensorRef) else self.const(np.asarray(scales_bf16, np.uint16), "bf16")
        return self._emit("embed", [tokens], (tokens.shape[0], tab.shape[1]), "bf16", consts={"weights": tab, "bias": sc},
                          f0=float(mult))

    def rmsnorm(self, x, weight_bf16, eps: float, residual=None):
        """y = [residual +] bf16(x * rsqrt(mean(x^2) + eps) * (1 + w))."""
        w = weight_bf16 if isinstance(weight_bf16, TensorRef) else self.const(np.asarray(weight_bf16, np.uint16), "bf16")
        ins = [x] + ([residual] if residual is not None else [])
        return self._emit("rmsnorm", ins, x.shape, "bf16", consts={"weights": w}, f0=float(eps))

    def gemv_w8(self, x, weights_i8, scales_bf16, splits: int = 0, out_dtype: str = "bf16", in_offset: int = 0):
        """y[b, n] = scale[n] * sum_k x[b, in_offset + k] * W[n, k], rounded to bf16 or kept in fp32 (out_dtype
        "f32"); W is [N, K] int8. A W narrower than x (with in_offset) takes a column slice of x; that form
        exists only inside the fused decode step (tensor-parallel shards)."""
        w = weights_i8 if isinstance(weights_i8, TensorRef) else self.const(np.asarray(weights_i8, np.int8))
        sc = scales_bf16 if isinstance(scales_bf16, TensorRef) else self.const(np.asarray(scales_bf16, np.uint16), "bf16")
        if in_offset < 0 or in_offset + w.shape[1] > x.shape[1] or (in_offset == 0 and w.shape[1] != x.shape[1] and out_dtype != "f32"):
            raise ValueError("weight K mismatch")
        return self._emit("gemv_w8", [x], (x.shape[0], w.shape[0]), out_dtype, consts={"weights": w, "bias": sc}, i0=splits,
                          i1=int(in_offset))

    def rope_kv(self, qkv, pos, q_norm_w, k_norm_w, k_cache, v_cache, *, n_q, n_kv, head_dim, theta, eps):
        """Per-head RMSNorm + rotary on q and k at position pos; k and v appended to the caches
        (state tensors [B, T, n_kv * head_dim]). Returns the rotated queries [B, n_q * head_dim]."""
        qw = self.const(np.asarray(q_norm_w, np.uint16), "bf16")
        kw = self.const(np.asarray(k_norm_w, np.uint16), "bf16")
        out = self._tensor((qkv.shape[0], n_q * head_dim), "bf16", ACTIVATION)
        self.ops.append(Op("rope_kv", [qkv, pos, v_cache], [out, k_cache], {"weights": qw, "bias": kw},
                           dict(i0=n_q, i1=n_kv, i2=head_dim, f0=float(theta), f1=float(eps))))
        return out

    def attn_decode(self, q, pos, k_cache, v_cache, *, n_q, n_kv, head_dim, window, scale):
        """Single-query attention over the cached keys [max(0, pos - window + 1), pos] (window 0 = all)."""
        out = self._tensor(q.shape, "bf16", ACTIVATION)
        self.ops.append(Op("attn_decode", [q, pos, k_cache], [out], {"weights": v_cache},
                           dict(i0=n_q, i1=n_kv, i2=head_dim, i3=window, f0=float(scale))))
        return out

    def geglu(self, gate_up):
        """y = bf16(bf16(gelu_tanh(gate)) * up), gate = first half of the columns."""
        return self._emit("geglu", [gate_up], (gate_up.shape[0], gate_up.shape[1] // 2), "bf16")

    def gemv_q8b(self, x, weights_kn_i8, block_scales_bf16, block_zero_points_i8=None, block_size: int = 32):
        """y = bf16(x . bf16((W - zp) * scale)): W int8 [K, N], scales bf16 and zero points int8 [K / block, N]
        (ONNX DequantizeLinear(axis=0, block_size) + MatMul)."""
        w = self.const(np.asarray(weights_kn_i8, np.int8))
        consts = {"weights": w, "bias": self.const(np.asarray(block_scales_bf16, np.uint16), "bf16")}
        if block_zero_points_i8 is not None:
            consts["multiplier"] = self.const(np.asarray(block_zero_points_i8, np.int8))
        if w.shape[0] != x.shape[1]:
            raise ValueError("weight K mismatch")
        return self._emit("gemv_q8b", [x], (x.shape[0], w.shape[1]), "bf16", consts=consts, i0=int(block_size))

    ACT_FUNCTIONS = {"sigmoid": 0, "gelu_tanh": 1, "exp": 2, "tanh": 3, "silu": 4}

    def act_bf16(self, x, function: str):
        """y = bf16(f(x)) with f evaluated in fp32: sigmoid, gelu_tanh, exp, tanh or silu."""
        if x.dtype != "bf16":
            raise ValueError("act_bf16 wants a bf16 tensor")
        return self._emit("act_bf16", [x], x.shape, "bf16", i0=self.ACT_FUNCTIONS[function])

    def argmax(self, logits, vocab_offset: int = 0, group_size: int = 1):
        """Greedy ids. group_size >= 2: `logits` is this GPU's vocabulary shard of a tensor-parallel
        group; the result is the arg max over all shards, this shard's ids offset by vocab_offset."""
        return self._emit("argmax", [logits], (logits.shape[0],), "i32", i0=int(vocab_offset), i1=int(group_size))

    def allreduce(self, partial_f32, group_size: int, rank: int):
        """bf16(sum over the group's GPUs of their fp32 partial results), in rank order. Exists only
        inside the fused decode step of a tensor-parallel shard."""
        if partial_f32.dtype != "f32" or not 2 <= group_size <= 8 or not 0 <= rank < group_size:
            raise ValueError("allreduce wants an f32 tensor, a group of 2..8 and a rank inside it")
        return self._emit("allreduce", [partial_f32], partial_f32.shape, "bf16", i0=int(group_size), i1=int(rank))

    # ---- serialisation ------------------------------------------------------
    @staticmethod
    def deserialize(blob: bytes) -> "Graph":
        """Rebuilds a Graph (tensors, op records with their constants) from a torq-b200-ops blob,
        e.g. a model file: the inverse of serialize()."""
        h = Header.from_buffer_copy(blob[:C.sizeof(Header)])
        if h.magic != MAGIC or h.version != VERSION:
            raise ValueError("not a torq-b200-ops blob of this version")
        kinds = {v: k for k, v in OP_KINDS.items()}
        dnames = {v: k for k, v in DTYPES.items()}
        g = Graph()
        for i in range(h.n_tensors):
            r = TensorRec.from_buffer_copy(blob[h.tensors_offset + i * C.sizeof(TensorRec):][:C.sizeof(TensorRec)])
            shape = tuple(r.shape[k] for k in range(r.rank))
            dt = dnames[r.dtype]
            data = None
            if r.kind == CONSTANT:
                raw = blob[h.const_offset + r.const_offset:h.const_offset + r.const_offset + r.const_bytes]
                data = np.frombuffer(raw, NP_DTYPE[dt]).reshape(shape).copy()
            g.tensors.append(TensorRef(i, shape, dt, r.kind, data))
        const_fields = _OP_INT_FIELDS[5:10]
        for i in range(h.n_ops):
            r = OpRec.from_buffer_copy(blob[h.ops_offset + i * C.sizeof(OpRec):][:C.sizeof(OpRec)])
            ins = [g.tensors[t] for t in (r.in0, r.in1, r.in2) if t >= 0]
            outs = [g.tensors[t] for t in (r.out0, r.out1) if t >= 0]
            consts = {n: g.tensors[getattr(r, n)] for n in const_fields if getattr(r, n) >= 0}
            attrs = {n: getattr(r, n) for n in _OP_INT_FIELDS[10:]}
            attrs["flags"] = r.flags
            attrs.update({f: getattr(r, f) for f in ("f0", "f1", "f2", "f3")})
            g.ops.append(Op(kinds[r.kind], ins, outs, consts, attrs))
        ids_in = np.frombuffer(blob[h.inputs_offset:h.inputs_offset + 4 * h.n_inputs], np.int32)
        ids_out = np.frombuffer(blob[h.outputs_offset:h.outputs_offset + 4 * h.n_outputs], np.int32)
        g.inputs = [g.tensors[i] for i in ids_in]
        g.outputs = [g.tensors[i] for i in ids_out]
        return g

    def serialize(self) -> bytes:
        const_blob = bytearray()
        trecs = []
        for t in self.tensors:
            r = TensorRec()
            r.dtype, r.kind, r.rank = DTYPES[t.dtype], t.kind, len(t.shape)
            for i in range(4):
                r.shape[i] = t.shape[i] if i < len(t.shape) else 1
            if t.kind == CONSTANT:
                pad = (-len(const_blob)) % 16
                const_blob.extend(b"\0" * pad)
                raw = t.data.tobytes()
                r.const_offset, r.const_bytes = len(const_blob), len(raw)
                const_blob.extend(raw)
            trecs.append(bytes(r))
        orecs = []
        for op in self.ops:
            r = OpRec()
            r.kind = OP_KINDS[op.kind]
            for n in _OP_INT_FIELDS[:10]:
                setattr(r, n, -1)
            for i, t in enumerate(op.inputs):
                setattr(r, f"in{i}", t.id)
            for i, t in enumerate(op.outputs):
                setattr(r, f"out{i}", t.id)
            for name, t in op.consts.items():
                setattr(r, name, t.id)
            r.dil_h = r.dil_w = r.stride_h = r.stride_w = 1
            r.clamp_min, r.clamp_max, r.out_shift, r.in0_shift, r.in1_shift = -128, 127, 2, 2, 2
            for k, v in op.attrs.items():
                setattr(r, k, v)
            orecs.append(bytes(r))

        def align(n):
            return (n + 15) & ~15

        h = Header()
        h.magic, h.version = MAGIC, VERSION
        h.n_tensors, h.n_ops, h.n_inputs, h.n_outputs = len(trecs), len(orecs), len(self.inputs), len(self.outputs)
        off = align(C.sizeof(Header))
        h.tensors_offset = off
        off = align(off + len(trecs) * C.sizeof(TensorRec))
        h.ops_offset = off
        off = align(off + len(orecs) * C.sizeof(OpRec))
        h.inputs_offset = off
        off = align(off + 4 * len(self.inputs))
        h.outputs_offset = off
        off = align(off + 4 * len(self.outputs))
        h.const_offset, h.const_bytes = off, len(const_blob)
        h.total_bytes = off + len(const_blob)
        out = bytearray(h.total_bytes)
        out[0:C.sizeof(Header)] = bytes(h)
        p = h.tensors_offset
        for b in trecs:
            out[p:p + len(b)] = b
            p += len(b)
        p = h.ops_offset
        for b in orecs:
            out[p:p + len(b)] = b
            p += len(b)
        out[h.inputs_offset:h.inputs_offset + 4 * len(self.inputs)] = np.array([t.id for t in self.inputs], np.int32).tobytes()
        out[h.outputs_offset:h.outputs_offset + 4 * len(self.outputs)] = np.array([t.id for t in self.outputs], np.int32).tobytes()
        out[h.const_offset:h.const_offset + len(const_blob)] = const_blob
        return bytes(out)
