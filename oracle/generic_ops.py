"""CPU restatement (test infrastructure, not the product) of the tensor ops outside the layer set:
elementwise integer / float ops, generic tosa.rescale, transpose, slice, pad, concat, reductions.

Semantics follow TOSA 1.0 as the reference's host path lowers it (MLIR TosaToLinalg inside the IREE fork, absent
here; the reference's own statement of the forms is compiler/torq/Conversions/TosaToTorqHL/Patterns.cpp:1735-1947
for rescale and doc/user-manual/ops.md for the op list): integers are computed in int32 with wrap-around and
truncated to the result type, int -> narrower int casts truncate, float -> int casts round to nearest even and
saturate, bf16 is computed in fp32 and rounded once to nearest even. Parity unpinned: the reference holds no
golden outputs for these ops and cannot be run here.

Vectorised numpy (int64 / float32 arithmetic); oracle_np.ew_elementwise is a second, element-by-element
statement with Python integers that the golden generator compares it with."""
from __future__ import annotations

import numpy as np

INT_BITS = {"i8": 8, "i16": 16, "i32": 32}
EW_NAMES = {0: "cast", 1: "abs", 2: "negate", 3: "bitwise_not", 4: "logical_not", 5: "clz", 6: "clamp", 7: "ceil", 8: "floor",
            9: "exp", 10: "log", 11: "reciprocal", 12: "rsqrt", 13: "tanh", 14: "sigmoid", 15: "erf",
            16: "add", 17: "sub", 18: "mul", 19: "maximum", 20: "minimum", 21: "bitwise_and", 22: "bitwise_or",
            23: "bitwise_xor", 24: "logical_left_shift", 25: "arithmetic_right_shift", 26: "equal", 27: "greater",
            28: "greater_equal", 29: "logical_and", 30: "logical_or", 31: "logical_xor"}


def _erf32(x):
    import math
    return np.vectorize(math.erf, otypes=[np.float64])(x.astype(np.float64))


FLOAT_FUNCTIONS = {"exp": np.exp, "log": np.log, "reciprocal": lambda v: np.float32(1.0) / v, "rsqrt": lambda v: np.float32(1.0) / np.sqrt(v),
                   "tanh": np.tanh, "sigmoid": lambda v: np.float32(1.0) / (np.float32(1.0) + np.exp(-v)), "erf": _erf32}


def bf16_to_f32(u16: np.ndarray) -> np.ndarray:
    return (u16.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(f: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(f, np.float32).view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = np.isnan(f)
    return np.where(nan, np.uint16(0x7FC0), rounded).astype(np.uint16)


def _load(x: np.ndarray, dtype: str):
    """-> (values as int64 or float32, is_float)"""
    if dtype == "bf16":
        return bf16_to_f32(x), True
    if dtype == "f32":
        return x.astype(np.float32), True
    return x.astype(np.int64), False


def wrap(v: np.ndarray, bits: int) -> np.ndarray:
    """two's-complement truncation of int64 values to `bits` bits, as int64"""
    m = (1 << bits) - 1
    u = v & m
    return np.where(u >= (1 << (bits - 1)), u - (1 << bits), u)


def _store(v, is_float: bool, out_dtype: str) -> np.ndarray:
    if out_dtype == "bf16":
        return f32_to_bf16(v.astype(np.float32))
    if out_dtype == "f32":
        return v.astype(np.float32)
    np_t = {"i8": np.int8, "i16": np.int16, "i32": np.int32}[out_dtype]
    if is_float:  # float -> int: nearest even, saturating, NaN -> 0
        lo, hi = -(1 << (INT_BITS[out_dtype] - 1)), (1 << (INT_BITS[out_dtype] - 1)) - 1
        r = np.rint(np.nan_to_num(v.astype(np.float64), nan=0.0, posinf=float(hi), neginf=float(lo)))
        return np.clip(r, lo, hi).astype(np_t)
    return wrap(v, INT_BITS[out_dtype]).astype(np_t)


def _clz32(v: np.ndarray) -> np.ndarray:
    u = (v & 0xFFFFFFFF).astype(np.uint64)
    out = np.full(u.shape, 32, np.int64)
    for b in range(32):
        out = np.where((u >> b) != 0, 31 - b, out)
    return out


def ew(fn: int, a: np.ndarray, a_dtype: str, b, b_dtype, out_dtype: str, *, arg=0, in_zp=0, out_zp=0, clamp=(0, 0),
       fclamp=(0.0, 0.0), bool_result=False) -> np.ndarray:
    name = EW_NAMES[fn]
    x, xf = _load(a, a_dtype)
    y, yf = _load(b, b_dtype) if b is not None else (None, False)
    flt = xf or yf
    if flt:
        x = x.astype(np.float32)
        y = y.astype(np.float32) if y is not None else None
    else:
        x = wrap(x, 32)
        y = wrap(y, 32) if y is not None else None
    if name == "cast":
        r = (x != 0).astype(np.int64) if bool_result else x
        if flt and out_dtype in INT_BITS and not bool_result:
            return _store(x, True, out_dtype)
        if bool_result:
            return r.astype(np.int8)
        if not flt and out_dtype in ("f32", "bf16"):
            return _store(x.astype(np.float32), True, out_dtype)
        return _store(r, flt, out_dtype)
    if name == "abs":
        r = np.abs(x)
    elif name == "negate":
        r = -x if flt else (out_zp - (x - in_zp))
    elif name == "bitwise_not":
        r = ~x
    elif name == "logical_not":
        r = (x == 0).astype(np.int64)
    elif name == "clz":
        r = _clz32(x)
    elif name == "clamp":
        r = np.clip(x, np.float32(fclamp[0]), np.float32(fclamp[1])) if flt else np.clip(x, clamp[0], clamp[1])
    elif name == "ceil":
        r = np.ceil(x)
    elif name == "floor":
        r = np.floor(x)
    elif name in FLOAT_FUNCTIONS:  # fp32 in and out; tolerance class (the last bits are the math library's)
        with np.errstate(all="ignore"):
            r = FLOAT_FUNCTIONS[name](x.astype(np.float32)).astype(np.float32)
    elif name == "add":
        r = x + y
    elif name == "sub":
        r = x - y
    elif name == "mul":
        if flt:
            r = x * y
        elif arg > 0:
            r = (x * y + (1 << (arg - 1))) >> arg
        else:
            r = x * y
    elif name == "maximum":
        r = np.maximum(x, y)
    elif name == "minimum":
        r = np.minimum(x, y)
    elif name == "bitwise_and":
        r = x & y
    elif name == "bitwise_or":
        r = x | y
    elif name == "bitwise_xor":
        r = x ^ y
    elif name == "logical_left_shift":
        r = x << (y & 31)
    elif name == "arithmetic_right_shift":
        s = y & 31
        r = x >> s
        if arg:  # round: add the last bit shifted out
            r = r + np.where(s > 0, (x >> np.maximum(s - 1, 0)) & 1, 0)
    elif name == "equal":
        return (x == y).astype(np.int8)
    elif name == "greater":
        return (x > y).astype(np.int8)
    elif name == "greater_equal":
        return (x >= y).astype(np.int8)
    elif name == "logical_and":
        return ((x != 0) & (y != 0)).astype(np.int8)
    elif name == "logical_or":
        return ((x != 0) | (y != 0)).astype(np.int8)
    elif name == "logical_xor":
        return ((x != 0) ^ (y != 0)).astype(np.int8)
    else:
        raise NotImplementedError(name)
    return _store(r, flt, out_dtype)


def apply_scale_32(v: np.ndarray, mult: np.ndarray, shift: np.ndarray, double_round: bool) -> np.ndarray:
    v = v.astype(np.int64)
    mult = mult.astype(np.int64)
    shift = shift.astype(np.int64)
    rnd = np.int64(1) << (shift - 1)
    if double_round:
        rnd = rnd + np.where(shift > 31, np.where(v >= 0, np.int64(1) << 30, -(np.int64(1) << 30)), 0)
    return (v * mult + rnd) >> shift


def rescale(x: np.ndarray, in_dtype: str, out_dtype: str, mult, shift, in_zp: int, out_zp: int, clamp, *, per_channel: bool,
            double_round: bool, input_unsigned=False, output_unsigned=False) -> np.ndarray:
    """tosa.rescale with scale32 = true between integer types. value = (in - in_zp) in int32 (wrapping), scaled, plus
    out_zp, clamped to `clamp` (the result type's range unless narrowed) and stored."""
    bits_in = INT_BITS[in_dtype]
    v = x.astype(np.int64)
    if input_unsigned:
        v = v & ((1 << bits_in) - 1)
    v = wrap(v - in_zp, 32)
    m = np.asarray(mult, np.int64).reshape(-1)
    s = np.asarray(shift, np.int64).reshape(-1)
    if not per_channel:
        m, s = m[:1], s[:1]
    r = apply_scale_32(v, m, s, double_round)   # broadcasts over the last axis when per channel
    r = np.clip(wrap(r, 32) + out_zp, clamp[0], clamp[1])
    return wrap(r, INT_BITS[out_dtype]).astype({"i8": np.int8, "i16": np.int16, "i32": np.int32}[out_dtype])


def reduce(fn: int, x: np.ndarray, dtype: str, axis: int, out_shape, out_dtype: str) -> np.ndarray:
    v, flt = _load(x, dtype)
    if fn in (0, 4) and flt:  # fp32 accumulation in index order (cumsum adds one element at a time)
        r = np.take(np.cumsum(v.astype(np.float32), axis=axis, dtype=np.float32), -1, axis=axis)
        if fn == 4:
            r = (r / np.float32(v.shape[axis])).astype(np.float32)
    elif fn == 0:
        r = v.sum(axis=axis, dtype=np.int64)
    elif fn == 1:
        r = v.max(axis=axis)
    elif fn == 2:
        r = v.min(axis=axis)
    else:
        return v.argmax(axis=axis).astype(np.int32).reshape(out_shape)
    return _store(r, flt, out_dtype).reshape(out_shape)


def matmul_int(a: np.ndarray, b: np.ndarray, a_zp: int, b_zp: int, out_dtype: str) -> np.ndarray:
    """tosa.matmul on int8 or int16 operands as the reference lowers it (doc/user-manual/ops.md: MatMul i16 x i16 -> i32,
    "TOSA specifies i48 output"): products added one k at a time into an int32 that wraps, stored as int32 or
    truncated to int16."""
    x = a.astype(np.int64) - a_zp
    y = b.astype(np.int64) - b_zp
    acc = np.zeros((x.shape[0], y.shape[1]), np.int64)
    for k in range(x.shape[1]):
        acc = wrap(acc + wrap(x[:, k, None] * y[None, k, :], 32), 32)
    return wrap(acc, INT_BITS[out_dtype]).astype({"i16": np.int16, "i32": np.int32}[out_dtype])


def conv2d_i16(x: np.ndarray, w: np.ndarray, bias: np.ndarray, mult, shift, *, stride, dilation, pad, input_zp: int, weight_zp: int,
               out_zp: int, clamp) -> np.ndarray:
    """tosa.conv2d on int16 activations / int8 weights with acc_type i48, then tosa.rescale {scale32 = false, SINGLE_ROUND}
    (TOSA 1.0 apply_scale_16: (value * multiplier + 2^(shift-1)) >> shift with a 16-bit multiplier), + out_zp, clamp, int16.
    x NHWC, w OHWI, pad = (top, bottom, left, right); padded positions contribute (input_zp - input_zp) = 0."""
    N, H, W, IC = x.shape
    OC, KH, KW, _ = w.shape
    OH = (H + pad[0] + pad[1] - (KH - 1) * dilation[0] - 1) // stride[0] + 1
    OW = (W + pad[2] + pad[3] - (KW - 1) * dilation[1] - 1) // stride[1] + 1
    xp = np.zeros((N, H + pad[0] + pad[1], W + pad[2] + pad[3], IC), np.int64)
    xp[:, pad[0]:pad[0] + H, pad[2]:pad[2] + W, :] = x.astype(np.int64) - input_zp
    wz = w.astype(np.int64) - weight_zp
    acc = np.zeros((N, OH, OW, OC), np.int64)
    for kh in range(KH):
        for kw in range(KW):
            h0, w0 = kh * dilation[0], kw * dilation[1]
            win = xp[:, h0:h0 + (OH - 1) * stride[0] + 1:stride[0], w0:w0 + (OW - 1) * stride[1] + 1:stride[1], :]
            acc += np.einsum("nhwc,oc->nhwo", win, wz[:, kh, kw, :])
    b = np.asarray(bias, np.int64).reshape(-1)
    acc = acc + (b if b.size == OC else b[:1])
    m = np.asarray(mult, np.int64).reshape(-1)
    s = np.asarray(shift, np.int64).reshape(-1)
    r = (acc * m + (np.int64(1) << (s - 1))) >> s
    return np.clip(r + out_zp, clamp[0], clamp[1]).astype(np.int16)


def matmul_f(a: np.ndarray, b: np.ndarray, dtype: str, out_dtype: str) -> np.ndarray:
    """tosa.matmul on floats: fp32 products, each rounded, added one k at a time in fp32 (index order), then stored as
    f32 or rounded once to bf16."""
    x, _ = _load(a, dtype)
    y, _ = _load(b, dtype)
    x, y = x.astype(np.float32), y.astype(np.float32)
    acc = np.zeros((x.shape[0], y.shape[1]), np.float32)
    for k in range(x.shape[1]):
        acc = (acc + (x[:, k, None] * y[None, k, :]).astype(np.float32)).astype(np.float32)
    return _store(acc, True, out_dtype)


def depthwise_f(x: np.ndarray, w: np.ndarray, bias: np.ndarray, dtype: str, stride, dilation, pad) -> np.ndarray:
    """tosa.depthwise_conv2d on floats (reference semantics: doc/user-manual/ops.md, DepthwiseConv2D bf16; TOSA: the
    accumulator is fp32): fp32 products, each rounded, added tap by tap in (kh, kw) order, taps outside the frame
    skipped, the bias last; stored in the operands' type. x [N, H, W, C], w [KH, KW, C, M], bias [C * M]."""
    xf, _ = _load(x, dtype)
    wf, _ = _load(w, dtype)
    bf, _ = _load(bias, dtype)
    xf, wf, bf = xf.astype(np.float32), wf.astype(np.float32), bf.astype(np.float32).reshape(-1)
    N, H, W, C = xf.shape
    KH, KW, _, M = wf.shape
    OH = (H + pad[0] + pad[1] - dilation[0] * (KH - 1) - 1) // stride[0] + 1
    OW = (W + pad[2] + pad[3] - dilation[1] * (KW - 1) - 1) // stride[1] + 1
    acc = np.zeros((N, OH, OW, C, M), np.float32)
    for kh in range(KH):
        for kw in range(KW):
            for oh in range(OH):
                ih = oh * stride[0] - pad[0] + kh * dilation[0]
                if ih < 0 or ih >= H:
                    continue
                ows = [ow for ow in range(OW) if 0 <= ow * stride[1] - pad[2] + kw * dilation[1] < W]
                if not ows:
                    continue
                iws = [ow * stride[1] - pad[2] + kw * dilation[1] for ow in ows]
                prod = (xf[:, ih, iws, :, None] * wf[kh, kw][None, None]).astype(np.float32)
                acc[:, oh, ows] = (acc[:, oh, ows] + prod).astype(np.float32)
    out = (acc.reshape(N, OH, OW, C * M) + bf[None, None, None, :]).astype(np.float32)
    return _store(out, True, dtype)


def gather(values: np.ndarray, indices: np.ndarray) -> np.ndarray:
    """tosa.gather (TOSA 1.0: output[n, w, c] = values[n, indices[n, w], c])."""
    return np.stack([values[n][indices[n]] for n in range(values.shape[0])])


def scatter(values: np.ndarray, indices: np.ndarray, updates: np.ndarray) -> np.ndarray:
    """tosa.scatter (TOSA 1.0: values_out = values_in with values_out[n, indices[n, w], c] = input[n, w, c])."""
    out = values.copy()
    for n in range(values.shape[0]):
        out[n][indices[n]] = updates[n]
    return out


def table16(x: np.ndarray, table: np.ndarray) -> np.ndarray:
    """tosa.table, int16 in, 513-entry int16 table, int32 out: linear interpolation over the low 7 bits."""
    v = x.astype(np.int64)
    t = table.astype(np.int64).reshape(-1)
    index = (v + 32768) >> 7
    frac = v & 0x7F
    base, nxt = t[index], t[index + 1]
    return ((base << 7) + (nxt - base) * frac).astype(np.int32)


def softmax(x: np.ndarray, dtype: str) -> np.ndarray:
    """softmax over the last axis, fp32 inside (tolerance class: the device's exp and summation order differ)."""
    v, _ = _load(x, dtype)
    v = v.astype(np.float32)
    e = np.exp(v - v.max(axis=-1, keepdims=True))
    return _store(e / e.sum(axis=-1, keepdims=True), True, dtype)
