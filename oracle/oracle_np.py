"""Second, independent restatement of the oracle in numpy (int64 arithmetic).

TEST INFRASTRUCTURE ONLY. PARITY UNPINNED (no golden outputs exist in the
reference; see tosa_oracle.h). Its one purpose: tosa_oracle.c and this file are
written separately and must agree bit-for-bit on seeded cases, so that a slip
in either restatement shows before a GPU kernel is compared with them.

Arithmetic order follows
compiler/torq/Conversions/LinalgToTorqHL/PatternUtils.cpp:426-451,3441-3451
(extsi -> subi(zp) -> apply_scale -> addi(zp) -> maxsi -> minsi -> trunci) and
TOSA 1.0.1 apply_scale_32.
"""
from __future__ import annotations

import math

import numpy as np


def wrap32(v):
    """int32 wrap-around of an int64 array (compiler/torq/Utils/ConversionUtils.cpp:40-45)."""
    v = np.asarray(v, dtype=np.int64)
    return ((v + (1 << 31)) & 0xFFFFFFFF) - (1 << 31)


def apply_scale_32(value, multiplier, shift, double_round=True):
    value = np.asarray(value, dtype=np.int64)
    multiplier = np.asarray(multiplier, dtype=np.int64)
    shift = np.asarray(shift, dtype=np.int64)
    rnd = np.left_shift(np.int64(1), shift - 1)
    if double_round:
        extra = np.where(value >= 0, np.int64(1 << 30), np.int64(-(1 << 30)))
        rnd = rnd + np.where(shift > 31, extra, 0)
    r = value * multiplier + rnd
    r = np.right_shift(r, shift)  # arithmetic on int64
    return wrap32(r)


def reciprocal_scale(count: int):
    """compiler/torq/Conversions/TosaToTorqHL/Patterns.cpp:796-805."""
    k = (count - 1).bit_length()
    numerator = ((1 << 30) + 1) << k
    return numerator // count, 30 + k


def quantize_multiplier(real: float):
    if real == 0.0:
        return 0, 2
    q, e = math.frexp(real)
    f = q * (1 << 31)  # llround semantics: ties away from zero
    m = int(math.floor(f + 0.5)) if f >= 0 else -int(math.floor(-f + 0.5))
    if m == (1 << 31):
        m //= 2
        e += 1
    s = 31 - e
    if s > 62:
        m >>= s - 62
        s = 62
    return m, s


def requant(acc, multiplier, shift, out_zp, clamp_min, clamp_max, double_round=True, mode=0):
    """acc [..., OC] int64 (already wrapped to int32 range)."""
    multiplier = np.asarray(multiplier, dtype=np.int64)
    shift = np.asarray(shift, dtype=np.int64)
    if mode == 0:
        r = apply_scale_32(acc, multiplier, shift, double_round)
    else:  # compiler/torq/Utils/Kernel.h:607-635
        sh = int(shift.min())
        scale = np.right_shift(multiplier, shift - sh)
        r = wrap32(np.right_shift(acc * scale + (1 << (sh - 1)), sh))
    r = wrap32(r + out_zp)
    return np.clip(r, clamp_min, clamp_max).astype(np.int8)


def _out_dim(i, k, s, d, p0, p1):
    return (i + p0 + p1 - d * (k - 1) - 1) // s + 1


def conv2d(x, w, bias, multiplier, shift, out_zp, clamp_min, clamp_max, stride=(1, 1), dilation=(1, 1),
           pad=(0, 0, 0, 0), input_zp=0, weight_zp=0, double_round=True, mode=0):
    x = np.asarray(x, np.int64)
    w = np.asarray(w, np.int64)
    N, H, W, IC = x.shape
    OC, KH, KW, _ = w.shape
    OH = _out_dim(H, KH, stride[0], dilation[0], pad[0], pad[1])
    OW = _out_dim(W, KW, stride[1], dilation[1], pad[2], pad[3])
    # literal padding with input_zp: padded taps then contribute exactly zero
    xp = np.full((N, H + pad[0] + pad[1], W + pad[2] + pad[3], IC), input_zp, np.int64)
    xp[:, pad[0]:pad[0] + H, pad[2]:pad[2] + W, :] = x
    acc = np.zeros((N, OH, OW, OC), np.int64)
    for kh in range(KH):
        for kw in range(KW):
            ys = kh * dilation[0]
            xs = kw * dilation[1]
            patch = xp[:, ys:ys + (OH - 1) * stride[0] + 1:stride[0], xs:xs + (OW - 1) * stride[1] + 1:stride[1], :]
            acc += np.einsum("nhwc,oc->nhwo", patch - input_zp, w[:, kh, kw, :] - weight_zp)
    acc = wrap32(wrap32(acc) + np.asarray(bias, np.int64))
    return requant(acc, multiplier, shift, out_zp, clamp_min, clamp_max, double_round, mode)


def depthwise(x, w, bias, multiplier, shift, out_zp, clamp_min, clamp_max, stride=(1, 1), dilation=(1, 1),
              pad=(0, 0, 0, 0), input_zp=0, weight_zp=0, double_round=True, mode=0):
    x = np.asarray(x, np.int64)
    w = np.asarray(w, np.int64)
    N, H, W, C = x.shape
    KH, KW, _, M = w.shape
    OH = _out_dim(H, KH, stride[0], dilation[0], pad[0], pad[1])
    OW = _out_dim(W, KW, stride[1], dilation[1], pad[2], pad[3])
    xp = np.full((N, H + pad[0] + pad[1], W + pad[2] + pad[3], C), input_zp, np.int64)
    xp[:, pad[0]:pad[0] + H, pad[2]:pad[2] + W, :] = x
    acc = np.zeros((N, OH, OW, C, M), np.int64)
    for kh in range(KH):
        for kw in range(KW):
            ys = kh * dilation[0]
            xs = kw * dilation[1]
            patch = xp[:, ys:ys + (OH - 1) * stride[0] + 1:stride[0], xs:xs + (OW - 1) * stride[1] + 1:stride[1], :]
            acc += (patch - input_zp)[..., None] * (w[kh, kw] - weight_zp)[None, None, None]
    acc = acc.reshape(N, OH, OW, C * M)
    acc = wrap32(wrap32(acc) + np.asarray(bias, np.int64))
    return requant(acc, multiplier, shift, out_zp, clamp_min, clamp_max, double_round, mode)


def fully_connected(a, w, bias, multiplier, shift, out_zp, clamp_min, clamp_max, input_zp=0, weight_zp=0,
                    double_round=True, mode=0):
    a = np.asarray(a, np.int64) - input_zp
    w = np.asarray(w, np.int64) - weight_zp
    acc = wrap32(wrap32(a @ w.T) + np.asarray(bias, np.int64))
    return requant(acc, multiplier, shift, out_zp, clamp_min, clamp_max, double_round, mode)


def matmul_i32(a, b, a_zp=0, b_zp=0):
    return wrap32((np.asarray(a, np.int64) - a_zp) @ (np.asarray(b, np.int64) - b_zp)).astype(np.int32)


def _windows(x, kernel, stride, pad, fill):
    N, H, W, C = x.shape
    OH = _out_dim(H, kernel[0], stride[0], 1, pad[0], pad[1])
    OW = _out_dim(W, kernel[1], stride[1], 1, pad[2], pad[3])
    xp = np.full((N, H + pad[0] + pad[1], W + pad[2] + pad[3], C), fill, np.int64)
    xp[:, pad[0]:pad[0] + H, pad[2]:pad[2] + W, :] = x
    for kh in range(kernel[0]):
        for kw in range(kernel[1]):
            yield xp[:, kh:kh + (OH - 1) * stride[0] + 1:stride[0], kw:kw + (OW - 1) * stride[1] + 1:stride[1], :]


def maxpool(x, kernel, stride, pad=(0, 0, 0, 0), pad_value=-128):
    out_dtype = np.int16 if np.asarray(x).dtype == np.int16 else np.int8
    x = np.asarray(x, np.int64)
    out = None
    for win in _windows(x, kernel, stride, pad, pad_value):
        out = win.copy() if out is None else np.maximum(out, win)
    return out.astype(out_dtype)


def avgpool(x, kernel, stride, pad=(0, 0, 0, 0), input_zp=0, output_zp=0):
    x = np.asarray(x, np.int64)
    acc = None
    cnt = None
    ones = np.ones_like(x)
    for win, one in zip(_windows(x - input_zp, kernel, stride, pad, 0), _windows(ones, kernel, stride, pad, 0)):
        acc = win.copy() if acc is None else acc + win
        cnt = one.copy() if cnt is None else cnt + one
    acc = wrap32(acc)
    mult = np.zeros_like(cnt)
    sh = np.zeros_like(cnt)
    for c in np.unique(cnt):
        m, s = reciprocal_scale(int(c))
        mult[cnt == c] = m
        sh[cnt == c] = s
    r = wrap32(apply_scale_32(acc, mult, sh, False) + output_zp)
    return np.clip(r, -128, 127).astype(np.int8)


def binary(kind, a, b, a_zp, a_mult, a_shift, b_zp, b_mult, b_shift, out_mult, out_shift, out_zp,
           double_round=True, clamp_min=-128, clamp_max=127, a_lshift=0, b_lshift=0):
    # x_lshift: the exact left shift that the first stage of a two-stage input rescale amounts to
    ra = apply_scale_32((np.asarray(a, np.int64) - a_zp) << a_lshift, a_mult, a_shift, double_round)
    rb = apply_scale_32((np.asarray(b, np.int64) - b_zp) << b_lshift, b_mult, b_shift, double_round)
    v = wrap32({"add": ra + rb, "sub": ra - rb, "mul": ra * rb}[kind])
    r = wrap32(apply_scale_32(v, out_mult, out_shift, double_round) + out_zp)
    return np.clip(r, clamp_min, clamp_max).astype(np.int8)


def table(x, tbl):
    return np.asarray(tbl, np.int8)[np.asarray(x, np.int64) + 128]


def rescale(x, multiplier, shift, input_zp, out_zp, clamp_min=-128, clamp_max=127, double_round=True, mode=0):
    return requant(np.asarray(x, np.int64) - input_zp, multiplier, shift, out_zp, clamp_min, clamp_max,
                   double_round, mode)


def resize_nn2x(x):
    return np.repeat(np.repeat(np.asarray(x, np.int8), 2, axis=1), 2, axis=2)


def concat2(a, b, a_zp, a_mult, a_shift, b_zp, b_mult, b_shift, out_zp, double_round=True):
    ra = rescale(a, a_mult, a_shift, a_zp, out_zp, double_round=double_round)
    rb = rescale(b, b_mult, b_shift, b_zp, out_zp, double_round=double_round)
    return np.concatenate([ra, rb], axis=-1)


# ---- tensor ops outside the layer set: a second, element-by-element statement with Python integers -------------------
# (the vectorised one is oracle/generic_ops.py; the golden generator wants the two to agree bit for bit)

def _wrap_py(v: int, bits: int) -> int:
    v &= (1 << bits) - 1
    return v - (1 << bits) if v >> (bits - 1) else v


def _bf16_round_py(f: float) -> int:
    import struct
    u = struct.unpack("<I", struct.pack("<f", f))[0]
    if f != f:
        return 0x7FC0
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF


def _f32(v: float) -> float:
    return float(np.float32(v))


def ew_elementwise(fn_name, a, a_dtype, b, b_dtype, out_dtype, out_shape, *, arg=0, in_zp=0, out_zp=0, clamp=(0, 0),
                   fclamp=(0.0, 0.0), bool_result=False):
    """Same contract as generic_ops.ew, one element at a time."""
    import math
    bits = {"i8": 8, "i16": 16, "i32": 32}

    def elems(x, dt):
        x = np.broadcast_to(x, out_shape).reshape(-1)
        if dt == "bf16":
            return [float(v) for v in (x.astype(np.uint32) << 16).view(np.float32)], True
        if dt == "f32":
            return [float(v) for v in x], True
        return [int(v) for v in x], False

    xs, xf = elems(a, a_dtype)
    ys, yf = elems(b, b_dtype) if b is not None else ([0] * len(xs), False)
    flt = xf or yf
    out = []
    for x, y in zip(xs, ys):
        if flt:
            x, y = _f32(x), _f32(y)
            r = {"cast": lambda: x, "abs": lambda: abs(x), "negate": lambda: -x, "ceil": lambda: math.copysign(float(math.ceil(x)), x) if math.ceil(x) == 0 else float(math.ceil(x)),
                 "floor": lambda: math.copysign(float(math.floor(x)), x) if math.floor(x) == 0 else float(math.floor(x)), "clamp": lambda: min(max(x, _f32(fclamp[0])), _f32(fclamp[1])),
                 "add": lambda: _f32(x + y), "sub": lambda: _f32(x - y), "mul": lambda: _f32(x * y), "maximum": lambda: max(x, y),
                 "minimum": lambda: min(x, y), "equal": lambda: int(x == y), "greater": lambda: int(x > y),
                 "greater_equal": lambda: int(x >= y),
                 # the float functions through Python's double-precision math, rounded to fp32 (tolerance class)
                 "exp": lambda: _f32(math.exp(min(x, 700.0))), "log": lambda: _f32(math.log(x)) if x > 0 else (float("-inf") if x == 0 else float("nan")),
                 "reciprocal": lambda: _f32(1.0 / x) if x != 0 else math.copysign(float("inf"), x),
                 "rsqrt": lambda: _f32(1.0 / math.sqrt(x)) if x > 0 else (float("inf") if x == 0 else float("nan")),
                 "tanh": lambda: _f32(math.tanh(x)), "sigmoid": lambda: _f32(1.0 / (1.0 + math.exp(-x))) if x > -700 else 0.0,
                 "erf": lambda: _f32(math.erf(x))}[fn_name]()
            if fn_name in ("equal", "greater", "greater_equal"):
                out.append(r)
            elif fn_name == "cast" and bool_result:
                out.append(int(x != 0.0))
            elif out_dtype in bits:
                lo, hi = -(1 << (bits[out_dtype] - 1)), (1 << (bits[out_dtype] - 1)) - 1
                if r != r:
                    q = 0
                else:
                    fl = math.floor(r)
                    d = r - fl
                    q = fl + (1 if d > 0.5 or (d == 0.5 and fl % 2 != 0) else 0)  # nearest, ties to even
                out.append(min(max(q, lo), hi))
            elif out_dtype == "bf16":
                out.append(_bf16_round_py(_f32(r)))
            else:
                out.append(_f32(r))
            continue
        x, y = _wrap_py(x, 32), _wrap_py(y, 32)
        if fn_name == "cast":
            r = int(x != 0) if bool_result else x
            if out_dtype in ("f32", "bf16"):
                out.append(_bf16_round_py(_f32(float(x))) if out_dtype == "bf16" else _f32(float(x)))
                continue
        elif fn_name == "abs":
            r = abs(x)
        elif fn_name == "negate":
            r = out_zp - (x - in_zp)
        elif fn_name == "bitwise_not":
            r = ~x
        elif fn_name == "logical_not":
            r = int(x == 0)
        elif fn_name == "clz":
            r = 32 - (x & 0xFFFFFFFF).bit_length()
        elif fn_name == "clamp":
            r = min(max(x, clamp[0]), clamp[1])
        elif fn_name == "add":
            r = x + y
        elif fn_name == "sub":
            r = x - y
        elif fn_name == "mul":
            r = (x * y + (1 << (arg - 1))) >> arg if arg > 0 else x * y
        elif fn_name == "maximum":
            r = max(x, y)
        elif fn_name == "minimum":
            r = min(x, y)
        elif fn_name == "bitwise_and":
            r = x & y
        elif fn_name == "bitwise_or":
            r = x | y
        elif fn_name == "bitwise_xor":
            r = x ^ y
        elif fn_name == "logical_left_shift":
            r = x << (y & 31)
        elif fn_name == "arithmetic_right_shift":
            sft = y & 31
            r = (x >> sft) + (((x >> (sft - 1)) & 1) if arg and sft > 0 else 0)
        elif fn_name == "equal":
            r = int(x == y)
        elif fn_name == "greater":
            r = int(x > y)
        elif fn_name == "greater_equal":
            r = int(x >= y)
        elif fn_name == "logical_and":
            r = int(x != 0 and y != 0)
        elif fn_name == "logical_or":
            r = int(x != 0 or y != 0)
        elif fn_name == "logical_xor":
            r = int((x != 0) != (y != 0))
        else:
            raise NotImplementedError(fn_name)
        out.append(_wrap_py(r, bits.get(out_dtype, 32)))
    np_t = {"i8": np.int8, "i16": np.int16, "i32": np.int32, "f32": np.float32, "bf16": np.uint16}[out_dtype]
    return np.array(out, dtype=np_t).reshape(out_shape)


def rescale_elementwise(x, in_dtype, out_dtype, mult, shift, in_zp, out_zp, clamp, *, per_channel, double_round,
                        input_unsigned=False):
    bits = {"i8": 8, "i16": 16, "i32": 32}
    flat = x.reshape(-1)
    C = x.shape[-1]
    out = []
    for i, v in enumerate(int(t) for t in flat):
        if input_unsigned:
            v &= (1 << bits[in_dtype]) - 1
        v = _wrap_py(v - in_zp, 32)
        m, s = (int(mult[i % C]), int(shift[i % C])) if per_channel else (int(mult[0]), int(shift[0]))
        rnd = 1 << (s - 1)
        if double_round and s > 31:
            rnd += (1 << 30) if v >= 0 else -(1 << 30)
        r = _wrap_py((v * m + rnd) >> s, 32) + out_zp
        out.append(_wrap_py(min(max(r, clamp[0]), clamp[1]), bits[out_dtype]))
    return np.array(out, dtype={"i8": np.int8, "i16": np.int16, "i32": np.int32}[out_dtype]).reshape(x.shape)


def table16_elementwise(x, table):
    t = [int(v) for v in table.reshape(-1)]
    out = []
    for v in (int(q) for q in x.reshape(-1)):
        i, f = (v + 32768) >> 7, v & 0x7F
        out.append(t[i] * 128 + (t[i + 1] - t[i]) * f)
    return np.array(out, np.int32).reshape(x.shape)


def conv2d_i16_elementwise(x, w, bias, mult, shift, stride, dilation, pad, input_zp, weight_zp, out_zp, clamp_min, clamp_max):
    """Element-by-element statement with Python integers of the int16 convolution + 16-bit rescale (small cases only)."""
    N, H, W, IC = x.shape
    OC, KH, KW, _ = w.shape
    OH = (H + pad[0] + pad[1] - (KH - 1) * dilation[0] - 1) // stride[0] + 1
    OW = (W + pad[2] + pad[3] - (KW - 1) * dilation[1] - 1) // stride[1] + 1
    xl, wl = x.tolist(), w.tolist()
    bl = [int(v) for v in np.asarray(bias).reshape(-1)]
    ml = [int(v) for v in np.asarray(mult).reshape(-1)]
    sl = [int(v) for v in np.asarray(shift).reshape(-1)]
    out = np.empty((N, OH, OW, OC), np.int16)
    for n in range(N):
        for oh in range(OH):
            for ow in range(OW):
                for oc in range(OC):
                    acc = bl[oc if len(bl) > 1 else 0]
                    for kh in range(KH):
                        ih = oh * stride[0] - pad[0] + kh * dilation[0]
                        if not 0 <= ih < H:
                            continue
                        for kw in range(KW):
                            iw = ow * stride[1] - pad[2] + kw * dilation[1]
                            if not 0 <= iw < W:
                                continue
                            px, wt = xl[n][ih][iw], wl[oc][kh][kw]
                            for c in range(IC):
                                acc += (px[c] - input_zp) * (wt[c] - weight_zp)
                    m, sh = ml[oc if len(ml) > 1 else 0], sl[oc if len(sl) > 1 else 0]
                    r = ((acc * m + (1 << (sh - 1))) >> sh) + out_zp
                    out[n, oh, ow, oc] = min(max(r, clamp_min), clamp_max)
    return out
