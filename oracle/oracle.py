"""ctypes front of libtosa_oracle.so (the C restatement in tosa_oracle.c).

TEST INFRASTRUCTURE ONLY. PARITY UNPINNED: the reference tree holds no golden
outputs for this path; see tosa_oracle.h.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class _Requant(C.Structure):
    _fields_ = [
        ("multiplier", C.POINTER(C.c_int32)),
        ("shift", C.POINTER(C.c_int8)),
        ("per_channel", C.c_int32),
        ("double_round", C.c_int32),
        ("mode", C.c_int32),
        ("out_zp", C.c_int32),
        ("clamp_min", C.c_int32),
        ("clamp_max", C.c_int32),
    ]


def build() -> str:
    """Compile the oracle if its .so is missing or older than its sources."""
    so = os.path.join(_HERE, "libtosa_oracle.so")
    srcs = [os.path.join(_HERE, f) for f in ("tosa_oracle.c", "tosa_oracle.h")]
    if not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in srcs):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libtosa_oracle.so"], stdout=subprocess.DEVNULL)
    return so


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
        _LIB.tq_apply_scale_32.restype = C.c_int32
        _LIB.tq_apply_scale_32.argtypes = [C.c_int32] * 4
        _LIB.tq_num_threads.restype = C.c_int
    return _LIB


def _p8(a):
    return a.ctypes.data_as(C.POINTER(C.c_int8))


def _p32(a):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def _i8(a):
    a = np.ascontiguousarray(a, dtype=np.int8)
    return a


class Requant:
    """multiplier/shift (+ zero point and clamp) of the tosa.rescale that ends an op."""

    def __init__(self, multiplier, shift, out_zp=0, clamp_min=-128, clamp_max=127,
                 per_channel=None, double_round=True, mode=0):
        self.multiplier = np.ascontiguousarray(np.atleast_1d(multiplier), dtype=np.int32)
        self.shift = np.ascontiguousarray(np.atleast_1d(shift), dtype=np.int8)
        assert self.multiplier.shape == self.shift.shape
        self.per_channel = (self.multiplier.size > 1) if per_channel is None else bool(per_channel)
        self.double_round = bool(double_round)
        self.mode = int(mode)
        self.out_zp, self.clamp_min, self.clamp_max = int(out_zp), int(clamp_min), int(clamp_max)

    def c(self):
        return _Requant(_p32(self.multiplier), _p8(self.shift), int(self.per_channel),
                        int(self.double_round), self.mode, self.out_zp, self.clamp_min, self.clamp_max)


def apply_scale_32(value, multiplier, shift, double_round=True) -> int:
    return lib().tq_apply_scale_32(int(value), int(multiplier), int(shift), int(double_round))


def reciprocal_scale(count):
    m, s = C.c_int32(), C.c_int32()
    lib().tq_reciprocal_scale(C.c_uint32(count), C.byref(m), C.byref(s))
    return m.value, s.value


def quantize_multiplier(real):
    m, s = C.c_int32(), C.c_int32()
    lib().tq_quantize_multiplier(C.c_double(real), C.byref(m), C.byref(s))
    return m.value, s.value


def num_threads() -> int:
    return lib().tq_num_threads()


def set_num_threads(n: int):
    lib().tq_set_num_threads(int(n))


def out_dim(i, k, s, d, p0, p1):
    return (i + p0 + p1 - d * (k - 1) - 1) // s + 1


def conv2d(x, w, bias, rq: Requant, stride=(1, 1), dilation=(1, 1), pad=(0, 0, 0, 0), input_zp=0,
           weight_zp=0):
    """x NHWC int8, w OHWI int8, pad = (top, bottom, left, right)."""
    x, w = _i8(x), _i8(w)
    bias = np.ascontiguousarray(bias, dtype=np.int32)
    N, H, W, IC = x.shape
    OC, KH, KW, IC2 = w.shape
    assert IC == IC2
    OH = out_dim(H, KH, stride[0], dilation[0], pad[0], pad[1])
    OW = out_dim(W, KW, stride[1], dilation[1], pad[2], pad[3])
    out = np.empty((N, OH, OW, OC), np.int8)
    r = rq.c()
    lib().tq_conv2d(_p8(x), N, H, W, IC, _p8(w), OC, KH, KW, _p32(bias), bias.size, stride[0], stride[1],
                    dilation[0], dilation[1], pad[0], pad[1], pad[2], pad[3], int(input_zp), int(weight_zp),
                    C.byref(r), _p8(out), OH, OW)
    return out


def depthwise(x, w, bias, rq: Requant, stride=(1, 1), dilation=(1, 1), pad=(0, 0, 0, 0), input_zp=0,
              weight_zp=0):
    """x NHWC int8, w [KH,KW,C,M] int8."""
    x, w = _i8(x), _i8(w)
    bias = np.ascontiguousarray(bias, dtype=np.int32)
    N, H, W, Cc = x.shape
    KH, KW, C2, M = w.shape
    assert Cc == C2
    OH = out_dim(H, KH, stride[0], dilation[0], pad[0], pad[1])
    OW = out_dim(W, KW, stride[1], dilation[1], pad[2], pad[3])
    out = np.empty((N, OH, OW, Cc * M), np.int8)
    r = rq.c()
    lib().tq_depthwise(_p8(x), N, H, W, Cc, _p8(w), M, KH, KW, _p32(bias), bias.size, stride[0], stride[1],
                       dilation[0], dilation[1], pad[0], pad[1], pad[2], pad[3], int(input_zp),
                       int(weight_zp), C.byref(r), _p8(out), OH, OW)
    return out


def fully_connected(a, w, bias, rq: Requant, input_zp=0, weight_zp=0):
    """a [M,K] int8, w [N,K] int8."""
    a, w = _i8(a), _i8(w)
    bias = np.ascontiguousarray(bias, dtype=np.int32)
    M, K = a.shape
    N, K2 = w.shape
    assert K == K2
    out = np.empty((M, N), np.int8)
    r = rq.c()
    lib().tq_fully_connected(_p8(a), M, K, _p8(w), N, _p32(bias), bias.size, int(input_zp),
                             int(weight_zp), C.byref(r), _p8(out))
    return out


def matmul_i32(a, b, a_zp=0, b_zp=0):
    a, b = _i8(a), _i8(b)
    M, K = a.shape
    K2, N = b.shape
    assert K == K2
    out = np.empty((M, N), np.int32)
    lib().tq_matmul_i32(_p8(a), M, K, _p8(b), N, int(a_zp), int(b_zp), _p32(out))
    return out


def maxpool(x, kernel, stride, pad=(0, 0, 0, 0), pad_value=-128):
    """int8, or int16 when x is an int16 array."""
    if np.asarray(x).dtype == np.int16:
        x = np.ascontiguousarray(x)
        N, H, W, Cc = x.shape
        OH = out_dim(H, kernel[0], stride[0], 1, pad[0], pad[1])
        OW = out_dim(W, kernel[1], stride[1], 1, pad[2], pad[3])
        out = np.empty((N, OH, OW, Cc), np.int16)
        p16 = C.POINTER(C.c_int16)
        lib().tq_maxpool_i16(x.ctypes.data_as(p16), N, H, W, Cc, kernel[0], kernel[1], stride[0], stride[1], pad[0],
                             pad[2], int(pad_value), out.ctypes.data_as(p16), OH, OW)
        return out
    x = _i8(x)
    N, H, W, Cc = x.shape
    OH = out_dim(H, kernel[0], stride[0], 1, pad[0], pad[1])
    OW = out_dim(W, kernel[1], stride[1], 1, pad[2], pad[3])
    out = np.empty((N, OH, OW, Cc), np.int8)
    lib().tq_maxpool(_p8(x), N, H, W, Cc, kernel[0], kernel[1], stride[0], stride[1], pad[0], pad[1],
                     pad[2], pad[3], int(pad_value), _p8(out), OH, OW)
    return out


def avgpool(x, kernel, stride, pad=(0, 0, 0, 0), input_zp=0, output_zp=0):
    x = _i8(x)
    N, H, W, Cc = x.shape
    OH = out_dim(H, kernel[0], stride[0], 1, pad[0], pad[1])
    OW = out_dim(W, kernel[1], stride[1], 1, pad[2], pad[3])
    out = np.empty((N, OH, OW, Cc), np.int8)
    lib().tq_avgpool(_p8(x), N, H, W, Cc, kernel[0], kernel[1], stride[0], stride[1], pad[0], pad[1],
                     pad[2], pad[3], int(input_zp), int(output_zp), _p8(out), OH, OW)
    return out


_KIND = {"add": 0, "sub": 1, "mul": 2}


def binary(kind, a, b, a_zp, a_mult, a_shift, b_zp, b_mult, b_shift, out_mult, out_shift, out_zp,
           double_round=True, clamp_min=-128, clamp_max=127, a_lshift=0, b_lshift=0):
    a, b = _i8(a), _i8(b)
    assert a.shape == b.shape
    out = np.empty(a.shape, np.int8)
    lib().tq_binary_pre(_KIND[kind], _p8(a), _p8(b), C.c_int64(a.size), int(a_zp), int(a_lshift), int(a_mult),
                        int(a_shift), int(b_zp), int(b_lshift), int(b_mult), int(b_shift), int(out_mult),
                        int(out_shift), int(out_zp), int(double_round), int(clamp_min), int(clamp_max), _p8(out))
    return out


def table(x, tbl):
    x, tbl = _i8(x), _i8(tbl)
    assert tbl.size == 256
    out = np.empty(x.shape, np.int8)
    lib().tq_table(_p8(x), C.c_int64(x.size), _p8(tbl), _p8(out))
    return out


def rescale(x, rq: Requant, input_zp=0):
    x = _i8(x)
    Cc = x.shape[-1]
    out = np.empty(x.shape, np.int8)
    r = rq.c()
    lib().tq_rescale(_p8(x), C.c_int64(x.size // Cc), Cc, int(input_zp), C.byref(r), _p8(out))
    return out


def resize_nn2x(x):
    x = _i8(x)
    N, H, W, Cc = x.shape
    out = np.empty((N, 2 * H, 2 * W, Cc), np.int8)
    lib().tq_resize_nn2x(_p8(x), N, H, W, Cc, _p8(out))
    return out


def concat2(a, b, a_zp, a_mult, a_shift, b_zp, b_mult, b_shift, out_zp, double_round=True):
    a, b = _i8(a), _i8(b)
    Ca, Cb = a.shape[-1], b.shape[-1]
    rows = a.size // Ca
    assert b.size // Cb == rows
    out = np.empty(a.shape[:-1] + (Ca + Cb,), np.int8)
    lib().tq_concat2(_p8(a), Ca, _p8(b), Cb, C.c_int64(rows), int(a_zp), int(a_mult), int(a_shift),
                     int(b_zp), int(b_mult), int(b_shift), int(out_zp), int(double_round), _p8(out))
    return out
