"""YOLOv8n-style int8 detector, random-init, as an op-list graph.

Backbone: conv s2 to 16 ch, conv s2 to 32, C2f(32, n=1), conv s2 to 64, C2f(64, n=2),
conv s2 to 128, C2f(128, n=2), conv s2 to 256, C2f(256, n=1), SPPF (5x5 max pool x3).
Neck: PAN-FPN with nearest 2x upsample and rescaled concat. Head: three decoupled detect
heads at strides 8/16/32, each giving 64 box channels (DFL, reg_max 16) and 80 class
channels. Every convolution is followed by SiLU as a 256-entry int8 table
(the form the reference fuses: tests/testdata/tosa_ops/yolov8_block_mul_rescale.mlir,
compiler/torq/Transforms/Linalg/OptimizeSwishActivationPattern.cpp:100-190), except the
final 1x1 of each head branch. Weights: per-channel symmetric int8 uniform [-127,127];
activations per-tensor asymmetric int8; bias int32 normal(0,1000).

A C2f block's first 1x1 convolution is emitted as two convolutions (one per half of its
output channels): that is the same arithmetic as one convolution followed by a channel
split, and needs no slice op.
"""
from __future__ import annotations

import math

import numpy as np

from ..oplist import Graph
from ..quant import add_rescale_params, quantize_multiplier, quantize_multipliers

W_VAR = 127.0 * 128.0 / 3.0
POST_SCALE = 6.7 / 255.0          # SiLU output range [-0.28, 6.4]
POST_ZP = -128 + int(round(0.28 / POST_SCALE))


class _Act:
    def __init__(self, t, scale, zp, m2):
        self.t, self.scale, self.zp, self.m2 = t, scale, zp, m2


def silu_table(in_scale, in_zp, out_scale, out_zp):
    q = np.arange(-128, 128, dtype=np.float64)
    x = in_scale * (q - in_zp)
    y = x / (1.0 + np.exp(-x))
    return np.clip(np.round(y / out_scale) + out_zp, -128, 127).astype(np.int8)


class YoloV8nBuilder:
    def __init__(self, batch: int, resolution: int = 640, seed: int = 1234, num_classes: int = 80):
        self.rng = np.random.default_rng(seed)
        self.g = Graph()
        self.batch, self.res, self.nc = batch, resolution, num_classes
        self.macs = 0

    def conv(self, x: _Act, oc, k, s, act=True) -> _Act:
        N, H, W, IC = x.t.shape
        w = self.rng.integers(-127, 128, (oc, k, k, IC), dtype=np.int8)
        pre_scale = float(self.rng.uniform(0.03, 0.06))
        pre_zp = int(self.rng.integers(-10, 11))
        sigma = 2.0
        w_scale = sigma / math.sqrt(max(k * k * IC * x.m2 * W_VAR, 1e-12)) * self.rng.uniform(0.7, 1.3, oc)
        mult, shift = quantize_multipliers(x.scale * w_scale / pre_scale)
        bias = np.round(self.rng.normal(0.0, 1000.0, oc)).astype(np.int32)
        p = (k - 1) // 2
        pad = (p, p, p, p) if s == 1 else (p - 1 if k == 3 and H % 2 == 0 else p, p, p - 1 if k == 3 and W % 2 == 0 else p, p)
        y = self.g.conv2d(x.t, w, bias, mult, shift, stride=(s, s), pad=pad, input_zp=x.zp, out_zp=pre_zp)
        self.macs += int(np.prod(y.shape)) * k * k * IC // self.batch
        if not act:
            return _Act(y, pre_scale, pre_zp, sigma ** 2)
        z = self.g.table(y, silu_table(pre_scale, pre_zp, POST_SCALE, POST_ZP))
        return _Act(z, POST_SCALE, POST_ZP, 1.4)

    def add(self, a: _Act, b: _Act) -> _Act:
        out_scale = POST_SCALE * 1.6
        m0, m1, mo = add_rescale_params(a.scale, b.scale, out_scale)
        y = self.g.add(a.t, b.t, a_zp=a.zp, a_ms=m0, b_zp=b.zp, b_ms=m1, out_ms=mo, out_zp=POST_ZP)
        return _Act(y, out_scale, POST_ZP, a.m2 + b.m2)

    def concat(self, parts) -> _Act:
        out_scale = max(p.scale for p in parts)
        acc = parts[0]
        for nxt in parts[1:]:
            y = self.g.concat(acc.t, nxt.t, a_zp=acc.zp, a_ms=quantize_multiplier(acc.scale / out_scale), b_zp=nxt.zp,
                              b_ms=quantize_multiplier(nxt.scale / out_scale), out_zp=POST_ZP)
            ca, cb = acc.t.shape[-1], nxt.t.shape[-1]
            acc = _Act(y, out_scale, POST_ZP, (acc.m2 * ca + nxt.m2 * cb) / (ca + cb))
        return acc

    def maxpool5(self, x: _Act) -> _Act:
        return _Act(self.g.maxpool2d(x.t, (5, 5), (1, 1), (2, 2, 2, 2), pad_value=-128), x.scale, x.zp, x.m2)

    def upsample(self, x: _Act) -> _Act:
        return _Act(self.g.resize_nearest_2x(x.t), x.scale, x.zp, x.m2)

    def c2f(self, x: _Act, c, n, shortcut) -> _Act:
        ch = c // 2
        parts = [self.conv(x, ch, 1, 1), self.conv(x, ch, 1, 1)]
        for _ in range(n):
            y = self.conv(self.conv(parts[-1], ch, 3, 1), ch, 3, 1)
            parts.append(self.add(parts[-1], y) if shortcut else y)
        return self.conv(self.concat(parts), c, 1, 1)

    def sppf(self, x: _Act, c) -> _Act:
        y = self.conv(x, c // 2, 1, 1)
        p1 = self.maxpool5(y)
        p2 = self.maxpool5(p1)
        p3 = self.maxpool5(p2)
        return self.conv(self.concat([y, p1, p2, p3]), c, 1, 1)

    def build(self) -> Graph:
        g, N, R = self.g, self.batch, self.res
        in_scale, in_zp = float(self.rng.uniform(0.015, 0.025)), int(self.rng.integers(-10, 11))
        x = _Act(g.input((N, R, R, 3)), in_scale, in_zp, (in_scale * 74.0) ** 2)
        x = self.conv(x, 16, 3, 2)
        x = self.conv(x, 32, 3, 2)
        x = self.c2f(x, 32, 1, True)
        x = self.conv(x, 64, 3, 2)
        p3 = self.c2f(x, 64, 2, True)
        x = self.conv(p3, 128, 3, 2)
        p4 = self.c2f(x, 128, 2, True)
        x = self.conv(p4, 256, 3, 2)
        x = self.c2f(x, 256, 1, True)
        p5 = self.sppf(x, 256)
        # neck
        n4 = self.c2f(self.concat([self.upsample(p5), p4]), 128, 1, False)
        n3 = self.c2f(self.concat([self.upsample(n4), p3]), 64, 1, False)
        d4 = self.c2f(self.concat([self.conv(n3, 64, 3, 2), n4]), 128, 1, False)
        d5 = self.c2f(self.concat([self.conv(d4, 128, 3, 2), p5]), 256, 1, False)
        # decoupled heads
        c_box, c_cls = 64, max(16, min(self.nc, 100))
        for feat in (n3, d4, d5):
            box = self.conv(self.conv(self.conv(feat, c_box, 3, 1), c_box, 3, 1), 64, 1, 1, act=False)
            cls = self.conv(self.conv(self.conv(feat, c_cls, 3, 1), c_cls, 3, 1), self.nc, 1, 1, act=False)
            g.output(box.t)
            g.output(cls.t)
        return g


def build_yolov8n(batch: int, resolution: int = 640, seed: int = 1234):
    """Returns (graph, MACs per image)."""
    b = YoloV8nBuilder(batch, resolution, seed)
    g = b.build()
    return g, b.macs


def synthetic_images(batch: int, resolution: int = 640, seed: int = 1234) -> np.ndarray:
    rng = np.random.default_rng(seed + 1)
    return rng.integers(-128, 128, (batch, resolution, resolution, 3), dtype=np.int8)
