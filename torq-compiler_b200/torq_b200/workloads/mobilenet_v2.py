"""MobileNetV2 (width 1.0) int8, random-init, as an op-list graph.

Topology: 3x3 stride-2 stem to 32 channels; 17 inverted-residual blocks
(t, c, n, s) = (1,16,1,1) (6,24,2,2) (6,32,3,2) (6,64,4,2) (6,96,3,1) (6,160,3,2)
(6,320,1,1); 1x1 head to 1280; global average pool; FC to 1000. ReLU6 follows
the stem, expand, depthwise and head convolutions (folded into the clamp range);
the residual add is the TOSA rescale-add-rescale form. "SAME" padding follows
the TFLite convention the reference's Keras models make explicit with their
block_N_pad layers (tests/test_mbv2.py:26-28): 3x3 stride 1 pads 1 on every
side, 3x3 stride 2 on an even extent pads (top,bottom,left,right) = (0,1,0,1).

Weights: int8 uniform [-127,127], symmetric per output channel. Activations:
per-tensor asymmetric, scales in [0.01,0.1], zero points in [-10,10]. Bias:
int32 normal(0,1000). Weight scales are chosen analytically so that the
pre-activation spread stays inside the quantised range (otherwise every output
would saturate and a parity check would see only two values).
"""
from __future__ import annotations

import math

import numpy as np

from ..oplist import Graph
from ..quant import add_rescale_params, quantize_multipliers, relu6_clamp

BLOCKS = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]
W_VAR = 127.0 * 128.0 / 3.0  # variance of an int8 weight uniform on [-127,127]


class _Act:
    """A quantised activation and the second moment of the real values it holds."""

    def __init__(self, t, scale, zp, m2):
        self.t, self.scale, self.zp, self.m2 = t, scale, zp, m2


def _same_pad(size, k, s):
    out = -(-size // s)
    total = max((out - 1) * s + k - size, 0)
    return total // 2, total - total // 2


class MobileNetV2Builder:
    def __init__(self, batch: int, seed: int = 1234, resolution: int = 224, num_classes: int = 1000):
        self.rng = np.random.default_rng(seed)
        self.g = Graph()
        self.batch, self.resolution, self.num_classes = batch, resolution, num_classes
        self.layers = []  # (name, kind, macs_per_image, in_bytes_per_image, out_bytes_per_image, weight_bytes)

    # -- quantisation parameter draws ------------------------------------
    def _relu6_out(self):
        zp = int(self.rng.integers(-10, 11))
        # the natural scale of a [0,6] range, jittered but kept inside [0.01,0.1]
        scale = float(np.clip(6.0 / 255.0 * self.rng.uniform(0.9, 1.3), 0.01, 0.1))
        return scale, zp

    def _linear_out(self):
        return float(self.rng.uniform(0.02, 0.1)), int(self.rng.integers(-10, 11))

    def _conv_params(self, k_taps, oc, x: _Act, out_scale, sigma_real):
        """Per-channel weight scales giving a pre-activation std of about sigma_real."""
        base = sigma_real / math.sqrt(max(k_taps * x.m2 * W_VAR, 1e-12))
        w_scale = base * self.rng.uniform(0.7, 1.3, oc)
        mult, shift = quantize_multipliers(x.scale * w_scale / out_scale)
        bias = np.round(self.rng.normal(0.0, 1000.0, oc)).astype(np.int32)
        return mult, shift, bias

    def _record(self, name, kind, macs, tin, tout, wbytes):
        n = self.batch
        self.layers.append(dict(name=name, kind=kind, macs=macs // n, in_bytes=int(np.prod(tin.shape)) // n,
                                out_bytes=int(np.prod(tout.shape)) // n, weight_bytes=wbytes))

    # -- layers -------------------------------------------------------------
    def conv(self, name, x: _Act, oc, k, stride, relu6: bool) -> _Act:
        N, H, W, IC = x.t.shape
        w = self.rng.integers(-127, 128, (oc, k, k, IC), dtype=np.int8)
        out_scale, out_zp = self._relu6_out() if relu6 else self._linear_out()
        sigma = 2.5 if relu6 else out_scale * 40.0
        mult, shift, bias = self._conv_params(k * k * IC, oc, x, out_scale, sigma)
        pt, pb = _same_pad(H, k, stride)
        pl, pr = _same_pad(W, k, stride)
        clamp = relu6_clamp(out_scale, out_zp) if relu6 else (-128, 127)
        y = self.g.conv2d(x.t, w, bias, mult, shift, stride=(stride, stride), pad=(pt, pb, pl, pr), input_zp=x.zp,
                          out_zp=out_zp, clamp=clamp)
        self._record(name, "conv2d", int(np.prod(y.shape)) * k * k * IC, x.t, y, w.size)
        m2 = 0.5 * min(sigma, 6.0) ** 2 if relu6 else sigma ** 2
        return _Act(y, out_scale, out_zp, m2)

    def depthwise(self, name, x: _Act, stride) -> _Act:
        N, H, W, Cc = x.t.shape
        w = self.rng.integers(-127, 128, (3, 3, Cc, 1), dtype=np.int8)
        out_scale, out_zp = self._relu6_out()
        mult, shift, bias = self._conv_params(9, Cc, x, out_scale, 2.5)
        pt, pb = _same_pad(H, 3, stride)
        pl, pr = _same_pad(W, 3, stride)
        y = self.g.depthwise_conv2d(x.t, w, bias, mult, shift, stride=(stride, stride), pad=(pt, pb, pl, pr),
                                    input_zp=x.zp, out_zp=out_zp, clamp=relu6_clamp(out_scale, out_zp))
        self._record(name, "depthwise", int(np.prod(y.shape)) * 9, x.t, y, w.size)
        return _Act(y, out_scale, out_zp, 0.5 * 2.5 ** 2)

    def add(self, name, a: _Act, b: _Act) -> _Act:
        out_scale, out_zp = self._linear_out()
        out_scale = max(out_scale, math.sqrt(a.m2 + b.m2) / 45.0)
        m0, m1, mo = add_rescale_params(a.scale, b.scale, out_scale)
        y = self.g.add(a.t, b.t, a_zp=a.zp, a_ms=m0, b_zp=b.zp, b_ms=m1, out_ms=mo, out_zp=out_zp)
        self.layers.append(dict(name=name, kind="add", macs=0, in_bytes=2 * int(np.prod(y.shape)) // self.batch,
                                out_bytes=int(np.prod(y.shape)) // self.batch, weight_bytes=0))
        return _Act(y, out_scale, out_zp, a.m2 + b.m2)

    def build(self) -> Graph:
        g, N, R = self.g, self.batch, self.resolution
        in_scale = float(self.rng.uniform(0.015, 0.025))
        in_zp = int(self.rng.integers(-10, 11))
        x = _Act(g.input((N, R, R, 3)), in_scale, in_zp, (in_scale * 74.0) ** 2)
        self.input_scale, self.input_zp = in_scale, in_zp
        x = self.conv("stem", x, 32, 3, 2, True)
        cin = 32
        bi = 0
        for t, c, n, s in BLOCKS:
            for r in range(n):
                stride = s if r == 0 else 1
                inp = x
                h = x
                if t != 1:
                    h = self.conv(f"block{bi}_expand", h, cin * t, 1, 1, True)
                h = self.depthwise(f"block{bi}_dw", h, stride)
                h = self.conv(f"block{bi}_project", h, c, 1, 1, False)
                if stride == 1 and cin == c:
                    h = self.add(f"block{bi}_add", inp, h)
                x = h
                cin = c
                bi += 1
        x = self.conv("head", x, 1280, 1, 1, True)
        Nn, H, W, Cc = x.t.shape
        gap_zp = int(self.rng.integers(-10, 11))
        y = g.avg_pool2d(x.t, (H, W), (1, 1), input_zp=x.zp, output_zp=gap_zp)
        self.layers.append(dict(name="gap", kind="avgpool", macs=0, in_bytes=H * W * Cc, out_bytes=Cc, weight_bytes=0))
        x = _Act(g.reshape(y, (N, Cc)), x.scale, gap_zp, x.m2 / 2)
        w = self.rng.integers(-127, 128, (self.num_classes, Cc), dtype=np.int8)
        out_scale, out_zp = self._linear_out()
        mult, shift, bias = self._conv_params(Cc, self.num_classes, x, out_scale, out_scale * 40.0)
        logits = g.fully_connected(x.t, w, bias, mult, shift, input_zp=x.zp, out_zp=out_zp)
        self.layers.append(dict(name="fc", kind="fc", macs=Cc * self.num_classes, in_bytes=Cc,
                                out_bytes=self.num_classes, weight_bytes=w.size))
        g.output(logits)
        return g


def build_mobilenet_v2(batch: int, seed: int = 1234, resolution: int = 224):
    """Returns (graph, layer table). The layer table has per-image MACs and bytes."""
    b = MobileNetV2Builder(batch, seed, resolution)
    g = b.build()
    return g, b.layers


def synthetic_images(batch: int, seed: int = 1234, resolution: int = 224) -> np.ndarray:
    rng = np.random.default_rng(seed + 1)
    return rng.integers(-128, 128, (batch, resolution, resolution, 3), dtype=np.int8)
