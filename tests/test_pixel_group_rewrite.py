"""The planner rewrites a narrow stride-1 KH x 3 convolution as the same convolution on pixel groups: tensors read as
[N, H, W / G, G C] -> [N, OH, OW / G, G OC], weights placed at [(j, oc)][kh][kp][(h, c)] for kw = G (kp - 1) + h - j + 1
(csrc/plan.cu). This checks the algebra of that rewrite on the CPU oracle: the transformed op gives the same bytes."""
import numpy as np
import pytest

from oracle_exec import run_graph
from torq_b200.oplist import Graph
from torq_b200.quant import quantize_multipliers


def group_weights(w, G):
    OC, KH, KW, C = w.shape
    assert KW == 3
    out = np.zeros((G * OC, KH, 3, G * C), np.int8)
    for j in range(G):
        for kp in range(3):
            for h in range(G):
                kw = G * (kp - 1) + h - j + 1
                if 0 <= kw < 3:
                    out[j * OC:(j + 1) * OC, :, kp, h * C:(h + 1) * C] = w[:, :, kw, :]
    return out


@pytest.mark.parametrize("G,shape,OC,KH,pad_tb,izp", [
    (2, (2, 9, 12, 16), 16, 3, (1, 1), -6),
    (4, (1, 7, 16, 16), 32, 3, (1, 1), 5),
    (2, (1, 11, 10, 32), 48, 5, (2, 2), 9),
    (2, (1, 8, 14, 32), 32, 3, (0, 0), 0),
])
def test_pixel_group_convolution_equals_the_original(G, shape, OC, KH, pad_tb, izp):
    rng = np.random.default_rng(G * 100 + KH)
    N, H, W, C = shape
    x = rng.integers(-128, 128, shape, dtype=np.int8)
    w = rng.integers(-127, 128, (OC, KH, 3, C), dtype=np.int8)
    bias = np.round(rng.normal(0, 800, OC)).astype(np.int32)
    m, s = quantize_multipliers(rng.uniform(0.5, 1.5, OC) * 40.0 / (np.sqrt(KH * 3 * C) * 74 * 74))
    pad = (pad_tb[0], pad_tb[1], 1, 1)

    g = Graph()
    g.output(g.conv2d(g.input(shape), w, bias, m, s, pad=pad, input_zp=izp, out_zp=-4, clamp=(-120, 110)))
    want = run_graph(g, [x])[0]

    g2 = Graph()
    g2.output(g2.conv2d(g2.input((N, H, W // G, G * C)), group_weights(w, G), np.tile(bias, G), np.tile(m, G), np.tile(s, G),
                        pad=pad, input_zp=izp, out_zp=-4, clamp=(-120, 110)))
    got = run_graph(g2, [x.reshape(N, H, W // G, G * C)])[0]
    assert got.shape == (N, want.shape[1], W // G, G * OC)
    assert (got.reshape(want.shape) == want).all()
    assert len(np.unique(want)) > 20
