"""Per-op parity of the CUDA path against the CPU oracle, bit-exact, through the C ABI.
Cases mirror the attribute combinations of the reference's TOSA fixtures
(tests/testdata/tosa_ops, tests/testdata/gen_ops) and its seeded input generator
(python/torq/testing/iree.py:1262-1285: seed 1234)."""
import numpy as np
import pytest

from gpu_exec import run_graph_gpu
from oracle_exec import run_graph
from torq_b200.oplist import Graph
from torq_b200.quant import quantize_multiplier, quantize_multipliers

pytestmark = pytest.mark.gpu


def _check(device, g, inputs, host_call=False):
    want = run_graph(g, inputs)
    got = run_graph_gpu(device, g, inputs, host_call=host_call)
    for w, o in zip(want, got):
        assert w.shape == o.shape
        bad = np.flatnonzero(w.ravel() != o.ravel())
        assert bad.size == 0, f"{bad.size} of {w.size} differ; first at {bad[:5]}: want {w.ravel()[bad[:5]]} got {o.ravel()[bad[:5]]}"
        assert len(np.unique(w)) > 2 or w.size < 8
    return got


CONV_CASES = [
    # x shape, OC, kernel, stride, dilation, pad(t,b,l,r), izp, wzp
    ((1, 8, 8, 1), 1, (3, 3), (1, 1), (1, 1), (1, 1, 1, 1), -128, 0),       # gen_ops/conv2d_8x8.mlir
    ((1, 15, 17, 3), 8, (5, 5), (2, 2), (1, 1), (2, 2, 2, 2), 3, 0),        # conv_5x5_odd_frame_stride2 class
    ((2, 9, 11, 5), 7, (3, 3), (2, 1), (1, 1), (1, 1, 0, 1), -3, 0),
    ((1, 13, 13, 4), 6, (5, 5), (2, 2), (1, 1), (2, 2, 2, 2), 7, 3),        # weight zero point
    ((1, 10, 12, 8), 16, (3, 3), (1, 1), (2, 2), (2, 2, 2, 2), 0, 0),       # dilation
    ((3, 6, 6, 16), 24, (1, 1), (1, 1), (1, 1), (0, 0, 0, 0), -5, 0),       # 1x1 = matmul as conv
    ((1, 56, 56, 64), 64, (3, 3), (1, 1), (1, 1), (1, 1, 1, 1), -3, 0),     # single-conv benchmark config
    ((2, 14, 14, 96), 576, (1, 1), (1, 1), (1, 1), (0, 0, 0, 0), 9, 0),
    ((1, 224, 224, 3), 32, (3, 3), (2, 2), (1, 1), (0, 1, 0, 1), -4, 0),    # MobileNetV2 stem
    ((1, 7, 7, 100), 130, (1, 1), (1, 1), (1, 1), (0, 0, 0, 0), 2, -1),
    ((2, 20, 22, 16), 32, (3, 3), (1, 1), (1, 1), (1, 1, 1, 1), -5, 0),     # 16 input channels: direct dp4a kernel
    ((1, 21, 21, 16), 24, (3, 3), (2, 2), (1, 1), (0, 1, 0, 1), 3, 0),
    ((1, 12, 12, 16), 7, (5, 5), (1, 1), (1, 1), (2, 2, 2, 2), 9, 0),
]


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("case", CONV_CASES)
def test_conv2d(device, case, mode):
    shape, OC, k, stride, dil, pad, izp, wzp = case
    rng = np.random.default_rng(1234)
    x = rng.integers(-128, 128, shape, dtype=np.int8)
    w = rng.integers(-127, 128, (OC,) + k + (shape[3],), dtype=np.int8)
    bias = np.round(rng.normal(0, 2000, OC)).astype(np.int32)
    K = k[0] * k[1] * shape[3]
    m, s = quantize_multipliers(rng.uniform(0.5, 1.5, OC) * 40.0 / (np.sqrt(K) * 74 * 74))
    g = Graph()
    y = g.conv2d(g.input(shape), w, bias, m, s, stride=stride, dilation=dil, pad=pad, input_zp=izp, weight_zp=wzp,
                 out_zp=5, clamp=(-128, 127), requant_mode=mode)
    g.output(y)
    _check(device, g, [x])


IGEMM_CASES = [
    # x shape, OC, kernel, stride, pad(t,b,l,r), izp   (IC % 16 == 0, OC % 16 == 0: tensor-core implicit GEMM)
    ((1, 56, 56, 64), 64, (3, 3), 1, (1, 1, 1, 1), -3),      # the benchmark set's single-conv configuration
    ((2, 20, 20, 128), 128, (3, 3), 1, (1, 1, 1, 1), 7),     # ragged patches (20 is no multiple of the patch)
    ((1, 13, 17, 32), 48, (3, 3), 1, (1, 1, 1, 1), -9),      # odd frame, 32-byte rows
    ((2, 40, 40, 64), 128, (3, 3), 2, (0, 1, 0, 1), 4),      # stride 2, TensorFlow SAME padding
    ((1, 33, 29, 96), 32, (3, 3), 2, (1, 1, 1, 1), -1),      # stride 2, odd frame, 96 channels = 3 blocks of 32
    ((1, 24, 24, 256), 272, (3, 3), 1, (1, 1, 1, 1), 5),     # weights too large to stay in shared memory; 3 N tiles
    ((1, 18, 18, 64), 16, (5, 5), 1, (2, 2, 2, 2), 11),      # 25 taps, 3 x 3 border classes per axis
    ((3, 16, 16, 32), 64, (3, 3), 1, (0, 0, 0, 0), 6),       # no padding: no border classes
    ((1, 12, 12, 64), 64, (3, 3), 1, (1, 1, 1, 1), 0),       # zero input zero point: no correction table
    ((1, 9, 140, 32), 32, (1, 7), 1, (0, 0, 3, 3), -20),     # one-row window, wide frame
    ((2, 20, 20, 80), 80, (3, 3), 1, (1, 1, 1, 1), 3),       # 80 channels: the last 32-byte block is half zero fill
    ((1, 30, 34, 16), 32, (3, 3), 2, (0, 1, 0, 1), -6),      # 16 channels, stride 2: pixel pairs of 32 bytes, left pad 0
    ((2, 41, 38, 16), 16, (3, 3), 2, (1, 1, 1, 1), 4),       # the same with left pad 1 and an odd height
    ((1, 30, 33, 16), 32, (3, 3), 2, (1, 1, 1, 1), -6),      # odd width: no pixel pairs (dp4a kernel)
    ((3, 36, 52, 32), 64, (3, 3), 2, (1, 0, 1, 0), 12),      # 32 channels, stride 2, pairs of 64 bytes
    ((1, 64, 64, 64), 64, (3, 3), 2, (1, 1, 1, 1), -1),      # 64 channels, stride 2, pairs of 128 bytes, two K steps
    ((2, 37, 45, 16), 16, (3, 3), 1, (1, 1, 1, 1), -6),      # 16 channels, stride 1: halo patches, rows half zero fill
    ((2, 36, 44, 16), 16, (3, 3), 1, (1, 1, 1, 1), -6),      # the same with a width of 4 k: read as groups of four pixels (64 channels)
    ((2, 21, 42, 16), 32, (3, 3), 1, (1, 1, 1, 1), 5),       # an even width that is no multiple of 4: pixel pairs (32 channels)
    ((1, 22, 30, 32), 48, (3, 3), 1, (1, 1, 1, 1), 9),       # 32 channels as pairs of 64, 48 filters as 96
    ((2, 17, 26, 16), 32, (5, 3), 1, (2, 2, 1, 1), -11),     # five kernel rows over pixel pairs
    ((1, 20, 28, 32), 32, (3, 3), 1, (0, 0, 1, 1), 3),       # pairs, no padding above and below
    ((1, 23, 31, 64), 32, (5, 5), 1, (2, 2, 2, 2), 9),       # 5x5 over halo patches (12 output columns per tile)
    ((1, 19, 33, 128), 64, (3, 3), 1, (1, 1, 1, 1), -2),     # 128-byte rows over halo patches, weights 72 KB resident
    ((1, 11, 11, 48), 16, (3, 3), 1, (1, 1, 1, 1), 8),       # 48 channels in one 64-byte block
]


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("case", IGEMM_CASES)
def test_conv2d_implicit_gemm(device, case, mode):
    from torq_b200.runtime import Executable
    shape, OC, k, stride, pad, izp = case
    rng = np.random.default_rng(1234)
    x = rng.integers(-128, 128, shape, dtype=np.int8)
    w = rng.integers(-127, 128, (OC,) + k + (shape[3],), dtype=np.int8)
    bias = np.round(rng.normal(0, 2000, OC)).astype(np.int32)
    K = k[0] * k[1] * shape[3]
    m, s = quantize_multipliers(rng.uniform(0.5, 1.5, OC) * 40.0 / (np.sqrt(K) * 74 * 74))
    g = Graph()
    y = g.conv2d(g.input(shape), w, bias, m, s, stride=(stride, stride), pad=pad, input_zp=izp, out_zp=-7, clamp=(-128, 127),
                 requant_mode=mode)
    g.output(y)
    ex = Executable(device, g.serialize())
    # 16 input channels make 16-byte operand rows: where neither halo patches nor pixel pairs apply, the dp4a kernel takes those
    assert ex.op_kernels() == ["conv2d_c16_dp4a" if shape[3] == 16 and stride == 2 and shape[2] % 2 else "conv_igemm_i8_tcgen05"]
    ex.destroy()
    _check(device, g, [x])


def test_conv2d_per_tensor_scale_and_relu6_clamp(device):
    rng = np.random.default_rng(1234)
    x = rng.integers(-128, 128, (1, 8, 8, 1), dtype=np.int8)
    w = np.array([[[[119], [23], [-114]], [[115], [-127], [125]], [[7], [-35], [-13]]]], np.int8)  # conv2d_8x8.mlir
    g = Graph()
    y = g.conv2d(g.input(x.shape), w, np.zeros(1, np.int32), [2003370132], [39], pad=(1, 1, 1, 1), input_zp=-128,
                 out_zp=-128, clamp=(-128, 127))
    g.output(y)
    _check(device, g, [x])
    g = Graph()
    y = g.conv2d(g.input(x.shape), w, np.array([77], np.int32), [2003370132], [37], pad=(1, 1, 1, 1), input_zp=-128,
                 out_zp=-10, clamp=(-10, 90))
    g.output(y)
    _check(device, g, [x])


DW_CASES = [
    ((1, 56, 56, 11), (5, 5), 1, (1, 1), (2, 2, 2, 2), -128),   # tosa_ops/dw_peeling.mlir shape
    ((2, 9, 8, 8), (3, 3), 1, (2, 2), (0, 1, 0, 1), 4),
    ((1, 7, 7, 3), (3, 3), 2, (1, 1), (1, 1, 1, 1), -1),
    ((1, 12, 12, 4), (4, 4), 1, (2, 2), (1, 1, 1, 1), 0),       # dw_4x4_stride2 class
    ((1, 23, 23, 16), (21, 21), 1, (2, 2), (10, 10, 10, 10), 6),  # dw_21x21_odd_frame_stride2 class
    ((2, 28, 28, 192), (3, 3), 1, (1, 1), (1, 1, 1, 1), -7),
    ((2, 28, 28, 144), (3, 3), 1, (2, 2), (0, 1, 0, 1), 10),
    # C % 16 == 0: the cooperative-tile 3x3 kernel in each of its block shapes (16..128 channels per block),
    # widths below, at and beyond a tile, odd frames, stride 2 with either padding style
    ((3, 14, 14, 64), (3, 3), 1, (1, 1), (1, 1, 1, 1), 5),
    ((2, 7, 7, 960), (3, 3), 1, (1, 1), (1, 1, 1, 1), -3),
    ((1, 15, 17, 48), (3, 3), 1, (2, 2), (0, 1, 0, 1), 9),
    ((2, 112, 112, 32), (3, 3), 1, (1, 1), (1, 1, 1, 1), -128),
    ((1, 33, 130, 16), (3, 3), 1, (1, 1), (1, 1, 1, 1), 127),
    ((1, 33, 131, 128), (3, 3), 1, (2, 2), (1, 1, 1, 1), 0),
    ((1, 10, 300, 32), (3, 3), 1, (2, 2), (0, 1, 0, 1), -20),
]


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("case", DW_CASES)
def test_depthwise(device, case, mode):
    shape, k, M, stride, pad, izp = case
    rng = np.random.default_rng(1234)
    x = rng.integers(-128, 128, shape, dtype=np.int8)
    w = rng.integers(-127, 128, k + (shape[3], M), dtype=np.int8)
    OC = shape[3] * M
    bias = np.round(rng.normal(0, 1000, OC)).astype(np.int32)
    m, s = quantize_multipliers(rng.uniform(0.5, 1.5, OC) * 40.0 / (np.sqrt(k[0] * k[1]) * 74 * 74))
    g = Graph()
    y = g.depthwise_conv2d(g.input(shape), w, bias, m, s, stride=stride, pad=pad, input_zp=izp, out_zp=28,
                           requant_mode=mode)
    g.output(y)
    _check(device, g, [x])


@pytest.mark.parametrize("M,K,N,azp", [(1, 512, 512, 0), (64, 512, 512, -7), (512, 1024, 1024, 0), (5, 40, 9, -7),
                                       (33, 100, 130, 3), (256, 1280, 1000, -2),
                                       # the large corners of the FC sweep (M up to 4096, K = N up to 8192)
                                       (64, 4096, 4096, -7), (1, 8192, 8192, 0), (512, 8192, 8192, -7), (4096, 4096, 4096, 0)])
def test_fully_connected(device, M, K, N, azp):
    rng = np.random.default_rng(1234)
    a = rng.integers(-128, 128, (M, K), dtype=np.int8)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    bias = np.round(rng.normal(0, 1000, N)).astype(np.int32)
    m, s = quantize_multipliers(rng.uniform(0.5, 1.5, N) * 40.0 / (np.sqrt(K) * 74 * 74))
    g = Graph()
    y = g.fully_connected(g.input((M, K)), w, bias, m, s, input_zp=azp, out_zp=-3)
    g.output(y)
    _check(device, g, [a])


@pytest.mark.parametrize("M,K,N", [(1, 16, 8), (2, 1280, 1000), (3, 4096, 1031), (4, 12288, 520), (4, 64, 4096)])
@pytest.mark.parametrize("double_round", [True, False])
@pytest.mark.parametrize("with_table", [False, True])
def test_fully_connected_few_rows(device, M, K, N, double_round, with_table):
    """At most four rows take the weight-streaming kernel (one warp per output channel): every row count, the largest K
    it accepts, N not a multiple of the 8 channels of a block, both roundings, a clamp inside int8, shifts below 32 on
    some channels, and a table behind it."""
    rng = np.random.default_rng(M * 7 + K)
    a = rng.integers(-128, 128, (M, K), dtype=np.int8)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    bias = np.round(rng.normal(0, 1000, N)).astype(np.int32)
    m, s = quantize_multipliers(rng.uniform(0.5, 1.5, N) * 40.0 / (np.sqrt(K) * 74 * 74))
    if K == 1280:  # low shifts: the general 64-bit form of the rescale
        m, s = quantize_multipliers(rng.uniform(0.5, 1.5, N) * 40.0 / (np.sqrt(K) * 74 * 74))
        m = (m >> 8).astype(np.int32); s = (s - 8).astype(np.int32)
    g = Graph()
    y = g.fully_connected(g.input((M, K)), w, bias, m, s, input_zp=5, out_zp=-3, clamp=(-100, 90),
                          double_round=double_round)
    if with_table:
        y = g.table(y, rng.integers(-128, 128, 256, dtype=np.int8))
    g.output(y)
    _check(device, g, [a])
    from torq_b200.runtime import Executable
    ex = Executable(device, g.serialize())
    assert ex.op_kernels()[0] == "fc_rows_dp4a", ex.op_kernels()
    ex.destroy()


@pytest.mark.parametrize("kn", [512, 1024, 4096, 8192])
@pytest.mark.parametrize("M", [1, 64, 512, 4096])
@pytest.mark.parametrize("azp", [0, -7])
def test_fully_connected_sweep_at_full_size(device, M, kn, azp):
    """All 32 points of the FullyConnected sweep (M x K = N, both activation zero points) at their full sizes. The whole
    result of the largest corner would cost the CPU oracle minutes, so the check is on a sample that does not depend
    on the size: 4096 seeded output positions (every row class and column tile is hit), each recomputed as an exact
    int64 dot product and passed through the numpy restatement of the rescale; plus whole rows 0 and M - 1."""
    from oracle import oracle_np as onp
    rng = np.random.default_rng(kn + M)
    a = rng.integers(-128, 128, (M, kn), dtype=np.int8)
    w = rng.integers(-127, 128, (kn, kn), dtype=np.int8)
    bias = np.round(rng.normal(0, 1000, kn)).astype(np.int32)
    m, s = quantize_multipliers(rng.uniform(0.5, 1.5, kn) * 40.0 / (np.sqrt(kn) * 74 * 74))
    g = Graph()
    g.output(g.fully_connected(g.input((M, kn)), w, bias, m, s, input_zp=azp, out_zp=-3))
    got = run_graph_gpu(device, g, [a])[0]
    rows = np.concatenate([rng.integers(0, M, 4096), np.zeros(kn, np.int64), np.full(kn, M - 1)])
    cols = np.concatenate([rng.integers(0, kn, 4096), np.arange(kn), np.arange(kn)])
    want = np.empty(rows.size, np.int8)
    for lo in range(0, rows.size, 1024):  # chunks keep the gathered int64 operands small
        r, c = rows[lo:lo + 1024], cols[lo:lo + 1024]
        acc = ((a[r].astype(np.int64) - azp) * w[c].astype(np.int64)).sum(1) + bias[c]
        want[lo:lo + 1024] = [onp.requant(onp.wrap32(np.array([v])), m[j:j + 1], s[j:j + 1], -3, -128, 127)[0]
                              for v, j in zip(acc, c)]
    assert (got[rows, cols] == want).all(), int((got[rows, cols] != want).sum())
    assert len(np.unique(got[rows, cols])) > 50


def test_pools_and_table_at_benchmark_size(device):
    """The pooling and table configurations at their full sizes: max / average pool 3x3 stride 2 on 64x112x112x64 and
    the 256-entry table on 64x56x56x256, whole tensors against the oracle (the C restatement takes a second or two)."""
    rng = np.random.default_rng(77)
    x = rng.integers(-128, 128, (64, 112, 112, 64), dtype=np.int8)
    g = Graph()
    xi = g.input(x.shape)
    g.output(g.maxpool2d(xi, (3, 3), (2, 2), (0, 1, 0, 1)))
    g.output(g.avg_pool2d(xi, (3, 3), (2, 2), (0, 1, 0, 1), input_zp=-5, output_zp=3))
    _check(device, g, [x])
    t = rng.integers(-128, 128, (64, 56, 56, 256), dtype=np.int8)
    table = rng.integers(-128, 128, 256).astype(np.int8)
    g = Graph()
    g.output(g.table(g.input(t.shape), table))
    _check(device, g, [t])


def test_matmul_int32(device):
    rng = np.random.default_rng(1234)
    a = rng.integers(-128, 128, (17, 70), dtype=np.int8)
    b = rng.integers(-128, 128, (70, 13), dtype=np.int8)
    g = Graph()
    g.output(g.matmul_i32(g.input(a.shape), b, a_zp=-7, b_zp=2))
    _check(device, g, [a])


@pytest.mark.parametrize("shape,kernel,stride,pad", [
    ((2, 112, 112, 64), (3, 3), (2, 2), (0, 1, 0, 1)),   # maxpool2d-stride2-k3x3-pad-112x112x64.mlir
    ((1, 20, 20, 48), (5, 5), (1, 1), (2, 2, 2, 2)),     # SPPF window
    ((2, 11, 12, 6), (2, 2), (2, 2), (0, 0, 0, 0)),
    ((1, 7, 7, 128), (7, 7), (1, 1), (0, 0, 0, 0)),      # avgpool2d.mlir (global)
])
def test_pools(device, shape, kernel, stride, pad):
    rng = np.random.default_rng(1234)
    x = rng.integers(-128, 128, shape, dtype=np.int8)
    g = Graph()
    g.output(g.maxpool2d(g.input(shape), kernel, stride, pad, pad_value=-100))
    _check(device, g, [x])
    g = Graph()
    g.output(g.avg_pool2d(g.input(shape), kernel, stride, pad, input_zp=4, output_zp=-3))
    _check(device, g, [x])


@pytest.mark.parametrize("shape", [(1, 56, 56, 24), (3, 7, 5, 3), (2, 28, 28, 32)])
def test_add_sub_mul(device, shape):
    rng = np.random.default_rng(1234)
    a = rng.integers(-128, 128, shape, dtype=np.int8)
    b = rng.integers(-128, 128, shape, dtype=np.int8)
    for kind in ("add", "sub"):
        g = Graph()
        fn = getattr(g, kind)
        # constants of tests/testdata/tosa_ops/add-single-rescale.mlir: shift 49 takes the double-round branch
        g.output(fn(g.input(shape), g.input(shape), a_zp=-3, a_ms=(1 << 30, 11), b_zp=5, b_ms=(1 << 30, 11),
                    out_ms=(1093202297, 49), out_zp=-2))
        _check(device, g, [a, b])
        # two-stage input rescale (left shift 20, then a 32-bit multiplier with shift 32: the double-round branch
        # on the input side), the form of tests/testdata/tosa_ops/add-56x56x256.mlir with other constants
        g = Graph()
        fn = getattr(g, kind)
        g.output(fn(g.input(shape), g.input(shape), a_zp=-60, a_ms=(1400000001, 32), a_lshift=20, b_zp=9, b_ms=(1 << 30, 11),
                    out_ms=(1090000000, 48), out_zp=-128))
        _check(device, g, [a, b])
    g = Graph()
    g.output(g.mul(g.input(shape), g.input(shape), a_zp=3, a_ms=(1 << 30, 30), b_zp=-4, b_ms=(1 << 30, 30),
                   out_ms=quantize_multiplier(1.0 / 150), out_zp=1, clamp=(-100, 100)))
    _check(device, g, [a, b])


def test_table_rescale_resize_concat(device):
    rng = np.random.default_rng(1234)
    shape = (2, 13, 9, 20)
    x = rng.integers(-128, 128, shape, dtype=np.int8)
    # sigmoid table from seeded scales
    s_in, zp_in, s_out, zp_out = 0.05, -3, 1.0 / 256, -128
    idx = np.arange(-128, 128)
    tbl = np.clip(np.round(1.0 / (1.0 + np.exp(-s_in * (idx - zp_in))) / s_out) + zp_out, -128, 127).astype(np.int8)
    g = Graph()
    g.output(g.table(g.input(shape), tbl))
    _check(device, g, [x])

    m, s = quantize_multipliers(rng.uniform(0.3, 1.9, 20))
    g = Graph()
    g.output(g.rescale(g.input(shape), m, s, input_zp=5, out_zp=3))
    _check(device, g, [x])
    g = Graph()
    g.output(g.rescale(g.input(shape), [1518500250], [30], input_zp=-7, out_zp=0, clamp=(-50, 50)))
    _check(device, g, [x])

    g = Graph()
    g.output(g.resize_nearest_2x(g.input(shape)))
    _check(device, g, [x])

    z = rng.integers(-128, 128, (2, 13, 9, 12), dtype=np.int8)
    g = Graph()
    g.output(g.concat(g.input(shape), g.input(z.shape), a_zp=3, a_ms=(1500000000, 31), b_zp=-5,
                      b_ms=(1200000000, 30), out_zp=7))
    _check(device, g, [x, z])


def test_chain_with_intermediates_and_host_call(device):
    """conv -> depthwise -> conv + residual add: exercises the arena and tb200_invoke_host."""
    rng = np.random.default_rng(1234)
    shape = (2, 14, 14, 16)
    x = rng.integers(-128, 128, shape, dtype=np.int8)
    g = Graph()
    xin = g.input(shape)
    m, s = quantize_multipliers(rng.uniform(0.5, 1.5, 96) * 40.0 / (4 * 74 * 74))
    h = g.conv2d(xin, rng.integers(-127, 128, (96, 1, 1, 16), dtype=np.int8), np.zeros(96, np.int32), m, s,
                 input_zp=2, out_zp=-128, clamp=(-128, 127))
    m, s = quantize_multipliers(rng.uniform(0.5, 1.5, 96) * 40.0 / (3 * 74 * 74))
    h = g.depthwise_conv2d(h, rng.integers(-127, 128, (3, 3, 96, 1), dtype=np.int8), np.zeros(96, np.int32), m, s,
                           pad=(1, 1, 1, 1), input_zp=-128, out_zp=-128)
    m, s = quantize_multipliers(rng.uniform(0.5, 1.5, 16) * 40.0 / (10 * 74 * 74))
    h = g.conv2d(h, rng.integers(-127, 128, (16, 1, 1, 96), dtype=np.int8), np.zeros(16, np.int32), m, s,
                 input_zp=-128, out_zp=4)
    y = g.add(xin, h, a_zp=2, a_ms=(1 << 30, 11), b_zp=4, b_ms=(1 << 30, 11), out_ms=(1093202297, 49), out_zp=-2)
    g.output(y)
    _check(device, g, [x])
    _check(device, g, [x], host_call=True)


@pytest.mark.parametrize("shape,OC,conv_first,double_round", [
    ((2, 28, 28, 96), 32, True, True),      # the residual connection of an inverted-residual block
    ((2, 28, 28, 96), 32, False, True),     # the convolution's result as the add's second operand
    ((1, 56, 56, 48), 24, True, True),      # 24 channels: grouped rows
    ((3, 14, 14, 64), 64, True, False),     # single rounding: the record without the sign term
    ((1, 9, 7, 160), 80, False, True),      # ragged last tile
])
def test_pointwise_conv_with_fused_residual_add(device, shape, OC, conv_first, double_round):
    """With TB200_ADD_FUSION=1 a rescaled add whose one operand is the only use of a 1x1 convolution's result runs in
    that convolution's epilogue (one launch, the product never stored): bit-exact against the oracle, which runs the
    two ops apart, and against the default plan (two launches); a product with a second reader keeps its own launch."""
    import os
    from torq_b200.runtime import Executable
    rng = np.random.default_rng(shape[1] * 31 + OC)
    x = rng.integers(-128, 128, shape, dtype=np.int8)
    r = rng.integers(-128, 128, shape[:3] + (OC,), dtype=np.int8)
    w = rng.integers(-127, 128, (OC, 1, 1, shape[3]), dtype=np.int8)
    m, s = quantize_multipliers(rng.uniform(0.5, 1.5, OC) * 40.0 / (np.sqrt(shape[3]) * 74 * 74))

    def build(second_reader):
        g = Graph()
        xi, ri = g.input(shape), g.input(r.shape)
        h = g.conv2d(xi, w, np.round(rng.normal(0, 500, OC)).astype(np.int32) * 0 + 77, m, s, input_zp=-5, out_zp=4)
        kw = dict(a_zp=4 if conv_first else -2, a_ms=(1 << 30, 11), b_zp=-2 if conv_first else 4, b_ms=(1395864371, 12),
                  out_ms=(1093202297, 49), out_zp=-3, clamp=(-110, 120), double_round=double_round)
        y = g.add(h, ri, **kw) if conv_first else g.add(ri, h, **kw)
        g.output(y)
        if second_reader:
            g.output(g.table(h, np.arange(-128, 128, dtype=np.int8)[::-1].copy()))
        return g

    g = build(False)
    apart = _check(device, g, [x, r])[0]
    ex = Executable(device, g.serialize())
    assert ex.op_kernels() == ["gemm_i8_tcgen05", "binary_rescale"]
    ex.destroy()
    os.environ["TB200_ADD_FUSION"] = "1"
    try:
        ex = Executable(device, g.serialize())
        assert ex.op_kernels() == ["gemm_i8_tcgen05", "(add in the convolution's epilogue)"] and ex.launch_count == 1, ex.op_kernels()
        ex.destroy()
        got = _check(device, g, [x, r])[0]
        assert (apart == got).all()
        g2 = build(True)
        _check(device, g2, [x, r])
        ex = Executable(device, g2.serialize())
        assert "binary_rescale" in ex.op_kernels()
        ex.destroy()
    finally:
        del os.environ["TB200_ADD_FUSION"]


GEMM_CASES = [
    # M, K, N : the tensor-core path (K % 16 == 0); tails in M, N and K all appear
    (1, 16, 16), (127, 16, 24), (128, 32, 192), (129, 48, 16), (300, 144, 24), (1000, 160, 960), (513, 960, 320),
    (256, 320, 1280), (77, 1280, 1000), (4096, 64, 384), (2 * 56 * 56, 24 * 6, 24), (640, 576, 96), (64, 4096, 512),
    # K not a multiple of 16: r rows are read as one (block-diagonal weights)
    (2 * 56 * 56, 24, 144), (64, 40, 9), (256, 100, 130), (10, 8, 5), (1000, 24, 24),
]


@pytest.mark.parametrize("M,K,N", GEMM_CASES)
def test_pointwise_conv_tensor_core_sweep(device, M, K, N):
    """1x1 convolution = row-major GEMM; checked against the oracle and, for the same blob,
    against the CUDA-core kernel (TB200_FORCE_SIMT=1)."""
    import os
    rng = np.random.default_rng(1234 + M + K + N)
    a = rng.integers(-128, 128, (1, 1, M, K), dtype=np.int8)
    w = rng.integers(-127, 128, (N, 1, 1, K), dtype=np.int8)
    bias = np.round(rng.normal(0, 1000, N)).astype(np.int32)
    m, s = quantize_multipliers(rng.uniform(0.5, 1.5, N) * 40.0 / (np.sqrt(K) * 74 * 74))
    g = Graph()
    y = g.conv2d(g.input(a.shape), w, bias, m, s, input_zp=-6, out_zp=4, clamp=(-120, 115))
    g.output(y)
    got = _check(device, g, [a])[0]
    from torq_b200.runtime import Executable
    ex = Executable(device, g.serialize())
    assert ex.op_kernels() == ["gemm_i8_tcgen05" if M > 4 or K % 16 else "fc_rows_dp4a"]
    ex.destroy()
    os.environ["TB200_FORCE_SIMT"] = "1"
    try:
        ex = Executable(device, g.serialize())
        assert ex.op_kernels()[0] in ("conv2d_simt", "conv2d_c16_dp4a")  # CUDA-core kernels
        ex.destroy()
        simt = run_graph_gpu(device, g, [a])[0]
    finally:
        del os.environ["TB200_FORCE_SIMT"]
    assert (simt == got).all()


def test_pipelined_host_calls(device):
    """tb200_invoke_host_async: three calls in flight over the two staging sets, one wait at the end."""
    from torq_b200.runtime import Executable
    rng = np.random.default_rng(1234)
    shape = (4, 28, 28, 32)
    g = Graph()
    m, s = quantize_multipliers(rng.uniform(0.5, 1.5, 64) * 40.0 / (np.sqrt(32) * 74 * 74))
    y = g.conv2d(g.input(shape), rng.integers(-127, 128, (64, 1, 1, 32), dtype=np.int8),
                 np.round(rng.normal(0, 1000, 64)).astype(np.int32), m, s, input_zp=3, out_zp=-1)
    g.output(y)
    xs = [rng.integers(-128, 128, shape, dtype=np.int8) for _ in range(3)]
    outs = [np.zeros((4, 28, 28, 64), np.int8) for _ in range(3)]
    ex = Executable(device, g.serialize())
    for x, o in zip(xs, outs):
        ex.invoke_host_async([x], [o])
    device.wait()
    for x, o in zip(xs, outs):
        assert (o == run_graph(g, [x])[0]).all()
    ex.destroy()


def test_chained_concats_are_written_in_place(device):
    """concat(concat(a, b), c) with a pass-through rescale on the inner result: the planner writes the inner
    result straight into the outer one (one launch less); a non-identity rescale keeps the copy."""
    from torq_b200.runtime import Executable
    rng = np.random.default_rng(1234)
    shape = (2, 9, 7, 16)
    xs = [rng.integers(-128, 128, shape, dtype=np.int8) for _ in range(4)]
    ident = ((1 << 30), 30)
    for passthrough, want_launches in ((True, 4), (False, 6)):
        g = Graph()
        ins = [g.input(shape) for _ in range(4)]
        acc = g.concat(ins[0], ins[1], a_zp=3, a_ms=quantize_multiplier(0.7), b_zp=-2, b_ms=quantize_multiplier(1.3), out_zp=4)
        mid = ident if passthrough else quantize_multiplier(0.9)
        acc = g.concat(acc, ins[2], a_zp=4, a_ms=mid, b_zp=0, b_ms=quantize_multiplier(0.5), out_zp=4)
        acc = g.concat(acc, ins[3], a_zp=4, a_ms=mid, b_zp=7, b_ms=quantize_multiplier(1.1), out_zp=4)
        g.output(g.table(acc, np.arange(-128, 128, dtype=np.int8)[::-1].copy()))  # a consumer of the final result
        ex = Executable(device, g.serialize())
        assert ex.launch_count == want_launches + 1
        ex.destroy()
        _check(device, g, xs)


@pytest.mark.parametrize("shape,OC,k,dil", [((1, 12, 12, 64), 32, 1, 1),    # 1x1: tensor-core GEMM
                                            ((2, 14, 14, 32), 48, 3, 1),    # 3x3: tensor-core implicit GEMM
                                            ((1, 18, 18, 16), 20, 3, 1),    # 16 channels: direct dp4a kernel
                                            ((1, 20, 20, 3), 16, 3, 1),     # stem kernel
                                            ((1, 11, 11, 24), 10, 3, 2)])   # dilation: generic CUDA-core kernel
def test_table_fused_into_conv_epilogue(device, shape, OC, k, dil):
    """conv -> table (SiLU as a 256-entry table follows every convolution of the detector): when the table is
    the convolution's only reader it runs in the convolution's epilogue; same bytes as the two-kernel form."""
    import os
    from torq_b200.runtime import Executable
    rng = np.random.default_rng(1234)
    x = rng.integers(-128, 128, shape, dtype=np.int8)
    w = rng.integers(-127, 128, (OC, k, k, shape[3]), dtype=np.int8)
    m, s = quantize_multipliers(rng.uniform(0.5, 1.5, OC) * 40.0 / (np.sqrt(k * k * shape[3]) * 74 * 74))
    table = rng.integers(-128, 128, 256, dtype=np.int8)
    p = dil * (k - 1) // 2
    g = Graph()
    y = g.conv2d(g.input(shape), w, np.round(rng.normal(0, 2000, OC)).astype(np.int32), m, s, dilation=(dil, dil),
                 pad=(p, p, p, p), input_zp=-4, out_zp=3)
    g.output(g.table(y, table))
    ex = Executable(device, g.serialize())
    assert ex.launch_count == 1, ex.op_kernels()
    ex.destroy()
    fused = _check(device, g, [x])[0]
    os.environ["TB200_NO_TABLE_FUSION"] = "1"
    try:
        ex = Executable(device, g.serialize())
        assert ex.launch_count == 2
        ex.destroy()
        assert (run_graph_gpu(device, g, [x])[0] == fused).all()
    finally:
        del os.environ["TB200_NO_TABLE_FUSION"]
