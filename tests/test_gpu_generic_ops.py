"""The tensor ops outside the layer set on the GPU against the oracle (bit-exact for integers and for the exact
float ops) and, for softmax and float means, against torch fp32 within the bf16 tolerance of the decoder ops.
Shapes of the float cases are the reference's fixtures (tests/testdata/torch_ops/softmax-1x8x1x207xbf16.mlir,
reducemean.mlir: rows of 207 and 288 values)."""
import numpy as np
import pytest
import torch

from gpu_exec import run_graph_gpu
from oracle_exec import run_graph
from torq_b200.bf16 import from_bf16, to_bf16
from torq_b200.oplist import EW_FN, Graph

pytestmark = pytest.mark.gpu
NP = {"i8": np.int8, "i16": np.int16, "i32": np.int32}


def _same(device, g, inputs):
    want = run_graph(g, inputs)
    got = run_graph_gpu(device, g, inputs)
    for w, o in zip(want, got):
        assert w.shape == o.shape and w.dtype == o.dtype
        assert (w.view(np.uint8) == o.view(np.uint8)).all(), f"{(w != o).sum()} of {w.size} differ"
    return got


@pytest.mark.parametrize("fn", [f for f, code in EW_FN.items() if code >= 16])
@pytest.mark.parametrize("dtype", ["i8", "i16", "i32"])
def test_binary_integer_ops_with_broadcast(device, fn, dtype):
    if fn.startswith("logical_") and fn not in ("logical_left_shift",) and dtype != "i8":
        pytest.skip("boolean ops live on i8 tensors")
    rng = np.random.default_rng(EW_FN[fn] * 7 + len(dtype))
    lim = {"i8": 128, "i16": 30000, "i32": 2 ** 31 - 1}[dtype]
    a = rng.integers(-lim, lim, (3, 5, 7, 33)).astype(NP[dtype])
    b = rng.integers(-lim, lim, (1, 5, 1, 33)).astype(NP[dtype])
    arg = 0
    if fn in ("logical_left_shift", "arithmetic_right_shift"):
        b = rng.integers(0, 31, b.shape).astype(NP[dtype])
        arg = 1
    if fn == "mul" and dtype == "i32":
        arg = 31
    if fn.startswith("logical_") and fn != "logical_left_shift":
        a, b = (a > 0).astype(np.int8), (b > 0).astype(np.int8)
    if fn in ("equal", "greater_equal"):
        a[:, :, ::2, :] = b[:, :, :, :]  # ties on half of the rows
    out_dtype = "i8" if fn in ("equal", "greater", "greater_equal") or (fn.startswith("logical_") and fn != "logical_left_shift") else \
        ("i32" if fn == "mul" else dtype)
    g = Graph()
    g.output(g.ew(fn, g.input(a.shape, dtype), g.input(b.shape, dtype), out_dtype=out_dtype, arg=arg))
    got = _same(device, g, [a, b])
    assert len(np.unique(got[0])) > 1


@pytest.mark.parametrize("fn", ["abs", "negate", "bitwise_not", "clz", "clamp", "logical_not"])
def test_unary_integer_ops(device, fn):
    rng = np.random.default_rng(11)
    x = rng.integers(-2 ** 31, 2 ** 31 - 1, (4, 1001)).astype(np.int32)
    x[0, :4] = [0, -1, -2 ** 31, 2 ** 31 - 1]
    g = Graph()
    g.output(g.ew(fn, g.input(x.shape, "i32"), in_zp=3, out_zp=-5, clamp=(-1000, 77777)))
    _same(device, g, [x])


@pytest.mark.parametrize("src,dst", [("i32", "i8"), ("i32", "i16"), ("i8", "i32"), ("i16", "i8"), ("f32", "i8"), ("f32", "i32"),
                                     ("bf16", "i16"), ("i32", "bf16"), ("i8", "f32"), ("bf16", "f32"), ("f32", "bf16")])
def test_casts(device, src, dst):
    rng = np.random.default_rng(5)
    if src in ("f32", "bf16"):
        v = rng.uniform(-70000, 70000, (7, 301)).astype(np.float32)
        v[0, :6] = [0.5, 1.5, 2.5, -0.5, -1.5, 3e9]
        x = to_bf16(v) if src == "bf16" else v
    else:
        x = rng.integers(-2 ** 31, 2 ** 31 - 1, (7, 301)).astype(NP[src])
    g = Graph()
    g.output(g.ew("cast", g.input(x.shape, src), out_dtype=dst))
    _same(device, g, [x])


@pytest.mark.parametrize("fn", ["add", "sub", "mul", "maximum", "minimum", "equal", "greater", "greater_equal"])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_float_elementwise_is_exact(device, fn, dtype):
    rng = np.random.default_rng(9)
    a = rng.uniform(-40, 40, (2, 9, 129)).astype(np.float32)
    b = rng.uniform(-40, 40, (2, 1, 129)).astype(np.float32)
    if dtype == "bf16":
        a, b = to_bf16(a), to_bf16(b)
    out_dtype = "i8" if fn in ("equal", "greater", "greater_equal") else dtype
    g = Graph()
    g.output(g.ew(fn, g.input(a.shape, dtype), g.input(b.shape, dtype), out_dtype=out_dtype))
    _same(device, g, [a, b])


@pytest.mark.parametrize("in_dtype,out_dtype,unsigned", [("i32", "i8", (False, False)), ("i16", "i32", (False, False)),
                                                         ("i8", "i16", (False, False)), ("i32", "i32", (False, False)),
                                                         ("i8", "i8", (True, False)), ("i8", "i8", (False, True)),
                                                         ("i32", "i16", (False, False))])
@pytest.mark.parametrize("per_channel", [False, True])
def test_generic_rescale(device, in_dtype, out_dtype, unsigned, per_channel):
    rng = np.random.default_rng(21)
    C = 19
    lim = {"i8": 128, "i16": 20000, "i32": 3000000}[in_dtype]
    x = rng.integers(-lim, lim, (2, 6, 5, C)).astype(NP[in_dtype])
    n = C if per_channel else 1
    mult = rng.integers(1 << 30, (1 << 31) - 1, n).astype(np.int32)
    lo, hi = {"i8": (28, 34), "i16": (36, 42), "i32": (44, 48)}[in_dtype]
    shift = rng.integers(lo, hi, n).astype(np.int8)
    g = Graph()
    g.output(g.rescale(g.input(x.shape, in_dtype), mult, shift, input_zp=-3 if not unsigned[0] else 128, out_zp=7,
                       out_dtype=out_dtype, input_unsigned=unsigned[0], output_unsigned=unsigned[1]))
    got = _same(device, g, [x])
    assert len(np.unique(got[0])) > 2


def test_layout_ops(device):
    rng = np.random.default_rng(3)
    x = rng.integers(-128, 128, (3, 10, 7, 24)).astype(np.int8)
    h = rng.integers(-30000, 30000, (5, 33, 17)).astype(np.int16)
    w = rng.integers(-2 ** 31, 2 ** 31 - 1, (64, 96)).astype(np.int32)
    g = Graph()
    xi, hi, wi = g.input(x.shape), g.input(h.shape, "i16"), g.input(w.shape, "i32")
    g.output(g.transpose(xi, [0, 3, 1, 2]))
    g.output(g.transpose(hi, [2, 0, 1]))
    g.output(g.transpose(wi, [1, 0]))
    g.output(g.slice(xi, [1, 2, 3, 4], [2, 5, 3, 16]))
    g.output(g.pad(xi, [0, 1, 2, 0], [0, 3, 0, 5], value=-77))
    g.output(g.concat_axis(xi, g.slice(xi, [0, 0, 0, 0], [3, 4, 7, 24]), 1))
    g.output(g.concat_axis(hi, hi, 2))
    _same(device, g, [x, h, w])


def test_layout_ops_in_16_byte_pieces(device):
    """Extents, offsets and strides that let the copy move 16 (8, 4) bytes per index; padding repeats the element."""
    rng = np.random.default_rng(13)
    x = rng.integers(-128, 128, (2, 9, 6, 64)).astype(np.int8)
    h = rng.integers(-30000, 30000, (4, 10, 24)).astype(np.int16)
    w = rng.integers(-2 ** 31, 2 ** 31 - 1, (6, 5, 12)).astype(np.int32)
    g = Graph()
    xi, hi, wi = g.input(x.shape), g.input(h.shape, "i16"), g.input(w.shape, "i32")
    g.output(g.slice(xi, [0, 2, 1, 16], [2, 5, 4, 32]))
    g.output(g.pad(xi, [0, 1, 1, 16], [0, 2, 0, 48], value=-9))
    g.output(g.concat_axis(xi, xi, 3))
    g.output(g.concat_axis(xi, g.slice(xi, [0, 0, 0, 0], [2, 4, 6, 64]), 1))
    g.output(g.slice(hi, [1, 3, 8], [2, 6, 16]))
    g.output(g.pad(hi, [0, 0, 4], [1, 0, 4], value=-12345))     # 8-byte pieces
    g.output(g.pad(wi, [1, 0, 4], [0, 2, 8], value=-2 ** 31))
    g.output(g.transpose(xi, [0, 2, 1, 3]))                     # the channel axis stays innermost
    _same(device, g, [x, h, w])


@pytest.mark.parametrize("fn", ["sum", "max", "min", "argmax"])
@pytest.mark.parametrize("axis", [0, 1, 2])
def test_integer_reductions(device, fn, axis):
    rng = np.random.default_rng(17)
    x = rng.integers(-2 ** 30, 2 ** 30, (6, 37, 50)).astype(np.int32)
    g = Graph()
    g.output(g.reduce(fn, g.input(x.shape, "i32"), axis, keep_axis=fn != "argmax"))
    _same(device, g, [x])


def test_table16(device):
    rng = np.random.default_rng(8)
    x = rng.integers(-32768, 32768, (3, 4001)).astype(np.int16)
    x[0, :4] = [-32768, 32767, 0, -1]
    table = np.sort(rng.integers(-32768, 32767, 513)).astype(np.int16)
    g = Graph()
    g.output(g.table16(g.input(x.shape, "i16"), table))
    _same(device, g, [x])


@pytest.mark.parametrize("shape", [(1, 8, 1, 207), (1, 1000), (64, 1152)])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_softmax_against_torch(device, shape, dtype):
    rng = np.random.default_rng(2)
    v = rng.normal(0, 3, shape).astype(np.float32)
    x = to_bf16(v) if dtype == "bf16" else v
    g = Graph()
    g.output(g.softmax(g.input(shape, dtype)))
    got = run_graph_gpu(device, g, [x])[0]
    ref = torch.softmax(torch.from_numpy(from_bf16(x) if dtype == "bf16" else x), -1).numpy()
    got_f = from_bf16(got) if dtype == "bf16" else got
    # tolerance of the floating-point class: 2 bf16 ulp of the value (bf16), 1e-5 relative (f32), rows sum to one
    tol = 2.0 ** -7 if dtype == "bf16" else 1e-5
    assert np.all(np.abs(got_f - ref) <= tol * np.maximum(ref, 1e-3))
    assert np.allclose(got_f.sum(-1), 1.0, atol=2e-2 if dtype == "bf16" else 1e-5)


@pytest.mark.parametrize("fn", ["mean", "sum", "max"])
def test_float_reductions(device, fn):
    """Sums and means add in fp32 in index order on both sides, so they are bit-exact against the oracle; against
    torch (pairwise sums) they agree to fp32 rounding."""
    rng = np.random.default_rng(4)
    v = rng.normal(0, 1, (1, 207, 288)).astype(np.float32)
    x = to_bf16(v)
    g = Graph()
    g.output(g.reduce(fn, g.input(x.shape, "bf16"), 2))
    got = _same(device, g, [x])[0]
    t = torch.from_numpy(from_bf16(x))
    ref = {"mean": t.mean(-1, keepdim=True), "sum": t.sum(-1, keepdim=True), "max": t.max(-1, keepdim=True).values}[fn].numpy()
    assert np.all(np.abs(from_bf16(got) - ref) <= 2.0 ** -7 * np.maximum(np.abs(ref), 1e-2))


@pytest.mark.parametrize("shape,oc,k,stride,dil,pad", [((1, 64, 64, 1), 1, 3, 2, 1, (0, 1, 0, 1)), ((2, 17, 13, 5), 7, 3, 1, 1, (1, 1, 1, 1)),
                                                        ((1, 20, 20, 70), 4, 5, 2, 2, (3, 2, 2, 3)), ((3, 9, 9, 16), 33, 1, 1, 1, (0, 0, 0, 0))])
@pytest.mark.parametrize("per_channel", [False, True])
def test_conv2d_int16_activations(device, shape, oc, k, stride, dil, pad, per_channel):
    """Conv2D i16 x i8 with the 16-bit rescale (first case: the shape of the reference's gen_ops/conv2d_64x64_i16.mlir)."""
    rng = np.random.default_rng(oc * 31 + k)
    x = rng.integers(-32768, 32768, shape).astype(np.int16)
    w = rng.integers(-128, 128, (oc, k, k, shape[3])).astype(np.int8)
    bias = rng.integers(-2 ** 33, 2 ** 33, oc).astype(np.int64)   # beyond 32 bits: the accumulator is 64 bits wide
    n = oc if per_channel else 1
    mult = rng.integers(1 << 14, 1 << 15, n)
    base = int(np.ceil(np.log2(2 ** 33 * 23000 / 12000)))          # results spread over the int16 range, some saturate
    shift = rng.integers(base, base + 2, n)
    g = Graph()
    g.output(g.conv2d_i16(g.input(shape, "i16"), w, bias if per_channel else bias[:1], mult, shift, stride=(stride, stride),
                          dilation=(dil, dil), pad=pad, input_zp=0, weight_zp=0, out_zp=-11))
    got = _same(device, g, [x])
    assert len(np.unique(got[0])) > 16


@pytest.mark.parametrize("dtype", ["i8", "i16", "i32"])
def test_gather_and_scatter(device, dtype):
    rng = np.random.default_rng(6)
    N, K, C, W = 3, 50, 7, 12
    values = rng.integers(-100, 100, (N, K, C)).astype(NP[dtype])
    idx = np.stack([rng.permutation(K)[:W] for _ in range(N)]).astype(np.int32)   # distinct per batch, as TOSA asks
    upd = rng.integers(-100, 100, (N, W, C)).astype(NP[dtype])
    g = Graph()
    v, i, u = g.input(values.shape, dtype), g.input(idx.shape, "i32"), g.input(upd.shape, dtype)
    g.output(g.gather(v, i))
    g.output(g.scatter(v, i, u))
    _same(device, g, [values, idx, upd])


@pytest.mark.parametrize("view,perm", [((2, 4, 4, 2, 2, 8), (0, 1, 3, 2, 4, 5)), ((1, 8, 8, 2, 2, 32), (0, 1, 3, 2, 4, 5)),
                                        ((1, 8, 8, 32, 2, 2), (0, 1, 4, 2, 5, 3)), ((3, 5, 2, 7, 4), (0, 3, 1, 4, 2)),
                                        ((2, 3, 4, 5, 6), (4, 3, 2, 1, 0))])
def test_permute_of_five_and_six_dimensions(device, view, perm):
    """Depth-to-space forms (block in the channel's high or low part) and general five-dimensional transposes, the last
    one a full reversal that no merging of neighbours shortens."""
    rng = np.random.default_rng(len(view))
    n = int(np.prod(view))
    x = rng.integers(-128, 128, n).astype(np.int8).reshape(-1, view[-1])
    g = Graph()
    out_shape = (int(np.prod([view[p] for p in perm[:-1]])), view[perm[-1]])
    g.output(g.permute(g.input(x.shape), view, perm, out_shape))
    _same(device, g, [x])


@pytest.mark.parametrize("fn", ["exp", "log", "reciprocal", "rsqrt", "tanh", "sigmoid", "erf"])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_float_functions_against_torch(device, fn, dtype):
    """Tolerance class: the function's last bits belong to the math library. f32 within 4 ulp-ish (4e-6 relative, 1e-7
    absolute near zero), bf16 within one ulp of the fp32 torch value rounded."""
    rng = np.random.default_rng(3)
    v = rng.uniform(0.05, 8.0, (3, 1001)).astype(np.float32) if fn in ("log", "rsqrt", "reciprocal") else \
        rng.uniform(-6.0, 6.0, (3, 1001)).astype(np.float32)
    x = to_bf16(v) if dtype == "bf16" else v
    g = Graph()
    g.output(g.ew(fn, g.input(x.shape, dtype)))
    got = run_graph_gpu(device, g, [x])[0]
    t = torch.from_numpy(from_bf16(x) if dtype == "bf16" else x)
    ref = {"exp": torch.exp, "log": torch.log, "reciprocal": torch.reciprocal, "rsqrt": torch.rsqrt, "tanh": torch.tanh,
           "sigmoid": torch.sigmoid, "erf": torch.erf}[fn](t).numpy()
    if dtype == "bf16":
        assert np.all(np.abs(from_bf16(got) - ref) <= 2.0 ** -7 * np.abs(ref) + 1e-30)
    else:
        assert np.all(np.abs(got - ref) <= 4e-6 * np.abs(ref) + 1e-7)


@pytest.mark.parametrize("M,K,N", [(64, 128, 256), (207, 36, 207), (2, 2, 2), (33, 70, 5)])
@pytest.mark.parametrize("dtype,out_dtype", [("bf16", "f32"), ("bf16", "bf16"), ("f32", "f32")])
def test_float_matmul(device, M, K, N, dtype, out_dtype):
    """fp32 products and sums, each rounded, in index order of k: bit-exact against the oracle, close to torch."""
    rng = np.random.default_rng(M + N)
    a = rng.normal(0, 1, (M, K)).astype(np.float32)
    b = rng.normal(0, 1, (K, N)).astype(np.float32)
    if dtype == "bf16":
        a, b = to_bf16(a), to_bf16(b)
    g = Graph()
    g.output(g.matmul_f(g.input(a.shape, dtype), g.input(b.shape, dtype), out_dtype))
    got = _same(device, g, [a, b])[0]
    fa, fb = (from_bf16(a), from_bf16(b)) if dtype == "bf16" else (a, b)
    ref = (torch.from_numpy(fa).double() @ torch.from_numpy(fb).double()).numpy()
    gf = from_bf16(got) if out_dtype == "bf16" else got
    tol = 2.0 ** -7 if out_dtype == "bf16" else 1e-5
    assert np.all(np.abs(gf - ref) <= tol * np.abs(ref) + 1e-4 * np.sqrt(K))


@pytest.mark.parametrize("shape,kernel,M,stride,dil,pad", [
    ((1, 16, 16, 2), (3, 3), 1, (1, 1), (1, 1), (1, 1, 1, 1)),     # the reference's dw_16x16-bf16 fixture shape
    ((2, 13, 17, 5), (5, 5), 1, (1, 1), (1, 1), (2, 2, 2, 2)),
    ((1, 20, 14, 8), (3, 3), 2, (2, 2), (1, 1), (0, 1, 0, 1)),     # stride 2, channel multiplier 2
    ((1, 12, 12, 3), (3, 2), 1, (1, 2), (2, 1), (2, 2, 0, 1)),     # dilation, asymmetric window
])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_float_depthwise(device, shape, kernel, M, stride, dil, pad, dtype):
    """tosa.depthwise_conv2d on floats: fp32 products and sums, each rounded, taps in (kh, kw) order, the bias last:
    bit-exact against the oracle, close to a float64 torch convolution."""
    rng = np.random.default_rng(shape[1] + kernel[0])
    C = shape[3]
    x = rng.normal(0, 1, shape).astype(np.float32)
    w = rng.normal(0, 1, kernel + (C, M)).astype(np.float32)
    bias = rng.normal(0, 1, (C * M,)).astype(np.float32)
    if dtype == "bf16":
        x, w, bias = to_bf16(x), to_bf16(w), to_bf16(bias)
    g = Graph()
    g.output(g.depthwise_conv2d_f(g.input(x.shape, dtype), g.const(w, dtype), g.const(bias, dtype), stride=stride, dilation=dil, pad=pad))
    got = _same(device, g, [x])[0]
    fx, fw, fb = (from_bf16(x), from_bf16(w), from_bf16(bias)) if dtype == "bf16" else (x, w, bias)
    xt = torch.nn.functional.pad(torch.from_numpy(fx).double().permute(0, 3, 1, 2), (pad[2], pad[3], pad[0], pad[1]))
    wt = torch.from_numpy(fw).double().permute(2, 3, 0, 1).reshape(C * M, 1, kernel[0], kernel[1])
    ref = torch.nn.functional.conv2d(xt, wt, torch.from_numpy(fb).double(), stride=stride, dilation=dil, groups=C).permute(0, 2, 3, 1).numpy()
    gf = from_bf16(got) if dtype == "bf16" else got
    tol = 2.0 ** -7 if dtype == "bf16" else 1e-5
    assert gf.shape == ref.shape and np.all(np.abs(gf - ref) <= tol * np.abs(ref) + 1e-4 * kernel[0] * kernel[1])
