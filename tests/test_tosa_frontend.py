"""The TOSA-text front end on modules written for this test (same textual forms as the
reference's fixtures: tosa.const / arith.constant, hex dense blobs, fused rescale chains)."""
import numpy as np
import pytest

from oracle_exec import run_graph
from torq_b200 import tosa_frontend

CONV = '''
module {
  func.func @main(%arg0: tensor<1x6x6x4xi8> {some.attr = "x"}) -> (tensor<1x6x6x2xi8> {other = "y"}) {
    %0 = "tosa.const"() <{values = dense<"0xWEIGHTHEX"> : tensor<2x3x3x4xi8>}> : () -> tensor<2x3x3x4xi8>
    %1 = "tosa.const"() <{values = dense<[100, -200]> : tensor<2xi32>}> : () -> tensor<2xi32>
    %cst = arith.constant dense<-3> : tensor<1xi8>
    %cst_0 = arith.constant dense<0> : tensor<1xi8>
    %2 = tosa.conv2d %arg0, %0, %1, %cst, %cst_0 {acc_type = i32, dilation = array<i64: 1, 1>, pad = array<i64: 1, 1, 1, 1>, stride = array<i64: 1, 1>} : (tensor<1x6x6x4xi8>, tensor<2x3x3x4xi8>, tensor<2xi32>, tensor<1xi8>, tensor<1xi8>) -> tensor<1x6x6x2xi32>
    %cst_1 = arith.constant dense<[1500000000, 1300000000]> : tensor<2xi32>
    %cst_2 = arith.constant dense<40> : tensor<2xi8>
    %cst_3 = arith.constant dense<0> : tensor<1xi32>
    %cst_4 = arith.constant dense<5> : tensor<1xi8>
    %3 = tosa.rescale %2, %cst_1, %cst_2, %cst_3, %cst_4 {input_unsigned = false, output_unsigned = false, per_channel = true, rounding_mode = DOUBLE_ROUND, scale32 = true} : (tensor<1x6x6x2xi32>, tensor<2xi32>, tensor<2xi8>, tensor<1xi32>, tensor<1xi8>) -> tensor<1x6x6x2xi8>
    %4 = tosa.clamp %3 {max_val = 100 : i8, min_val = 5 : i8} : (tensor<1x6x6x2xi8>) -> tensor<1x6x6x2xi8>
    return %4 : tensor<1x6x6x2xi8>
  }
}
'''


def test_conv_rescale_clamp_chain_becomes_one_op():
    w = np.random.default_rng(1).integers(-127, 128, (2, 3, 3, 4), dtype=np.int8)
    text = CONV.replace("WEIGHTHEX", w.tobytes().hex().upper())
    g = tosa_frontend.build_graph(text)
    assert [op.kind for op in g.ops] == ["conv2d"]
    op = g.ops[0]
    assert (op.consts["weights"].data == w).all() and op.consts["bias"].data.tolist() == [100, -200]
    a = op.attrs
    assert (a["in0_zp"], a["out_zp"], a["clamp_min"], a["clamp_max"], a["per_channel"], a["double_round"]) == (-3, 5, 5, 100, 1, 1)
    assert op.consts["multiplier"].data.tolist() == [1500000000, 1300000000] and op.consts["shift"].data.tolist() == [40, 40]
    x = np.random.default_rng(2).integers(-40, 40, (1, 6, 6, 4), dtype=np.int8)
    out = run_graph(g, [x])[0]
    assert out.shape == (1, 6, 6, 2) and out.min() >= 5 and out.max() <= 100


ADD = '''
module {
  func.func @main(%arg0: tensor<1x4x4x8xi8>, %arg1: tensor<1x4x4x8xi8>) -> tensor<1x4x4x8xi8> {
    %c = arith.constant dense<1073741824> : tensor<1xi32>
    %s = arith.constant dense<11> : tensor<1xi8>
    %z0 = arith.constant dense<-3> : tensor<1xi8>
    %z1 = arith.constant dense<7> : tensor<1xi8>
    %zero = arith.constant dense<0> : tensor<1xi32>
    %0 = tosa.rescale %arg0, %c, %s, %z0, %zero {input_unsigned = false, output_unsigned = false, per_channel = false, rounding_mode = DOUBLE_ROUND, scale32 = true} : (tensor<1x4x4x8xi8>, tensor<1xi32>, tensor<1xi8>, tensor<1xi8>, tensor<1xi32>) -> tensor<1x4x4x8xi32>
    %1 = tosa.rescale %arg1, %c, %s, %z1, %zero {input_unsigned = false, output_unsigned = false, per_channel = false, rounding_mode = DOUBLE_ROUND, scale32 = true} : (tensor<1x4x4x8xi8>, tensor<1xi32>, tensor<1xi8>, tensor<1xi8>, tensor<1xi32>) -> tensor<1x4x4x8xi32>
    %2 = tosa.add %0, %1 : (tensor<1x4x4x8xi32>, tensor<1x4x4x8xi32>) -> tensor<1x4x4x8xi32>
    %m = arith.constant dense<1200000000> : tensor<1xi32>
    %sh = arith.constant dense<49> : tensor<1xi8>
    %oz = arith.constant dense<-2> : tensor<1xi8>
    %3 = tosa.rescale %2, %m, %sh, %zero, %oz {input_unsigned = false, output_unsigned = false, per_channel = false, rounding_mode = DOUBLE_ROUND, scale32 = true} : (tensor<1x4x4x8xi32>, tensor<1xi32>, tensor<1xi8>, tensor<1xi32>, tensor<1xi8>) -> tensor<1x4x4x8xi8>
    return %3 : tensor<1x4x4x8xi8>
  }
}
'''


def test_add_chain_and_unsupported_ops():
    g = tosa_frontend.build_graph(ADD)
    assert [op.kind for op in g.ops] == ["add"]
    a = g.ops[0].attrs
    assert (a["in0_zp"], a["in1_zp"], a["in0_shift"], a["out_mult"], a["out_shift"], a["out_zp"]) == (-3, 7, 11, 1200000000, 49, -2)
    # another op in the place of the add is not the fused form: the chain is read op by op (generic rescales + elementwise op)
    g2 = tosa_frontend.build_graph(ADD.replace("tosa.add", "tosa.bitwise_and"))
    assert [op.kind for op in g2.ops] == ["rescale", "rescale", "ew", "rescale"]
    assert g2.ops[0].outputs[0].dtype == "i32" and g2.ops[3].outputs[0].dtype == "i8"
    with pytest.raises(NotImplementedError):
        tosa_frontend.build_graph(ADD.replace("tosa.add", "tosa.erf"))


TWO_STAGE = '''
module {
  func.func @main(%arg0: tensor<1x3x5x16xi8>, %arg1: tensor<1x3x5x16xi8>) -> tensor<1x3x5x16xi8> {
    %one = arith.constant dense<1073741824> : tensor<1xi32>
    %s9 = arith.constant dense<9> : tensor<1xi8>
    %z0 = arith.constant dense<-21> : tensor<1xi8>
    %zero = arith.constant dense<0> : tensor<1xi32>
    %0 = tosa.rescale %arg0, %one, %s9, %z0, %zero {input_unsigned = false, output_unsigned = false, per_channel = false, rounding_mode = DOUBLE_ROUND, scale32 = true} : (tensor<1x3x5x16xi8>, tensor<1xi32>, tensor<1xi8>, tensor<1xi8>, tensor<1xi32>) -> tensor<1x3x5x16xi32>
    %m0 = arith.constant dense<1711111111> : tensor<1xi32>
    %s32 = arith.constant dense<32> : tensor<1xi8>
    %1 = tosa.rescale %0, %m0, %s32, %zero, %zero {input_unsigned = false, output_unsigned = false, per_channel = false, rounding_mode = DOUBLE_ROUND, scale32 = true} : (tensor<1x3x5x16xi32>, tensor<1xi32>, tensor<1xi8>, tensor<1xi32>, tensor<1xi32>) -> tensor<1x3x5x16xi32>
    %s10 = arith.constant dense<10> : tensor<1xi8>
    %z1 = arith.constant dense<4> : tensor<1xi8>
    %2 = tosa.rescale %arg1, %one, %s10, %z1, %zero {input_unsigned = false, output_unsigned = false, per_channel = false, rounding_mode = DOUBLE_ROUND, scale32 = true} : (tensor<1x3x5x16xi8>, tensor<1xi32>, tensor<1xi8>, tensor<1xi8>, tensor<1xi32>) -> tensor<1x3x5x16xi32>
    %3 = tosa.OPNAME %1, %2 : (tensor<1x3x5x16xi32>, tensor<1x3x5x16xi32>) -> tensor<1x3x5x16xi32>
    %m = arith.constant dense<1100000000> : tensor<1xi32>
    %sh = arith.constant dense<50> : tensor<1xi8>
    %oz = arith.constant dense<-100> : tensor<1xi8>
    %4 = tosa.rescale %3, %m, %sh, %zero, %oz {input_unsigned = false, output_unsigned = false, per_channel = false, rounding_mode = DOUBLE_ROUND, scale32 = true} : (tensor<1x3x5x16xi32>, tensor<1xi32>, tensor<1xi8>, tensor<1xi32>, tensor<1xi8>) -> tensor<1x3x5x16xi8>
    return %4 : tensor<1x3x5x16xi8>
  }
}
'''


@pytest.mark.parametrize("name", ["add", "sub"])
def test_two_stage_input_rescale_becomes_a_left_shift(name):
    """i8 -> i32 with multiplier 2^30 and shift s (an exact left shift by 30 - s) followed by an i32 -> i32
    rescale: one op whose operand is shifted before its rescale. Checked against the staged arithmetic
    written out with the numpy restatement of apply_scale_32."""
    from oracle import oracle_np as onp
    g = tosa_frontend.build_graph(TWO_STAGE.replace("OPNAME", name))
    assert [op.kind for op in g.ops] == [name]
    a = g.ops[0].attrs
    assert (a["i0"], a["i1"], a["in0_zp"], a["in1_zp"]) == (21, 0, -21, 4)  # the single-stage operand keeps its rescale
    assert (a["in0_mult"], a["in0_shift"], a["in1_mult"], a["in1_shift"]) == (1711111111, 32, 1 << 30, 10)
    rng = np.random.default_rng(3)
    x, y = (rng.integers(-128, 128, (1, 3, 5, 16), dtype=np.int8) for _ in range(2))
    got = run_graph(g, [x, y])[0]
    r0 = onp.apply_scale_32(onp.apply_scale_32(x.astype(np.int64) + 21, 1 << 30, 9, True), 1711111111, 32, True)
    r1 = onp.apply_scale_32(y.astype(np.int64) - 4, 1 << 30, 10, True)
    v = r0 + r1 if name == "add" else r0 - r1
    want = np.clip(onp.apply_scale_32(v, 1100000000, 50, True) - 100, -128, 127).astype(np.int8)
    assert (got == want).all() and len(np.unique(got)) > 20


DYNAMIC = '''
module {
  func.func @main(%arg0: tensor<?x5x3xi32>) -> tensor<?x5x3xi32> {
    %0 = tosa.abs %arg0 : (tensor<?x5x3xi32>) -> tensor<?x5x3xi32>
    return %0 : tensor<?x5x3xi32>
  }
}
'''

TWICE = '''
module {
  func.func @main(%arg0: tensor<1x6x4xi8>, %arg1: tensor<1x4x5xi8>) -> (tensor<1x6x5xi32>, tensor<1x6x5xi32>) {
    %z = arith.constant dense<0> : tensor<1xi8>
    %0 = tosa.matmul %arg0, %arg1, %z, %z : (tensor<1x6x4xi8>, tensor<1x4x5xi8>, tensor<1xi8>, tensor<1xi8>) -> tensor<1x6x5xi32>
    return %0, %0 : tensor<1x6x5xi32>, tensor<1x6x5xi32>
  }
}
'''

RUNTIME_WEIGHTS = '''
module {
  func.func @main(%arg0: tensor<6x8xi8>, %arg1: tensor<5x8xi8>) -> tensor<6x1x1x5xi32> {
    %sx = tosa.const_shape {values = dense<[6, 1, 1, 8]> : tensor<4xindex>} : () -> !tosa.shape<4>
    %sw = tosa.const_shape {values = dense<[5, 1, 1, 8]> : tensor<4xindex>} : () -> !tosa.shape<4>
    %b = "tosa.const"() <{values = dense<0> : tensor<1xi32>}> : () -> tensor<1xi32>
    %zx = "tosa.const"() <{values = dense<-3> : tensor<1xi8>}> : () -> tensor<1xi8>
    %zw = "tosa.const"() <{values = dense<2> : tensor<1xi8>}> : () -> tensor<1xi8>
    %0 = tosa.reshape %arg0, %sx : (tensor<6x8xi8>, !tosa.shape<4>) -> tensor<6x1x1x8xi8>
    %1 = tosa.reshape %arg1, %sw : (tensor<5x8xi8>, !tosa.shape<4>) -> tensor<5x1x1x8xi8>
    %2 = tosa.conv2d %0, %1, %b, %zx, %zw {acc_type = i32, dilation = array<i64: 1, 1>, pad = array<i64: 0, 0, 0, 0>, stride = array<i64: 1, 1>} : (tensor<6x1x1x8xi8>, tensor<5x1x1x8xi8>, tensor<1xi32>, tensor<1xi8>, tensor<1xi8>) -> tensor<6x1x1x5xi32>
    return %2 : tensor<6x1x1x5xi32>
  }
}
'''

FLOAT_DEPTHWISE = '''
module {
  func.func @main(%arg0: tensor<1x5x4x2xbf16>) -> tensor<1x5x4x2xbf16> {
    %b = "tosa.const"() <{values = dense<[1.000000e+00, -2.000000e+00]> : tensor<2xbf16>}> : () -> tensor<2xbf16>
    %w = "tosa.const"() <{values = dense<5.000000e-01> : tensor<3x3x2x1xbf16>}> : () -> tensor<3x3x2x1xbf16>
    %z = arith.constant dense<0.000000e+00> : tensor<1xbf16>
    %0 = tosa.depthwise_conv2d %arg0, %w, %b, %z, %z {acc_type = f32, dilation = array<i64: 1, 1>, pad = array<i64: 1, 1, 1, 1>, stride = array<i64: 1, 1>} : (tensor<1x5x4x2xbf16>, tensor<3x3x2x1xbf16>, tensor<2xbf16>, tensor<1xbf16>, tensor<1xbf16>) -> tensor<1x5x4x2xbf16>
    return %0 : tensor<1x5x4x2xbf16>
  }
}
'''


def test_dynamic_extent_is_specialised_to_one():
    g = tosa_frontend.build_graph(DYNAMIC)
    assert [op.kind for op in g.ops] == ["ew"] and int(np.prod(g.inputs[0].shape)) == 15
    x = np.arange(-7, 8, dtype=np.int32).reshape(g.inputs[0].shape)
    assert (run_graph(g, [x])[0].ravel() == np.abs(x).ravel()).all()


def test_a_value_returned_twice_gets_a_copy():
    g = tosa_frontend.build_graph(TWICE)
    assert len(g.outputs) == 2 and g.outputs[0].id != g.outputs[1].id
    rng = np.random.default_rng(3)
    a, b = rng.integers(-128, 128, (1, 6, 4), dtype=np.int8), rng.integers(-128, 128, (1, 4, 5), dtype=np.int8)
    o0, o1 = run_graph(g, [a.reshape(g.inputs[0].shape), b.reshape(g.inputs[1].shape)])
    want = a[0].astype(np.int32) @ b[0].astype(np.int32)
    assert (o0.reshape(6, 5) == want).all() and (o1.reshape(6, 5) == want).all()


def test_convolution_of_two_runtime_tensors_is_a_matmul():
    g = tosa_frontend.build_graph(RUNTIME_WEIGHTS)
    assert "matmul_i32" in [op.kind for op in g.ops] and "conv2d" not in [op.kind for op in g.ops]
    rng = np.random.default_rng(4)
    x, w = rng.integers(-128, 128, (6, 8), dtype=np.int8), rng.integers(-128, 128, (5, 8), dtype=np.int8)
    out = run_graph(g, [x, w])[0]
    want = (x.astype(np.int32) + 3) @ (w.astype(np.int32) - 2).T
    assert (out.reshape(6, 5) == want).all()


def test_float_depthwise_accumulates_in_fp32():
    g = tosa_frontend.build_graph(FLOAT_DEPTHWISE)
    assert [op.kind for op in g.ops] == ["depthwise_f"]
    x = np.ones((1, 5, 4, 2), np.float32)
    out = run_graph(g, [tosa_frontend._to_bf16_bits(x)])[0]
    got = (out.astype(np.uint32) << 16).view(np.float32)
    # an inner pixel sees nine taps of 0.5, a corner four; then the bias
    assert got[0, 2, 1, 0] == 9 * 0.5 + 1.0 and got[0, 0, 0, 1] == 4 * 0.5 - 2.0
