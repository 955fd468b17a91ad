"""The two restatements of the oracle (C and numpy) against each other, against
known-answer identities of TOSA apply_scale_32, and against the constants the
reference's own TOSA fixtures carry."""
import numpy as np
import pytest

from oracle import oracle as oc
from oracle import oracle_np as onp

RNG = lambda s=1234: np.random.default_rng(s)  # noqa: E731  (reference harness seed, python/torq/testing/iree.py:1264)


def test_apply_scale_identities():
    rng = RNG()
    vals = np.concatenate([rng.integers(-2**31, 2**31, 2000), [0, 1, -1, 2**31 - 1, -2**31]]).astype(np.int64)
    # M = 2^30, S = 30 is the identity
    assert (onp.apply_scale_32(vals, 1 << 30, 30, True) == vals).all()
    for v in vals[:200]:
        assert oc.apply_scale_32(int(v), 1 << 30, 30, True) == v
    # for S <= 31 double rounding equals single rounding
    for s in (2, 11, 30, 31):
        m = int(rng.integers(1 << 30, 1 << 31))
        assert (onp.apply_scale_32(vals, m, s, True) == onp.apply_scale_32(vals, m, s, False)).all()
    # input-side form of the reference's add fixture: M = 2^30, S = 11 is a left shift by 19
    small = rng.integers(-255, 256, 100)
    assert (onp.apply_scale_32(small, 1 << 30, 11, True) == small * (1 << 19)).all()


def test_apply_scale_c_equals_numpy():
    rng = RNG(7)
    for _ in range(3000):
        v = int(rng.integers(-2**31, 2**31))
        s = int(rng.integers(2, 63))
        m = int(rng.integers(0, 1 << 31))
        dr = bool(rng.integers(0, 2))
        assert oc.apply_scale_32(v, m, s, dr) == int(onp.apply_scale_32(v, m, s, dr))


def test_apply_scale_known_answers():
    # worked by hand from the TOSA definition
    assert oc.apply_scale_32(3, 1 << 30, 31, False) == 2      # 1.5 -> 2 (round half up)
    assert oc.apply_scale_32(-3, 1 << 30, 31, False) == -1    # -1.5 -> -1 (round half up)
    assert oc.apply_scale_32(-3, 1 << 30, 31, True) == -1     # shift 31: no second rounding
    # shift 32 with double rounding: ties move away from zero
    assert oc.apply_scale_32(3, 1 << 30, 32, True) == 1       # 0.75 -> 1
    assert oc.apply_scale_32(-2, 1 << 30, 32, True) == -1     # -0.5: (-2^31 + 2^31 - 2^30) >> 32 = -1
    assert oc.apply_scale_32(-2, 1 << 30, 32, False) == 0     # single rounding gives 0
    # constants of tests/testdata/gen_ops/conv2d_8x8.mlir: multiplier 2003370132, shift 39
    real = 2003370132 / 2.0**39
    for acc in (-50000, -1, 0, 1, 12345, 99999):
        assert abs(oc.apply_scale_32(acc, 2003370132, 39, True) - acc * real) <= 0.5 + 1e-9


def test_quantize_multiplier_and_reciprocal():
    rng = RNG(3)
    for r in np.concatenate([rng.uniform(1e-6, 4.0, 300), [0.5, 1.0, 0.25, 1e-9]]):
        m, s = oc.quantize_multiplier(float(r))
        assert (m, s) == onp.quantize_multiplier(float(r))
        assert 2 <= s <= 62
        if s < 62:
            assert (1 << 30) <= m < (1 << 31)
        assert abs(m / 2.0**s - r) <= r * 2**-30
    from torq_b200.quant import quantize_multiplier
    for r in rng.uniform(1e-6, 4.0, 300):
        assert quantize_multiplier(float(r)) == oc.quantize_multiplier(float(r))
    for c in list(range(1, 200)) + [49, 12544, 50176]:
        m, s = oc.reciprocal_scale(c)
        assert (m, s) == onp.reciprocal_scale(c)
        assert (1 << 30) <= m < (1 << 31) or c == 1
    # avgpool2d.mlir is a 7x7 global pool: count 49
    assert oc.reciprocal_scale(49) == ((((1 << 30) + 1) << 6) // 49, 36)


def _rand_requant(rng, oc_n, lo=2e-4, hi=8e-3):
    ms = [oc.quantize_multiplier(float(r)) for r in rng.uniform(lo, hi, oc_n)]
    return np.array([m for m, _ in ms], np.int32), np.array([s for _, s in ms], np.int8)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("case", [
    dict(x=(2, 9, 11, 5), oc=7, k=(3, 3), stride=(2, 1), dil=(1, 1), pad=(1, 1, 0, 1), izp=-3, wzp=0),
    dict(x=(1, 8, 8, 1), oc=1, k=(3, 3), stride=(1, 1), dil=(1, 1), pad=(1, 1, 1, 1), izp=-128, wzp=0),
    dict(x=(1, 13, 13, 4), oc=6, k=(5, 5), stride=(2, 2), dil=(1, 1), pad=(2, 2, 2, 2), izp=7, wzp=3),
    dict(x=(1, 10, 12, 8), oc=16, k=(3, 3), stride=(1, 1), dil=(2, 2), pad=(2, 2, 2, 2), izp=0, wzp=0),
    dict(x=(3, 6, 6, 16), oc=24, k=(1, 1), stride=(1, 1), dil=(1, 1), pad=(0, 0, 0, 0), izp=-5, wzp=0),
])
def test_conv2d_c_equals_numpy(case, mode):
    rng = RNG(11)
    x = rng.integers(-128, 128, case["x"], dtype=np.int8)
    w = rng.integers(-127, 128, (case["oc"],) + case["k"] + (case["x"][3],), dtype=np.int8)
    bias = np.round(rng.normal(0, 2000, case["oc"])).astype(np.int32)
    m, s = _rand_requant(rng, case["oc"])
    a = oc.conv2d(x, w, bias, oc.Requant(m, s, 5, -128, 127, mode=mode), case["stride"], case["dil"], case["pad"],
                  case["izp"], case["wzp"])
    b = onp.conv2d(x, w, bias, m, s, 5, -128, 127, case["stride"], case["dil"], case["pad"], case["izp"],
                   case["wzp"], mode=mode)
    assert a.shape == b.shape and (a == b).all()
    assert len(np.unique(a)) > 4  # not saturated into a corner


def test_conv_unit_weights_is_box_sum():
    rng = RNG(5)
    x = rng.integers(-20, 20, (1, 6, 7, 3), dtype=np.int8)
    w = np.ones((2, 3, 3, 3), np.int8)
    out = oc.conv2d(x, w, np.zeros(2, np.int32), oc.Requant([1 << 30], [30], 0, -128, 127), pad=(1, 1, 1, 1))
    xp = np.pad(x.astype(np.int64), ((0, 0), (1, 1), (1, 1), (0, 0)))
    box = sum(xp[:, i:i + 6, j:j + 7, :] for i in range(3) for j in range(3)).sum(-1)
    assert (out[..., 0] == np.clip(box, -128, 127)).all() and (out[..., 1] == out[..., 0]).all()


@pytest.mark.parametrize("mode", [0, 1])
def test_depthwise_c_equals_numpy(mode):
    rng = RNG(12)
    # the dw_peeling fixture shape class: odd channel count, 5x5, pad 2, shift 41
    for shape, k, M, stride, pad, izp in [((1, 14, 14, 11), (5, 5), 1, (1, 1), (2, 2, 2, 2), -128),
                                          ((2, 9, 8, 8), (3, 3), 1, (2, 2), (0, 1, 0, 1), 4),
                                          ((1, 7, 7, 3), (3, 3), 2, (1, 1), (1, 1, 1, 1), -1),
                                          ((1, 12, 12, 4), (4, 4), 1, (2, 2), (1, 1, 1, 1), 0)]:
        x = rng.integers(-128, 128, shape, dtype=np.int8)
        w = rng.integers(-127, 128, k + (shape[3], M), dtype=np.int8)
        OC = shape[3] * M
        bias = np.round(rng.normal(0, 1000, OC)).astype(np.int32)
        m, s = _rand_requant(rng, OC, 1e-3, 2e-2)
        a = oc.depthwise(x, w, bias, oc.Requant(m, s, 28, -128, 127, mode=mode), stride, (1, 1), pad, izp, 0)
        b = onp.depthwise(x, w, bias, m, s, 28, -128, 127, stride, (1, 1), pad, izp, 0, mode=mode)
        assert (a == b).all()


def test_requant_modes_differ_by_at_most_one_lsb():
    # the reference's own tolerance between its NPU and host arithmetic
    # (python/torq/testing/comparison.py:42-49)
    rng = RNG(13)
    x = rng.integers(-40, 40, (1, 12, 12, 16), dtype=np.int8)  # the reference's test input range
    w = rng.integers(-127, 128, (8, 3, 3, 16), dtype=np.int8)
    bias = np.zeros(8, np.int32)
    m, s = _rand_requant(rng, 8, 5e-4, 4e-3)
    a = oc.conv2d(x, w, bias, oc.Requant(m, s, 0, -128, 127, mode=0), pad=(1, 1, 1, 1)).astype(int)
    b = oc.conv2d(x, w, bias, oc.Requant(m, s, 0, -128, 127, mode=1), pad=(1, 1, 1, 1)).astype(int)
    assert np.abs(a - b).max() <= 1


def test_fc_matmul_pool_eltwise_c_equals_numpy():
    rng = RNG(14)
    a8 = rng.integers(-128, 128, (5, 40), dtype=np.int8)
    w8 = rng.integers(-127, 128, (9, 40), dtype=np.int8)
    bias = np.round(rng.normal(0, 500, 9)).astype(np.int32)
    m, s = _rand_requant(rng, 9, 1e-3, 5e-3)
    for izp in (0, -7):
        assert (oc.fully_connected(a8, w8, bias, oc.Requant(m, s, -2, -128, 127), izp) ==
                onp.fully_connected(a8, w8, bias, m, s, -2, -128, 127, izp)).all()
    b8 = rng.integers(-128, 128, (40, 6), dtype=np.int8)
    assert (oc.matmul_i32(a8, b8, -7, 2) == onp.matmul_i32(a8, b8, -7, 2)).all()

    x = rng.integers(-128, 128, (2, 11, 12, 6), dtype=np.int8)
    for kern, st, pad in [((3, 3), (2, 2), (0, 1, 0, 1)), ((5, 5), (1, 1), (2, 2, 2, 2)), ((2, 2), (2, 2), (0, 0, 0, 0))]:
        assert (oc.maxpool(x, kern, st, pad, -100) == onp.maxpool(x, kern, st, pad, -100)).all()
        assert (oc.avgpool(x, kern, st, pad, 4, -3) == onp.avgpool(x, kern, st, pad, 4, -3)).all()
    assert (oc.avgpool(x, (11, 12), (1, 1), (0, 0, 0, 0), 4, 0) == onp.avgpool(x, (11, 12), (1, 1), (0, 0, 0, 0), 4, 0)).all()

    y = rng.integers(-128, 128, x.shape, dtype=np.int8)
    # constants of tests/testdata/tosa_ops/add-single-rescale.mlir
    args = (-3, 1 << 30, 11, -3, 1 << 30, 11, 1093202297, 49, -2)
    for kind in ("add", "sub"):
        assert (oc.binary(kind, x, y, *args) == onp.binary(kind, x, y, *args)).all()
    margs = (3, 1 << 30, 30, -4, 1 << 30, 30, 1518500250, 38, 1)
    assert (oc.binary("mul", x, y, *margs) == onp.binary("mul", x, y, *margs)).all()
    assert len(np.unique(oc.binary("mul", x, y, *margs))) > 10

    tbl = rng.integers(-128, 128, 256, dtype=np.int8)
    assert (oc.table(x, tbl) == onp.table(x, tbl)).all()
    m6, s6 = _rand_requant(rng, 6, 0.3, 1.9)
    assert (oc.rescale(x, oc.Requant(m6, s6, 3), 5) == onp.rescale(x, m6, s6, 5, 3)).all()
    assert (oc.resize_nn2x(x) == onp.resize_nn2x(x)).all()
    z = rng.integers(-128, 128, (2, 11, 12, 10), dtype=np.int8)
    cargs = (3, 1500000000, 31, -5, 1200000000, 30, 7)
    assert (oc.concat2(x, z, *cargs) == onp.concat2(x, z, *cargs)).all()


def test_add_fixture_doubles_and_rescales():
    # add-single-rescale.mlir adds the input to itself: out = rescale(2 * (x + 3) << 19) - 2
    x = np.arange(-128, 128, dtype=np.int8).reshape(1, 16, 16, 1)
    out = oc.binary("add", x, x, -3, 1 << 30, 11, -3, 1 << 30, 11, 1093202297, 49, -2).astype(int)
    real = 2 * (x.astype(int) + 3) * 2.0**19 * 1093202297 / 2.0**49 - 2
    assert np.abs(out - np.clip(np.round(real), -128, 127)).max() <= 1
