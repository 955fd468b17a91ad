"""Golden cases made from the reference's own TOSA fixtures (tests/golden/make_tosa_cases.py):
the blob carries the fixture's constants, the .npz the seeded input and the output both
oracle restatements agreed on when the case was generated."""
import glob
import os

import numpy as np
import pytest

from oracle_exec import outputs_match, run_graph, uses_float_functions
from torq_b200.oplist import Graph

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = sorted(os.path.basename(p)[:-8] for p in glob.glob(os.path.join(HERE, "golden", "tosa_*.b200ops")))


def _load(name):
    with open(os.path.join(HERE, "golden", name + ".b200ops"), "rb") as f:
        blob = f.read()
    z = np.load(os.path.join(HERE, "golden", name + ".npz"))
    ins = [z[f"in{i}"] for i in range(sum(k.startswith("in") for k in z.files))]
    outs = [z[f"out{i}"] for i in range(sum(k.startswith("out") for k in z.files))]
    return blob, ins, outs


def test_cases_exist():
    assert len(CASES) >= 15


@pytest.mark.parametrize("name", CASES)
def test_oracle_reproduces_golden(name):
    blob, ins, outs = _load(name)
    g = Graph.deserialize(blob)
    assert g.serialize() == blob  # the reader is the exact inverse of the writer
    got = run_graph(g, ins)
    tolerant = uses_float_functions(g)
    for a, b, t in zip(got, outs, g.outputs):
        assert outputs_match(a, b, tolerant, t.dtype)


def test_fixture_constants_survive():
    # spot checks of constants that come from the reference's files
    g = Graph.deserialize(_load("tosa_conv2d_8x8")[0])
    op = g.ops[0]
    assert int(op.consts["multiplier"].data[0]) == 2003370132 and int(op.consts["shift"].data[0]) == 39
    assert op.attrs["in0_zp"] == -128 and op.attrs["out_zp"] == -128
    g = Graph.deserialize(_load("tosa_dw_peeling")[0])
    op = g.ops[0]
    assert op.consts["weights"].shape == (5, 5, 11, 1) and set(op.consts["shift"].data.tolist()) == {41}
    assert int(op.consts["multiplier"].data[0]) == 1494728868 and op.attrs["out_zp"] == 28
    g = Graph.deserialize(_load("tosa_add_single_rescale")[0])
    a = g.ops[0].attrs
    assert (a["in0_mult"], a["in0_shift"], a["out_mult"], a["out_shift"], a["out_zp"]) == (1 << 30, 11, 1093202297, 49, -2)
    g = Graph.deserialize(_load("tosa_maxpool2d_stride2_k3x3_pad_112x112x64")[0])
    a = g.ops[0].attrs
    assert (a["pad_t"], a["pad_b"], a["pad_l"], a["pad_r"], a["pad_value"]) == (0, 1, 0, 1, -100)


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_gpu_reproduces_golden(device, name):
    from torq_b200.runtime import Executable
    blob, ins, outs = _load(name)
    ex = Executable(device, blob)
    got = [np.empty(o.shape, o.np_dtype) for o in ex.outputs_info]
    ex.invoke_host([np.ascontiguousarray(a) for a in ins], got)
    ex.destroy()
    g = Graph.deserialize(blob)
    tolerant = uses_float_functions(g)  # exp and friends: +-1 LSB / a few ulp, everything else bit-exact
    for a, b, t in zip(got, outs, g.outputs):
        assert outputs_match(a, b, tolerant, t.dtype), f"{(a != b).sum()} of {a.size} differ"
