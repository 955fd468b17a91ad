"""Host-side checks that need no GPU: the C-ABI library loads and exports every symbol
include/torq_b200.h declares; the op-list serializer lays records out as the C header
does; failures surface as statuses, never as a CPU fallback."""
import ctypes
import os
import re

import numpy as np
import pytest

from torq_b200 import oplist, runtime
from torq_b200.oplist import Graph

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "torq_b200.h")).read()
    return sorted(set(re.findall(r"\b(tb200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = runtime.load_library()
    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/torq_b200.h but not exported"
    assert sorted(runtime.exported_symbols()) == declared


def test_status_strings_follow_iree_numbering():
    lib = runtime.load_library()
    assert lib.tb200_status_string(0) == b"OK"
    assert lib.tb200_status_string(3) == b"INVALID_ARGUMENT"
    assert lib.tb200_status_string(11) == b"OUT_OF_RANGE"
    assert lib.tb200_status_string(14) == b"UNAVAILABLE"


def test_struct_sizes_match_header():
    hdr = open(os.path.join(ROOT, "include", "torq_b200_ops.h")).read()
    # count the 4-byte fields of tb200_op_t in the header
    body = hdr.split("typedef struct tb200_op {")[1].split("} tb200_op_t;")[0]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    n_fields = sum(len(decl.split(",")) for decl in re.findall(r"(?:uint32_t|int32_t|float)\s+([^;]+);", body))
    assert n_fields * 4 == ctypes.sizeof(oplist.OpRec) == 184
    assert ctypes.sizeof(oplist.TensorRec) == 48 and ctypes.sizeof(oplist.Header) == 80
    for name, val in oplist.OP_KINDS.items():
        assert re.search(rf"TB200_OP_\w+ = {val},", hdr), name


def test_serialize_layout_roundtrip():
    g = Graph()
    x = g.input((1, 4, 4, 8))
    y = g.conv2d(x, np.ones((16, 1, 1, 8), np.int8), np.arange(16, dtype=np.int32), [1 << 30] * 16, [35] * 16,
                 input_zp=-3, out_zp=5)
    g.output(y)
    blob = g.serialize()
    h = oplist.Header.from_buffer_copy(blob[:80])
    assert h.magic == oplist.MAGIC and h.version == 1 and h.total_bytes == len(blob)
    assert (h.n_tensors, h.n_ops, h.n_inputs, h.n_outputs) == (6, 1, 1, 1)
    op = oplist.OpRec.from_buffer_copy(blob[h.ops_offset:h.ops_offset + 184])
    assert op.kind == 1 and op.in0 == x.id and op.out0 == y.id and op.in0_zp == -3 and op.out_zp == 5
    assert op.per_channel == 1 and op.double_round == 1 and op.in1 == -1
    bias_t = oplist.TensorRec.from_buffer_copy(blob[h.tensors_offset + 48 * op.bias:][:48])
    raw = blob[h.const_offset + bias_t.const_offset:][:bias_t.const_bytes]
    assert (np.frombuffer(raw, np.int32) == np.arange(16)).all()
    for off in (h.tensors_offset, h.ops_offset, h.inputs_offset, h.outputs_offset, h.const_offset):
        assert off % 16 == 0


def test_no_cpu_fallback_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(runtime.TorqB200Error) as e:
        runtime.Device(0)
    assert e.value.status_name == "UNAVAILABLE"


def test_graph_builder_rejects_bad_shapes():
    g = Graph()
    x = g.input((1, 4, 4, 8))
    with pytest.raises(ValueError):
        g.conv2d(x, np.ones((16, 1, 1, 7), np.int8), np.zeros(16, np.int32), [1 << 30], [30])
    with pytest.raises(ValueError):
        g.add(x, g.input((1, 4, 4, 9)), a_zp=0, a_ms=(1 << 30, 30), b_zp=0, b_ms=(1 << 30, 30), out_ms=(1 << 30, 30),
              out_zp=0)
    with pytest.raises(ValueError):
        g.table(x, np.zeros(255, np.int8))


def test_workload_builders_match_the_benchmark_shapes():
    from torq_b200.workloads.mobilenet_v2 import build_mobilenet_v2
    from torq_b200.workloads.yolov8n import build_yolov8n
    from torq_b200.workloads import gemma3
    g, layers = build_mobilenet_v2(1)
    assert sum(l["macs"] for l in layers) == 300774272 and sum(l["weight_bytes"] for l in layers) == 3469760
    assert sum(1 for l in layers if l["kind"] in ("conv2d", "depthwise")) == 52
    g, macs = build_yolov8n(1, 640)
    assert [o.shape for o in g.outputs] == [(1, 80, 80, 64), (1, 80, 80, 80), (1, 40, 40, 64), (1, 40, 40, 80),
                                            (1, 20, 20, 64), (1, 20, 20, 80)]
    assert 4.2e9 < macs < 4.6e9
    assert gemma3.weight_bytes_per_token(gemma3.GemmaConfig()) == 999751680
    cfg = gemma3.GemmaConfig()
    assert [cfg.is_global(l) for l in range(7)] == [False] * 5 + [True, False]
