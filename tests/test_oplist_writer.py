"""The compiler-side writer of torq-b200-ops executables (hal_shim/compiler_target/oplist_writer.h, plain C++) against
the Python serializer: the same small graph built through both must give the same bytes, and the C++ blob must
deserialize to the same graph. Compiled here with g++; no GPU and no MLIR involved."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "torq-compiler_b200"))
from torq_b200.oplist import Graph  # noqa: E402

PROGRAM = r'''
#include <cstdio>
#include "oplist_writer.h"
using namespace torq_b200;
int main(int argc, char** argv) {
  OpListWriter w;
  const int x = w.addTensor(TB200_I8, TB200_TENSOR_INPUT, {4, 8});
  int32_t mult[3] = {1342177280, 1500000000, 1100000000};
  int8_t shift[3] = {38, 39, 37};
  int8_t weights[3 * 8];
  for (int i = 0; i < 24; i++) weights[i] = (int8_t)(i * 7 - 80);
  int32_t bias[3] = {100, -200, 300};
  const int m = w.addConstant(TB200_I32, {3}, mult, sizeof(mult));
  const int s = w.addConstant(TB200_I8, {3}, shift, sizeof(shift));
  const int wt = w.addConstant(TB200_I8, {3, 8}, weights, sizeof(weights));
  const int b = w.addConstant(TB200_I32, {3}, bias, sizeof(bias));
  const int y = w.addTensor(TB200_I8, TB200_TENSOR_ACTIVATION, {4, 3});
  tb200_op_t op = OpListWriter::blankOp(TB200_OP_FC);
  op.in0 = x; op.out0 = y; op.weights = wt; op.bias = b; op.multiplier = m; op.shift = s;
  op.in0_zp = -3; op.weight_zp = 0; op.out_zp = 5; op.clamp_min = -128; op.clamp_max = 127;
  op.per_channel = 1; op.double_round = 1; op.requant_mode = TB200_REQUANT_TOSA;
  w.addOp(op);
  const int t = w.addTensor(TB200_I8, TB200_TENSOR_OUTPUT, {4, 3});
  int8_t table[256];
  for (int i = 0; i < 256; i++) table[i] = (int8_t)(255 - i);
  tb200_op_t top = OpListWriter::blankOp(TB200_OP_TABLE);
  top.in0 = y; top.out0 = t;
  top.table = w.addConstant(TB200_I8, {256}, table, sizeof(table));
  w.addOp(top);
  w.markOutput(t);
  const std::vector<uint8_t> blob = w.finish();
  FILE* f = fopen(argv[1], "wb");
  fwrite(blob.data(), 1, blob.size(), f);
  fclose(f);
  return 0;
}
'''


def test_cpp_writer_matches_python_serializer(tmp_path):
    src = tmp_path / "w.cc"
    src.write_text(PROGRAM)
    exe = tmp_path / "w"
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"),
                    "-I", os.path.join(ROOT, "torq-compiler_b200", "hal_shim", "compiler_target"), str(src), "-o", str(exe)],
                   check=True)
    out = tmp_path / "blob.bin"
    subprocess.run([str(exe), str(out)], check=True)
    blob = out.read_bytes()

    g = Graph()
    x = g.input((4, 8))
    weights = (np.arange(24) * 7 - 80).astype(np.int8).reshape(3, 8)
    y = g.fully_connected(x, weights, np.array([100, -200, 300], np.int32), np.array([1342177280, 1500000000, 1100000000]),
                          np.array([38, 39, 37]), input_zp=-3, out_zp=5)
    # the C++ side created the table's output tensor before the table constant: do the same here
    t = g._tensor((4, 3), "i8", 0)
    table = (255 - np.arange(256)).astype(np.uint8).view(np.int8)
    from torq_b200.oplist import Op
    g.ops.append(Op("table", [y], [t], {"table": g.const(table)}, {}))
    g.output(t)
    want = g.serialize()
    g2 = Graph.deserialize(blob)
    assert [op.kind for op in g2.ops] == ["fc", "table"]
    assert (g2.ops[0].consts["weights"].data == weights).all()
    assert g2.ops[0].attrs["in0_zp"] == -3 and g2.ops[0].attrs["per_channel"] == 1
    assert blob == want
