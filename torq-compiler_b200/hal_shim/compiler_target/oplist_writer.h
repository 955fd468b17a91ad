// Writer of torq-b200-ops executables (include/torq_b200_ops.h) for the compiler side: the sibling of the
// reference's flatbuffer serializer (compiler/torq/Serialization/Serialization.cpp:265-306 writes `torq-fb`; this
// writes the op list the B200 runtime plans from). Plain C++17, no MLIR: TorqB200Target.cpp drives it from TorqHL
// ops, and tests/test_oplist_writer.py compiles it alone and compares its bytes with the Python serializer's
// (torq_b200/oplist.py), which is what keeps the two in step.
#pragma once
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "torq_b200_ops.h"

namespace torq_b200 {

class OpListWriter {
 public:
  // A tensor of the graph; returns its id. `shape` has 1..4 extents.
  int addTensor(tb200_dtype dtype, tb200_tensor_kind kind, const std::vector<int64_t>& shape) {
    tb200_tensor_t t;
    std::memset(&t, 0, sizeof(t));
    t.dtype = (uint32_t)dtype;
    t.kind = (uint32_t)kind;
    t.rank = (uint32_t)shape.size();
    for (int i = 0; i < 4; i++) t.shape[i] = i < (int)shape.size() ? (int32_t)shape[i] : 1;
    tensors_.push_back(t);
    const int id = (int)tensors_.size() - 1;
    if (kind == TB200_TENSOR_INPUT) inputs_.push_back(id);
    return id;
  }
  // A constant tensor with its bytes (weights, bias, multipliers, shifts, tables); 16-byte aligned in the blob.
  int addConstant(tb200_dtype dtype, const std::vector<int64_t>& shape, const void* data, size_t bytes) {
    const int id = addTensor(dtype, TB200_TENSOR_CONSTANT, shape);
    consts_.resize((consts_.size() + 15) & ~(size_t)15, 0);
    tensors_[id].const_offset = consts_.size();
    tensors_[id].const_bytes = bytes;
    const uint8_t* p = static_cast<const uint8_t*>(data);
    consts_.insert(consts_.end(), p, p + bytes);
    return id;
  }
  void markOutput(int tensor) { outputs_.push_back(tensor); }

  // An op record with the defaults every producer of the format uses (no operands, unit strides and dilations,
  // int8 clamp range, shifts of 2); the caller fills in what its op has and appends it.
  static tb200_op_t blankOp(tb200_op_kind kind) {
    tb200_op_t op;
    std::memset(&op, 0, sizeof(op));
    op.kind = (uint32_t)kind;
    op.in0 = op.in1 = op.in2 = op.out0 = op.out1 = -1;
    op.weights = op.bias = op.multiplier = op.shift = op.table = -1;
    op.stride_h = op.stride_w = op.dil_h = op.dil_w = 1;
    op.clamp_min = -128;
    op.clamp_max = 127;
    op.out_shift = op.in0_shift = op.in1_shift = 2;
    return op;
  }
  void addOp(const tb200_op_t& op) { ops_.push_back(op); }

  // The executable: header, tensor records, op records, input ids, output ids, constants; every section 16-byte aligned.
  std::vector<uint8_t> finish() const {
    auto align = [](uint64_t n) { return (n + 15) & ~(uint64_t)15; };
    tb200_ops_header_t h;
    std::memset(&h, 0, sizeof(h));
    h.magic = TB200_OPS_MAGIC;
    h.version = TB200_OPS_VERSION;
    h.n_tensors = (uint32_t)tensors_.size();
    h.n_ops = (uint32_t)ops_.size();
    h.n_inputs = (uint32_t)inputs_.size();
    h.n_outputs = (uint32_t)outputs_.size();
    uint64_t off = align(sizeof(h));
    h.tensors_offset = off;
    off = align(off + tensors_.size() * sizeof(tb200_tensor_t));
    h.ops_offset = off;
    off = align(off + ops_.size() * sizeof(tb200_op_t));
    h.inputs_offset = off;
    off = align(off + 4 * inputs_.size());
    h.outputs_offset = off;
    off = align(off + 4 * outputs_.size());
    h.const_offset = off;
    h.const_bytes = consts_.size();
    h.total_bytes = off + consts_.size();
    std::vector<uint8_t> out(h.total_bytes, 0);
    std::memcpy(out.data(), &h, sizeof(h));
    if (!tensors_.empty()) std::memcpy(out.data() + h.tensors_offset, tensors_.data(), tensors_.size() * sizeof(tb200_tensor_t));
    if (!ops_.empty()) std::memcpy(out.data() + h.ops_offset, ops_.data(), ops_.size() * sizeof(tb200_op_t));
    for (size_t i = 0; i < inputs_.size(); i++) std::memcpy(out.data() + h.inputs_offset + 4 * i, &inputs_[i], 4);
    for (size_t i = 0; i < outputs_.size(); i++) std::memcpy(out.data() + h.outputs_offset + 4 * i, &outputs_[i], 4);
    if (!consts_.empty()) std::memcpy(out.data() + h.const_offset, consts_.data(), consts_.size());
    return out;
  }

 private:
  std::vector<tb200_tensor_t> tensors_;
  std::vector<tb200_op_t> ops_;
  std::vector<int32_t> inputs_, outputs_;
  std::vector<uint8_t> consts_;
};

}  // namespace torq_b200
