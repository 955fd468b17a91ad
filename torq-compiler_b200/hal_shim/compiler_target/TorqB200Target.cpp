// IREE HAL target backend "torq_b200": the compiler-side sibling of the reference's `torq` target
// (compiler/torq/Target/TorqTarget.cpp:111-146). UNCOMPILED HERE: it needs the IREE / MLIR trees the reference
// builds against (third_party/iree, absent from this build environment). The part that does not need them, the
// writer of the executable format, is oplist_writer.h and is compiled and tested on its own.
//
// What it does: the reference lowers a dispatch through Linalg -> TorqHL and then on to NPU descriptors
// (TorqHL -> TorqHW, LRAM tiling, NSS programs). A B200 executable needs none of the NPU part: this backend runs the
// reference's own front half up to the TorqHL level (the Linalg -> TorqHL conversion patterns are the semantic
// contract, compiler/torq/Conversions/LinalgToTorqHL) and then writes ONE record per TorqHL op into the
// `torq-b200-ops` format (include/torq_b200_ops.h); the B200 runtime plans kernels from those records
// (csrc/plan.cu). TorqHL carries the NPU form of the rescale - an interleaved (bias, scale) tensor and one
// `shift_factor` per op (compiler/torq/Dialect/TorqHL/TorqHLOps.td:119-170) - which is requant mode
// TB200_REQUANT_NPU of the format; a front end that still has the TOSA multiplier[] / shift[] pairs (the text front
// end, torq_b200/tosa_frontend.py) writes TB200_REQUANT_TOSA instead.
#include "torq/Dialect/TorqHL/TorqHLDialect.h"
#include "torq/Dialect/TorqHL/TorqHLOps.h"

#include "iree/compiler/Dialect/HAL/Target/TargetRegistry.h"
#include "iree/compiler/PluginAPI/Client.h"
#include "mlir/Dialect/Func/IR/FuncOps.h"
#include "mlir/IR/BuiltinAttributes.h"
#include "mlir/IR/BuiltinOps.h"
#include "mlir/IR/Matchers.h"
#include "llvm/ADT/DenseMap.h"

#include "oplist_writer.h"

namespace mlir::syna::torq_b200 {

using namespace mlir::iree_compiler;
namespace hl = mlir::syna::torq_hl;

namespace {

// The front half of the reference's pipeline: everything of addAllPasses() (compiler/torq/Codegen/
// TORQLowerExecutableTargetPass.cpp:395-407) before tiling and TorqHW, i.e. the TOSA / Linalg -> TorqHL conversions
// with the pattern fusions (rescale chains, activation tables, pad folding).
void buildTorqHLOnlyPassPipeline(OpPassManager &variantPassManager);  // declared by the reference's Codegen/Passes.h split

tb200_dtype dtypeOf(Type elementType) {
    if (elementType.isInteger(8)) return TB200_I8;
    if (elementType.isInteger(16)) return TB200_I16;
    if (elementType.isInteger(32)) return TB200_I32;
    if (elementType.isBF16()) return TB200_BF16;
    return TB200_F32;
}

class OpListEmitter {
  public:
    explicit OpListEmitter(func::FuncOp func) : func_(func) {}

    LogicalResult run(std::vector<uint8_t> &blob) {
        for (BlockArgument arg : func_.getArguments())
            ids_[arg] = addValue(arg, TB200_TENSOR_INPUT);
        WalkResult r = func_.walk([&](Operation *op) {
            if (isa<func::ReturnOp>(op)) {
                for (Value v : op->getOperands()) writer_.markOutput(ids_.lookup(v));
                return WalkResult::advance();
            }
            if (op->getDialect() && op->getDialect()->getNamespace() == "torq_hl")
                return failed(emit(op)) ? WalkResult::interrupt() : WalkResult::advance();
            return WalkResult::advance();
        });
        if (r.wasInterrupted()) return failure();
        blob = writer_.finish();
        return success();
    }

  private:
    int addValue(Value v, tb200_tensor_kind kind) {
        auto type = cast<ShapedType>(v.getType());
        std::vector<int64_t> shape(type.getShape().begin(), type.getShape().end());
        return writer_.addTensor(dtypeOf(type.getElementType()), kind, shape);
    }
    // A constant operand (weights, scale_bias, table): its bytes go into the constants section.
    int addConstantOperand(Value v) {
        DenseElementsAttr attr;
        if (!matchPattern(v, m_Constant(&attr))) return -1;
        auto type = cast<ShapedType>(attr.getType());
        std::vector<int64_t> shape(type.getShape().begin(), type.getShape().end());
        ArrayRef<char> raw = attr.getRawData();
        return writer_.addConstant(dtypeOf(type.getElementType()), shape, raw.data(), raw.size());
    }
    // TorqHL's scale_bias is (bias, scale) interleaved per output channel: split it into the two tables of a record.
    LogicalResult addScaleBias(Value scaleBias, int shiftFactor, tb200_op_t &op) {
        DenseIntElementsAttr attr;
        if (!matchPattern(scaleBias, m_Constant(&attr))) return failure();
        std::vector<int32_t> bias, scale;
        int i = 0;
        for (APInt v : attr.getValues<APInt>()) ((i++ & 1) ? scale : bias).push_back((int32_t)v.getSExtValue());
        const int64_t n = (int64_t)bias.size();
        std::vector<int8_t> shift(1, (int8_t)shiftFactor);
        op.bias = writer_.addConstant(TB200_I32, {n}, bias.data(), bias.size() * 4);
        op.multiplier = writer_.addConstant(TB200_I32, {n}, scale.data(), scale.size() * 4);
        op.shift = writer_.addConstant(TB200_I8, {1}, shift.data(), 1);
        op.per_channel = n > 1;
        op.requant_mode = TB200_REQUANT_NPU;
        return success();
    }
    template <typename ConvLike> LogicalResult emitConv(ConvLike conv, tb200_op_kind kind) {
        tb200_op_t op = torq_b200::OpListWriter::blankOp(kind);
        op.in0 = ids_.lookup(conv.getInput());
        op.weights = addConstantOperand(conv.getWeights());
        if (op.weights < 0 || failed(addScaleBias(conv.getScaleBias(), conv.getShiftFactor(), op)))
            return conv.emitError("weights and scale_bias must be constants");
        auto wshape = cast<ShapedType>(conv.getWeights().getType()).getShape();  // OHWI
        op.kh = (int32_t)wshape[1];
        op.kw = (int32_t)wshape[2];
        op.stride_h = (int32_t)conv.getStride()[0];
        op.stride_w = (int32_t)conv.getStride()[1];
        op.dil_h = (int32_t)conv.getDilation()[0];
        op.dil_w = (int32_t)conv.getDilation()[1];
        op.pad_l = (int32_t)conv.getPad()[0];  // TorqHL pad order: left, right, top, bottom
        op.pad_r = (int32_t)conv.getPad()[1];
        op.pad_t = (int32_t)conv.getPad()[2];
        op.pad_b = (int32_t)conv.getPad()[3];
        op.in0_zp = conv.getInputZp();
        op.weight_zp = conv.getWeightZp();
        op.out_zp = conv.getOutputZp();
        op.clamp_min = conv.getOutputMin();
        op.clamp_max = conv.getOutputMax();
        op.out0 = ids_[conv->getResult(0)] = addValue(conv->getResult(0), TB200_TENSOR_ACTIVATION);
        writer_.addOp(op);
        return success();
    }
    LogicalResult emit(Operation *op) {
        if (auto conv = dyn_cast<hl::Conv2DOp>(op)) return emitConv(conv, TB200_OP_CONV2D);
        if (auto dw = dyn_cast<hl::DepthwiseConv2DOp>(op)) return emitConv(dw, TB200_OP_DEPTHWISE);
        if (auto fc = dyn_cast<hl::FullyConnectedOp>(op)) {
            tb200_op_t rec = torq_b200::OpListWriter::blankOp(TB200_OP_FC);
            rec.in0 = ids_.lookup(fc.getInput());
            rec.weights = addConstantOperand(fc.getWeights());
            if (rec.weights < 0 || failed(addScaleBias(fc.getScaleBias(), fc.getShiftFactor(), rec)))
                return fc.emitError("weights and scale_bias must be constants");
            rec.in0_zp = fc.getInputZp();
            rec.weight_zp = fc.getWeightZp();
            rec.out_zp = fc.getOutputZp();
            rec.clamp_min = fc.getOutputMin();
            rec.clamp_max = fc.getOutputMax();
            rec.out0 = ids_[fc->getResult(0)] = addValue(fc->getResult(0), TB200_TENSOR_ACTIVATION);
            writer_.addOp(rec);
            return success();
        }
        if (auto pool = dyn_cast<hl::MaxPool2dOp>(op)) {
            tb200_op_t rec = torq_b200::OpListWriter::blankOp(TB200_OP_MAXPOOL);
            rec.in0 = ids_.lookup(pool.getInput());
            rec.kh = (int32_t)pool.getKernel()[0];
            rec.kw = (int32_t)pool.getKernel()[1];
            rec.stride_h = (int32_t)pool.getStride()[0];
            rec.stride_w = (int32_t)pool.getStride()[1];
            rec.pad_l = (int32_t)pool.getPad()[0];
            rec.pad_r = (int32_t)pool.getPad()[1];
            rec.pad_t = (int32_t)pool.getPad()[2];
            rec.pad_b = (int32_t)pool.getPad()[3];
            rec.pad_value = -128;
            rec.out0 = ids_[pool->getResult(0)] = addValue(pool->getResult(0), TB200_TENSOR_ACTIVATION);
            writer_.addOp(rec);
            return success();
        }
        if (auto table = dyn_cast<hl::TableOp>(op)) {
            tb200_op_t rec = torq_b200::OpListWriter::blankOp(TB200_OP_TABLE);
            rec.in0 = ids_.lookup(table.getInput());
            rec.table = addConstantOperand(table.getTable());
            if (rec.table < 0) return table.emitError("the table must be a constant");
            rec.out0 = ids_[table->getResult(0)] = addValue(table->getResult(0), TB200_TENSOR_ACTIVATION);
            writer_.addOp(rec);
            return success();
        }
        if (auto id = dyn_cast<hl::IdentityOp>(op)) {
            tb200_op_t rec = torq_b200::OpListWriter::blankOp(TB200_OP_RESHAPE);
            rec.in0 = ids_.lookup(id.getInput());
            rec.out0 = ids_[id->getResult(0)] = addValue(id->getResult(0), TB200_TENSOR_ACTIVATION);
            writer_.addOp(rec);
            return success();
        }
        // add / mul / avg_pool2d / resize / transpose / reduce / ... follow the same shape: operands by id,
        // attributes copied into the record's fields named in include/torq_b200_ops.h.
        return op->emitError("torq_hl op without a torq-b200-ops record: ") << op->getName();
    }

    func::FuncOp func_;
    torq_b200::OpListWriter writer_;
    llvm::DenseMap<Value, int> ids_;
};

class TorqB200TargetBackend final : public IREE::HAL::TargetBackend {
  public:
    std::string getLegacyDefaultDeviceID() const override { return "torq_b200"; }

    void getDefaultExecutableTargets(
        MLIRContext *context, StringRef deviceID, DictionaryAttr deviceConfigAttr,
        SmallVectorImpl<IREE::HAL::ExecutableTargetAttr> &executableTargetAttrs
    ) const override {
        Builder b(context);
        // the runtime answers ("hal.executable.format", "torq-b200-ops") -> 1 (tb200_device_query_i64)
        executableTargetAttrs.push_back(IREE::HAL::ExecutableTargetAttr::get(
            context, b.getStringAttr("torq_b200"), b.getStringAttr("torq-b200-ops"), b.getDictionaryAttr({})
        ));
    }

    void getDependentDialects(DialectRegistry &registry) const override {
        registry.insert<hl::TorqHLDialect>();
    }

    void buildTranslationPassPipeline(
        IREE::HAL::ExecutableTargetAttr targetAttr, OpPassManager &passManager
    ) override {
        buildTorqHLOnlyPassPipeline(passManager);
    }

    LogicalResult serializeExecutable(
        const SerializationOptions &options, IREE::HAL::ExecutableVariantOp variantOp, OpBuilder &executableBuilder
    ) override {
        ModuleOp innerModuleOp = variantOp.getInnerModule();
        auto funcs = llvm::to_vector(innerModuleOp.getOps<func::FuncOp>());
        if (funcs.size() != 1) return variantOp.emitError("expected one dispatch function");
        std::vector<uint8_t> blob;
        if (failed(OpListEmitter(funcs.front()).run(blob))) return failure();
        auto bytes = DenseIntElementsAttr::get(
            VectorType::get({(int64_t)blob.size()}, executableBuilder.getI8Type()),
            ArrayRef<int8_t>(reinterpret_cast<const int8_t *>(blob.data()), blob.size())
        );
        auto binaryOp = IREE::HAL::ExecutableBinaryOp::create(
            executableBuilder, variantOp.getLoc(), variantOp.getSymName(), variantOp.getTarget().getFormat(), bytes
        );
        binaryOp.setMimeTypeAttr(executableBuilder.getStringAttr("application/x-torq-b200-ops"));
        return success();
    }
};

} // namespace

std::shared_ptr<IREE::HAL::TargetBackend> createBackend() { return std::make_shared<TorqB200TargetBackend>(); }

} // namespace mlir::syna::torq_b200
