// --lower-qf-to-runtime written against the MLIR C++ API, for a QuantForge tree that is built with MLIR/LLVM.
//
// NOT COMPILED IN THIS REPOSITORY: the build hosts have no MLIR installation. The text-level driver
// (../quantforge_opt.cpp) implements the same rewrite and is what the tests exercise; this file is the form a
// maintainer of the reference would add: put it in lib/Transforms/, list it in lib/Transforms/CMakeLists.txt, and
// declare the create/register pair next to the others (include/QuantForge/Transforms/Passes.h:173-198).
//
// Rewrite (per module, because it adds private declarations):
//   %u = qf.unpack %w                       : tensor<KxNxi8> -> tensor<KxNxi8>       (or the doubling form)
//   %d = qf.dequant %u, %scale, %zp {attrs} : ... -> tensor<KxNxf16>
//   %y = linalg.matmul ins(%x, %d) outs(%init)
// becomes
//   %y = func.call @qf_w4a16_linear_m<M>_k<K>_n<N>(%x, %w, %scale, %zp, %init)
//            {group_size = ..., qf.weight_orientation = "kn"}
// with `func.func private @qf_w4a16_linear_m.._k.._n..(...) attributes {qf.runtime_symbol = "qf_w4a16_linear"}`.
// A qf.dequant(qf.unpack) without a matmul user becomes @qf_dequant_w4_<rows>x<cols>, a lone qf.unpack becomes
// @qf_unpack_int4_<rows>x<cols>. Any qf op that is left fails the pass: the runtime has no CPU evaluation of the
// dialect to fall back to. Bufferisation later turns the tensor operands into the bare pointers of
// include/quantforge_rt.h (the reference lowers with the bare-pointer convention, lib/Transforms/LowerToNVVMPass.cpp:55).
#include "QuantForge/Dialect/QuantForge/QuantForgeDialect.h"
#include "QuantForge/Dialect/QuantForge/QuantForgeOps.h"
#include "QuantForge/Transforms/Passes.h"

#include "mlir/Dialect/Func/IR/FuncOps.h"
#include "mlir/Dialect/Linalg/IR/Linalg.h"
#include "mlir/IR/Builders.h"
#include "mlir/IR/BuiltinOps.h"
#include "mlir/Pass/Pass.h"
#include "llvm/ADT/SetVector.h"
#include "llvm/ADT/SmallVector.h"
#include "llvm/ADT/Twine.h"

using namespace mlir;

namespace {

// Declares (once) the private function a call site binds to and returns its symbol.
FlatSymbolRefAttr declareRuntimeFunction(ModuleOp module, StringRef symbol, StringRef entryPoint, TypeRange inputs,
                                         TypeRange results) {
    MLIRContext *ctx = module.getContext();
    if (!module.lookupSymbol<func::FuncOp>(symbol)) {
        OpBuilder b(module.getBodyRegion());
        auto fn = b.create<func::FuncOp>(module.getLoc(), symbol, FunctionType::get(ctx, inputs, results));
        fn.setPrivate();
        fn->setAttr("qf.runtime_symbol", StringAttr::get(ctx, entryPoint));
    }
    return FlatSymbolRefAttr::get(ctx, symbol);
}

std::string shapeSuffix(RankedTensorType t) {
    std::string s;
    for (int64_t d : t.getShape()) s += (s.empty() ? "" : "x") + std::to_string(d);
    return s;
}

// Attributes of the dequant op travel to the call (group_size, zero_mode, zero_const, out_dtype); a missing
// group_size means one group spanning K.
SmallVector<NamedAttribute> callAttributes(quantforge::DequantOp dq, bool weightIsKN) {
    MLIRContext *ctx = dq.getContext();
    SmallVector<NamedAttribute> attrs(dq->getAttrs().begin(), dq->getAttrs().end());
    if (!dq->hasAttr("group_size"))
        attrs.emplace_back(StringAttr::get(ctx, "group_size"), IntegerAttr::get(IntegerType::get(ctx, 64), 0));
    if (weightIsKN) attrs.emplace_back(StringAttr::get(ctx, "qf.weight_orientation"), StringAttr::get(ctx, "kn"));
    return attrs;
}

struct LowerQFToRuntimePass : public PassWrapper<LowerQFToRuntimePass, OperationPass<ModuleOp>> {
    MLIR_DEFINE_EXPLICIT_INTERNAL_INLINE_TYPE_ID(LowerQFToRuntimePass)

    StringRef getArgument() const final { return "lower-qf-to-runtime"; }
    StringRef getDescription() const final {
        return "Replace matmul(x, qf.dequant(qf.unpack(w))) and lone qf ops by calls into the QuantForge runtime";
    }
    void getDependentDialects(DialectRegistry &registry) const override { registry.insert<func::FuncDialect>(); }

    void runOnOperation() override {
        ModuleOp module = getOperation();
        llvm::SetVector<Operation *> dead;  // each op once, in consumer-before-producer order

        // 1. the contraction: matmul whose B operand is dequant(unpack(w))
        module.walk([&](linalg::MatmulOp mm) {
            auto dq = mm.getInputs()[1].getDefiningOp<quantforge::DequantOp>();
            auto up = dq ? dq.getInput().getDefiningOp<quantforge::UnpackOp>() : quantforge::UnpackOp();
            auto xTy = dyn_cast<RankedTensorType>(mm.getInputs()[0].getType());
            auto wTy = dq ? dyn_cast<RankedTensorType>(dq.getOutput().getType()) : RankedTensorType();
            if (!up || !xTy || !wTy || xTy.getRank() != 2 || wTy.getRank() != 2 || !xTy.hasStaticShape() ||
                !wTy.hasStaticShape())
                return;
            SmallVector<Value> operands = {mm.getInputs()[0], up.getInput(), dq.getScale(), dq.getZeroPoint(),
                                           mm.getOutputs()[0]};
            SmallVector<Type> operandTypes;
            for (Value v : operands) operandTypes.push_back(v.getType());
            std::string symbol = ("qf_w4a16_linear_m" + Twine(xTy.getDimSize(0)) + "_k" + Twine(wTy.getDimSize(0)) +
                                  "_n" + Twine(wTy.getDimSize(1))).str();
            FlatSymbolRefAttr callee =
                declareRuntimeFunction(module, symbol, "qf_w4a16_linear", operandTypes, mm->getResultTypes());
            OpBuilder b(mm);
            auto call = b.create<func::CallOp>(mm.getLoc(), callee, mm->getResultTypes(), operands);
            for (NamedAttribute a : callAttributes(dq, /*weightIsKN=*/true)) call->setAttr(a.getName(), a.getValue());
            mm->replaceAllUsesWith(call);
            dead.insert(mm);
            dead.insert(dq);
            dead.insert(up);
        });
        eraseIfUnused(dead);

        // 2. dequant(unpack) that did not feed a matmul, then lone unpacks
        dead.clear();
        module.walk([&](quantforge::DequantOp dq) {
            auto up = dq.getInput().getDefiningOp<quantforge::UnpackOp>();
            auto inTy = up ? dyn_cast<RankedTensorType>(up.getInput().getType()) : RankedTensorType();
            if (!up || !inTy || !inTy.hasStaticShape()) return;
            SmallVector<Value> operands = {up.getInput(), dq.getScale(), dq.getZeroPoint()};
            SmallVector<Type> operandTypes;
            for (Value v : operands) operandTypes.push_back(v.getType());
            FlatSymbolRefAttr callee = declareRuntimeFunction(module, "qf_dequant_w4_" + shapeSuffix(inTy),
                                                              "qf_dequant_w4", operandTypes, dq->getResultTypes());
            OpBuilder b(dq);
            auto call = b.create<func::CallOp>(dq.getLoc(), callee, dq->getResultTypes(), operands);
            for (NamedAttribute a : callAttributes(dq, false)) call->setAttr(a.getName(), a.getValue());
            dq->replaceAllUsesWith(call);
            dead.insert(dq);
            dead.insert(up);
        });
        eraseIfUnused(dead);
        dead.clear();
        module.walk([&](quantforge::UnpackOp up) {
            auto inTy = dyn_cast<RankedTensorType>(up.getInput().getType());
            if (!inTy || !inTy.hasStaticShape()) return;
            FlatSymbolRefAttr callee = declareRuntimeFunction(module, "qf_unpack_int4_" + shapeSuffix(inTy),
                                                              "qf_unpack_int4", up.getInput().getType(),
                                                              up->getResultTypes());
            OpBuilder b(up);
            auto call = b.create<func::CallOp>(up.getLoc(), callee, up->getResultTypes(), ValueRange{up.getInput()});
            up->replaceAllUsesWith(call);
            dead.insert(up);
        });
        eraseIfUnused(dead);

        // 3. nothing evaluates the dialect on the host: whatever is left is an error
        bool left = false;
        module.walk([&](Operation *op) {
            if (op->getDialect() && op->getDialect()->getNamespace() == "qf") {
                op->emitError("cannot be lowered to a runtime call (no CPU fallback exists)");
                left = true;
            }
        });
        if (left) signalPassFailure();
    }

    // Erases the collected ops that lost their last user, consumers before producers.
    static void eraseIfUnused(const llvm::SetVector<Operation *> &ops) {
        for (Operation *op : ops)
            if (op->use_empty()) op->erase();
    }
};

}  // namespace

std::unique_ptr<Pass> mlir::quantforge::createLowerQFToRuntimePass() { return std::make_unique<LowerQFToRuntimePass>(); }
void mlir::quantforge::registerLowerQFToRuntimePass() { PassRegistration<LowerQFToRuntimePass>(); }
