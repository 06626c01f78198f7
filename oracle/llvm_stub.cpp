// TEST INFRASTRUCTURE ONLY — never linked into the product library.
//
// Link stub for the reference's three LLVM translation units (llvm_backend.cpp,
// attention_llvm_backend.cpp, aot_runtime.cpp), which need libLLVM-18 and are
// therefore left out of the oracle build.  The decoder hot path only calls
// LLVMJITBackend::benchmark at plan-build time to attach text artifacts; the
// executed kernels are the reference's native AVX2 C++ loops, so an empty
// result changes no arithmetic.
#include "schedforge/attention_compiler.h"
#include "schedforge/compiler.h"

#include <stdexcept>

namespace schedforge {

bool LLVMJITBackend::available() const { return false; }

LLVMJITResult LLVMJITBackend::benchmark(const LoopIR&, const TensorData&, int, int) const {
    return {};
}

bool LLVMAOTBackend::available() const { return false; }

AOTObject LLVMAOTBackend::compile(const LoopIR&) const {
    throw std::runtime_error("LLVM AOT backend is not part of the oracle build");
}

FusedAttentionLLVMResult execute_fused_attention_llvm(const AttentionExecutablePlan&,
                                                      const AttentionData&, int, int) {
    throw std::runtime_error("LLVM fused attention is not part of the oracle build");
}

}  // namespace schedforge
