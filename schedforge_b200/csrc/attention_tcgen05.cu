// Tensor-core flash-attention prefill (placeholder until the tcgen05 kernel lands: reports
// "unsupported" so that the dispatcher uses the CUDA-core kernel).
#include "common.cuh"

namespace sfb {

bool attention_prefill_tcgen05_supported(const sfb_attention_args&) { return false; }

sfb_status attention_prefill_tcgen05(const sfb_attention_args&, cudaStream_t) {
    return fail(SFB_UNSUPPORTED, "attention: tcgen05 prefill kernel not built");
}

}  // namespace sfb
