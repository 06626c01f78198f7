// Parameters and the split rule shared by the paged-decode kernels (generic CUDA-core kernel in
// attention_simt.cu, tensor-core kernel for head_dim 128 in attention_decode.cu).
#pragma once

#include "common.cuh"

namespace sfb {

// partial record per (batch, q_head, split): [max, sum, numerator[Dv]] as float32.
struct DecodeParams {
    const void *q, *k_pool, *v_pool;
    const int *block_table, *context_len;
    void* out;
    float* partials;
    int batch, q_heads, kv_heads, dim, dim_v, block_tokens, max_blocks, splits;
    float scale;
    int chunk_tokens;
    // Guards against a bad length or table entry written by an earlier kernel: a context longer than the table
    // covers is cut to context_limit, a block id outside [0, num_blocks) is skipped (its keys count as zeros);
    // either one ORs kCodeDecodeBounds into the device status word instead of touching memory out of bounds.
    int context_limit, num_blocks;
    uint32_t* status;
    int uniform_context;  // > 0: the length of every sequence (context_len is not read)
};

constexpr uint32_t kCodeDecodeBounds = 0x200;

__device__ __forceinline__ int guarded_context(const DecodeParams& p, int b) {
    int ctx = p.uniform_context > 0 ? p.uniform_context : p.context_len[b];
    if (ctx > p.context_limit || ctx < 0) {
        ctx = ctx < 0 ? 0 : p.context_limit;
        if (threadIdx.x == 0) atomicOr(p.status, kCodeDecodeBounds);
    }
    return ctx;
}

// Split s covers tokens [s*chunk, (s+1)*chunk) of every sequence (chunk is a multiple of four KV
// blocks), so all non-empty splits carry the same amount of work whatever the context length;
// splits beyond a sequence's length are empty and write a neutral partial.
__device__ __forceinline__ void split_range(int ctx, int chunk_tokens, int split, int& begin, int& end) {
    begin = min(ctx, split * chunk_tokens);
    end = min(ctx, begin + chunk_tokens);
}

constexpr int kDecodeMaxPages = 4096;  // KV blocks one split may cover (page-id list in shared memory)

// bf16, head_dim = head_dim_value = 128, 16-token blocks, group = q_heads / kv_heads <= 8.
sfb_status decode_paged_d128_launch(const DecodeParams& p, const sfb_decode_args& args, int group, cudaStream_t stream);

}  // namespace sfb
