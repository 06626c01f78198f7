// Decoder layer compiler + runtime on the host: the counterpart of the reference's
// DecoderCompiler::compile / execute_decoder_layer (include/schedforge/decoder_compiler.h:
// 17-138, 205-223; src/decoder_compiler.cpp:218-304, 518-620) with the same configuration
// fields, the same validation and fusion requirements and the same stage accounting, but
// with every weight resident in device memory and every stage a CUDA kernel entry point.
#pragma once

#include <memory>
#include <string>
#include <vector>

#include "graph.hpp"
#include "runtime.hpp"

namespace sfb {

struct DecoderConfig {
    int batch = 1;
    int sequence = 16;
    int hidden = 64;
    int intermediate = 128;
    int query_heads = 4;
    int kv_heads = 2;
    int head_dim = 16;
    float rms_epsilon = 1.0e-5F;
    float rope_theta = 10000.0F;
    bool causal = true;
    DecoderFFNKind ffn = DecoderFFNKind::Dense;
    int experts = 4;
    int top_k = 2;
    int context_sequence = 0;
    int rows() const { return batch * sequence; }
    int kv_width() const { return kv_heads * head_dim; }
    int qkv_width() const { return hidden + 2 * kv_width(); }
};

// Throws std::invalid_argument with the reference's messages (src/decoder_compiler.cpp:26-39).
void validate(const DecoderConfig& config);

// Canonical 23-operation layer graph written into the plan dump
// (build_decoder_layer_graph, src/decoder_compiler.cpp:412-481).
TensorGraph build_decoder_layer_graph(const DecoderConfig& config);

struct DecoderPlanPolicy {
    bool token_major_attention = true;
    bool fuse_epilogues = true;
    bool reuse_workspace = true;
    int gemm_backend = SFB_GEMM_AUTO;
    int attention_backend = 0;
    std::string dump() const;
};

struct DecoderConstant {
    std::string name;
    std::vector<int> logical_shape, packed_shape;
    std::string layout;
    std::size_t bytes = 0;
    std::string dump() const;
};

struct RoutingTraceView {
    const int* expert_ids = nullptr;
    const float* expert_weights = nullptr;
    const int* counts = nullptr;
    explicit operator bool() const { return expert_ids && expert_weights && counts; }
};

class DecoderExecutablePlan {
public:
    ~DecoderExecutablePlan();
    DecoderConfig config;        // the FULL (unsharded) layer
    sfb_compile_options options{};
    DecoderPlanPolicy policy;
    TensorGraph imported_graph, graph;
    DecoderFusionSummary fusion;
    std::vector<DecoderConstant> constants;
    std::size_t naive_bytes = 0, workspace_bytes = 0, weight_bytes = 0;
    double compile_milliseconds = 0.0;
    std::string attention_strategy;  // "io_aware" | "split_kv_decode"

    // One layer pass.  input/output: host float32 [T, H].
    void execute(const float* input, float* output, RoutingTraceView trace, sfb_decoder_result* result);
    void execute_pipelined(const float* input, float* output, sfb_decoder_result* result);
    void execute_rows(const float* input_rows, float* output_rows, int row_begin, int row_count, sfb_decoder_result* result);
    // Autoregressive decode loop on a plan compiled with append_new_token: one pass that appends the new token's
    // K/V at the cache length, attends over length + 1 keys and then advances the length (taking a page from the
    // back of the free list when the token opens one), plus the reference's page accounting calls
    // (append_paged_kv / truncate_paged_kv / release_paged_kv_pages, src/next_milestones.cpp:486-550).
    void step(const float* input, float* output, sfb_decoder_result* result);
    void kv_info(int* info, int* page_table, int table_capacity, int* free_pages, int free_capacity) const;
    void kv_truncate(int new_length);
    void kv_release(const int* pages, int count);
    void upload_input(const float* input);
    void run(cudaStream_t stream, RoutingTraceView trace, bool stage_events);
    void download_output(float* output);
    void set_allreduce(sfb_allreduce_fn fn, void* user) { allreduce_ = fn; allreduce_user_ = user; }
    // Fused all-reduce over peer memory for the O and Down projections of a sharded plan.
    std::size_t peer_bytes() const;
    // mode: 0 = pick, 1 = one-shot (every rank pushes its whole partial tensor to every peer), 2 = two-shot
    // (reduce-scatter under the GEMM, sum + all-gather by the row owners)
    void set_peer_allreduce(void* local_base, void* const* peer_bases, int mode = 1);
    std::string dump() const;
    // Copies the named intermediate to the host as float32; returns the element count.
    int64_t read_tensor(const std::string& name, float* host_out, int64_t capacity);
    cudaStream_t stream() const { return stream_; }

private:
    friend class DecoderCompiler;
    struct Impl;
    std::unique_ptr<Impl> impl_;
    cudaStream_t stream_ = nullptr;
    sfb_allreduce_fn allreduce_ = nullptr;
    void* allreduce_user_ = nullptr;
};

// ExecutablePlanOptimizer::optimize on the GPU (optimizer.cpp); returns the winning plan.
std::unique_ptr<DecoderExecutablePlan> optimize_decoder_plan(
    const TensorGraph& graph, const DecoderConfig& config, const sfb_decoder_data& data, const sfb_compile_options& base,
    const float* input, int measurement_budget, int repetitions, sfb_optimization_result* result,
    sfb_plan_candidate* candidates_out, int capacity);

// Row chunks (in blocks of 128 rows) that sfb_decoder_execute pipelines a dense causal prefill pass in; empty when
// the shape takes none.  Pure arithmetic (decoder.cpp).
std::vector<int> pipelined_row_blocks(int rows, int hidden, int sms);

class DecoderCompiler {
public:
    // Throws std::invalid_argument for an invalid configuration or missing fusion patterns.
    std::unique_ptr<DecoderExecutablePlan> compile(const TensorGraph& imported_graph, const DecoderConfig& config,
                                                   const sfb_decoder_data& data, const sfb_compile_options& options) const;
};

}  // namespace sfb
