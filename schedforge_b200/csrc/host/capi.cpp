// extern "C" plan-level entry points: thin wrappers that turn the host runtime's
// exceptions into sfb_status codes (see include/schedforge_b200.h, group 2).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <numeric>

#include "../common.cuh"
#include "decoder.hpp"

using namespace sfb;

struct sfb_decoder_plan {
    std::unique_ptr<DecoderExecutablePlan> plan;
};

namespace {

DecoderConfig to_config(const sfb_decoder_config& c) {
    DecoderConfig config;
    config.batch = c.batch; config.sequence = c.sequence; config.hidden = c.hidden;
    config.intermediate = c.intermediate; config.query_heads = c.query_heads; config.kv_heads = c.kv_heads;
    config.head_dim = c.head_dim; config.rms_epsilon = c.rms_epsilon; config.rope_theta = c.rope_theta;
    config.causal = c.causal != 0;
    config.ffn = c.ffn_moe ? DecoderFFNKind::MoE : DecoderFFNKind::Dense;
    config.experts = c.experts; config.top_k = c.top_k; config.context_sequence = c.context_sequence;
    return config;
}

void copy_text(const std::string& text, char* buffer, size_t capacity) {
    if (!buffer || capacity == 0) throw std::invalid_argument("null text buffer");
    const size_t n = std::min(capacity - 1, text.size());
    std::memcpy(buffer, text.data(), n);
    buffer[n] = '\0';
}

}  // namespace

extern "C" {

sfb_status sfb_import_stablehlo(const char* text, sfb_graph_summary* summary) {
    return guarded([&] {
        if (!text || !summary) throw std::invalid_argument("null StableHLO text or summary");
        const TensorGraph graph = StableHLOImporter{}.importText(text);
        const DecoderFusionSummary fusion = DecoderFusionPass{}.run(graph, DecoderFFNKind::Dense);
        *summary = {};
        summary->operations = static_cast<int>(graph.operations().size());
        summary->values = static_cast<int>(graph.values().size());
        for (const auto& op : graph.operations()) {
            summary->inputs += op.kind == GraphOpKind::Input;
            summary->matmuls += op.kind == GraphOpKind::MatMul;
        }
        summary->fused_qkv = fusion.fused_qkv;
        summary->fused_gate_up = fusion.fused_gate_up;
        summary->fused_rope = fusion.fused_rope;
    });
}

sfb_status sfb_import_stablehlo_dump(const char* text, char* buffer, size_t capacity) {
    return guarded([&] {
        if (!text) throw std::invalid_argument("null StableHLO text");
        copy_text(StableHLOImporter{}.importText(text).dump(), buffer, capacity);
    });
}

sfb_status sfb_decoder_compile(const sfb_decoder_config* config, const sfb_decoder_data* data,
                               const char* stablehlo_text, const sfb_compile_options* options,
                               sfb_decoder_plan** plan) {
    return guarded([&] {
        if (!config || !data || !plan) throw std::invalid_argument("null decoder compile argument");
        *plan = nullptr;
        const DecoderConfig c = to_config(*config);
        validate(c);
        sfb_compile_options opt{};
        if (options) opt = *options;
        else { opt.dtype = SFB_BF16; opt.token_major_attention = 1; opt.fuse_epilogues = 1; }
        if (opt.tp_size <= 0) opt.tp_size = 1;
        const TensorGraph imported = stablehlo_text && *stablehlo_text
            ? StableHLOImporter{}.importText(stablehlo_text) : build_decoder_layer_graph(c);
        auto owned = std::make_unique<sfb_decoder_plan>();
        owned->plan = DecoderCompiler{}.compile(imported, c, *data, opt);
        *plan = owned.release();
    });
}

sfb_status sfb_decoder_optimize(const sfb_decoder_config* config, const sfb_decoder_data* data,
                                const char* stablehlo_text, const sfb_compile_options* base_options,
                                const float* input, int measurement_budget, int repetitions,
                                sfb_optimization_result* result, sfb_plan_candidate* candidates_out, int capacity,
                                sfb_decoder_plan** plan) {
    return guarded([&] {
        if (!config || !data || !plan || !result) throw std::invalid_argument("null decoder optimize argument");
        *plan = nullptr;
        const DecoderConfig c = to_config(*config);
        validate(c);
        sfb_compile_options opt{};
        if (base_options) opt = *base_options;
        else { opt.dtype = SFB_BF16; opt.token_major_attention = 1; opt.fuse_epilogues = 1; }
        if (opt.tp_size <= 0) opt.tp_size = 1;
        const TensorGraph imported = stablehlo_text && *stablehlo_text
            ? StableHLOImporter{}.importText(stablehlo_text) : build_decoder_layer_graph(c);
        auto owned = std::make_unique<sfb_decoder_plan>();
        owned->plan = optimize_decoder_plan(imported, c, *data, opt, input, measurement_budget, repetitions, result,
                                            candidates_out, capacity);
        *plan = owned.release();
    });
}

void sfb_decoder_destroy(sfb_decoder_plan* plan) { delete plan; }

sfb_status sfb_decoder_execute_rows(sfb_decoder_plan* plan, const float* input_rows, float* output_rows, int row_begin,
                                    int row_count, sfb_decoder_result* result) {
    return guarded([&] {
        if (!plan || !plan->plan) throw std::invalid_argument("null decoder plan");
        plan->plan->execute_rows(input_rows, output_rows, row_begin, row_count, result);
    });
}

double sfb_decoder_compile_milliseconds(const sfb_decoder_plan* plan) {
    return plan && plan->plan ? plan->plan->compile_milliseconds : 0.0;
}

sfb_status sfb_decoder_execute(sfb_decoder_plan* plan, const float* input, float* output,
                               const int* trace_expert_ids, const float* trace_expert_weights,
                               const int* trace_counts, sfb_decoder_result* result) {
    return guarded([&] {
        if (!plan || !plan->plan) throw std::invalid_argument("null decoder plan");
        RoutingTraceView trace;
        trace.expert_ids = trace_expert_ids;
        trace.expert_weights = trace_expert_weights;
        trace.counts = trace_counts;
        if ((trace_expert_ids || trace_expert_weights || trace_counts) && !trace)  // a trace is all three arrays or none
            throw std::invalid_argument("routing trace does not match MoE configuration");
        if (trace && plan->plan->config.ffn != DecoderFFNKind::MoE)
            throw std::invalid_argument("routing trace does not match MoE configuration");
        plan->plan->execute(input, output, trace, result);
    });
}

sfb_status sfb_decoder_step(sfb_decoder_plan* plan, const float* input, float* output, sfb_decoder_result* result) {
    return guarded([&] {
        if (!plan || !plan->plan) throw std::invalid_argument("null decoder plan");
        plan->plan->step(input, output, result);
    });
}

sfb_status sfb_decoder_kv_info(const sfb_decoder_plan* plan, int* info, int* page_table, int table_capacity,
                               int* free_pages, int free_capacity) {
    return guarded([&] {
        if (!plan || !plan->plan) throw std::invalid_argument("null decoder plan");
        plan->plan->kv_info(info, page_table, table_capacity, free_pages, free_capacity);
    });
}

sfb_status sfb_decoder_kv_truncate(sfb_decoder_plan* plan, int new_length) {
    return guarded([&] {
        if (!plan || !plan->plan) throw std::invalid_argument("null decoder plan");
        plan->plan->kv_truncate(new_length);
    });
}

sfb_status sfb_decoder_kv_release(sfb_decoder_plan* plan, const int* pages, int count) {
    return guarded([&] {
        if (!plan || !plan->plan) throw std::invalid_argument("null decoder plan");
        plan->plan->kv_release(pages, count);
    });
}

sfb_status sfb_decoder_upload_input(sfb_decoder_plan* plan, const float* input) {
    return guarded([&] {
        if (!plan || !plan->plan) throw std::invalid_argument("null decoder plan");
        plan->plan->upload_input(input);
        cuda_check(cudaStreamSynchronize(plan->plan->stream()), "input upload sync");
    });
}

sfb_status sfb_decoder_execute_resident(sfb_decoder_plan* plan, sfb_stream stream) {
    return guarded([&] {
        if (!plan || !plan->plan) throw std::invalid_argument("null decoder plan");
        plan->plan->run(stream ? static_cast<cudaStream_t>(stream) : plan->plan->stream(), RoutingTraceView{}, false);
    });
}

sfb_status sfb_decoder_download_output(sfb_decoder_plan* plan, float* output) {
    return guarded([&] {
        if (!plan || !plan->plan) throw std::invalid_argument("null decoder plan");
        plan->plan->download_output(output);
    });
}

sfb_status sfb_decoder_set_allreduce(sfb_decoder_plan* plan, sfb_allreduce_fn fn, void* user) {
    return guarded([&] {
        if (!plan || !plan->plan) throw std::invalid_argument("null decoder plan");
        plan->plan->set_allreduce(fn, user);
    });
}

sfb_status sfb_decoder_dump(const sfb_decoder_plan* plan, char* buffer, size_t capacity) {
    return guarded([&] {
        if (!plan || !plan->plan) throw std::invalid_argument("null decoder plan");
        copy_text(plan->plan->dump(), buffer, capacity);
    });
}

int sfb_decoder_row_chunks(int rows, int hidden, int sm_count, int* blocks, int capacity) {
    const std::vector<int> sizes = sfb::pipelined_row_blocks(rows, hidden, sm_count);
    for (std::size_t i = 0; blocks && i < sizes.size() && static_cast<int>(i) < capacity; ++i) blocks[i] = sizes[i];
    return static_cast<int>(sizes.size());
}

size_t sfb_decoder_peer_bytes(const sfb_decoder_plan* plan) {
    return plan && plan->plan ? plan->plan->peer_bytes() : 0;
}

sfb_status sfb_decoder_set_peer_allreduce(sfb_decoder_plan* plan, void* local_base, void* const* peer_bases) {
    return guarded([&] {
        if (!plan || !plan->plan) throw std::invalid_argument("null decoder plan");
        plan->plan->set_peer_allreduce(local_base, peer_bases);
    });
}

sfb_status sfb_decoder_set_peer_collective(sfb_decoder_plan* plan, void* local_base, void* const* peer_bases, int mode) {
    return guarded([&] {
        if (!plan || !plan->plan) throw std::invalid_argument("null decoder plan");
        plan->plan->set_peer_allreduce(local_base, peer_bases, mode);
    });
}

size_t sfb_decoder_workspace_bytes(const sfb_decoder_plan* plan) {
    return plan && plan->plan ? plan->plan->workspace_bytes : 0;
}

sfb_status sfb_decoder_read_tensor(sfb_decoder_plan* plan, const char* name, float* host_out,
                                   int64_t capacity, int64_t* count) {
    return guarded([&] {
        if (!plan || !plan->plan || !name) throw std::invalid_argument("null decoder plan or tensor name");
        const int64_t n = plan->plan->read_tensor(name, host_out, capacity);
        if (count) *count = n;
    });
}

sfb_stream sfb_decoder_stream(sfb_decoder_plan* plan) {
    return plan && plan->plan ? plan->plan->stream() : nullptr;
}

}  // extern "C"
