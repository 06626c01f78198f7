// TEST INFRASTRUCTURE ONLY — never linked into the product library.
//
// C-ABI harness around the UNMODIFIED reference sources, compiled where they
// lie (the Makefile passes -I<reference> and lists <reference>/src/*.cpp; no
// reference source is copied).  It exists so that the Python tests and the
// CPU-baseline leg of bench.py can drive the reference's own implementation
// of the decoder-layer hot path: plan build + native execution, the scalar
// layer reference, the attention / paged-KV / MoE sub-entry points, and the
// StableHLO importer with the decoder fusion pass.
//
// This translation unit textually includes the reference's
// src/decoder_compiler.cpp so that the functions it keeps in an anonymous
// namespace (execute_once, rms_norm, split_qkv, swiglu, ...) are reachable:
// execute_decoder_layer() itself always runs the scalar layer reference
// afterwards, which takes hours at Llama-3-8B shapes.
#include "src/decoder_compiler.cpp"  // NOLINT: resolved through -I<reference root>

#include "schedforge/next_milestones.h"

#include <cstring>
#include <filesystem>
#include <fstream>
#include <sstream>
#include <memory>
#include <string>

namespace {

thread_local std::string g_error;

template <class F>
int guarded(F&& body) {
    try {
        body();
        return 0;
    } catch (const std::invalid_argument& error) {
        g_error = error.what();
        return 1;
    } catch (const std::exception& error) {
        g_error = error.what();
        return 2;
    }
}

std::vector<float> vec(const float* data, std::size_t count) {
    return data ? std::vector<float>(data, data + count) : std::vector<float>{};
}

void out(const std::vector<float>& values, float* destination) {
    if (destination && !values.empty())
        std::memcpy(destination, values.data(), values.size() * sizeof(float));
}

}  // namespace

extern "C" {

struct sfref_decoder_config {
    int batch, sequence, hidden, intermediate, query_heads, kv_heads, head_dim;
    float rms_epsilon, rope_theta;
    int causal, ffn_moe, experts, top_k, context_sequence;
};

struct sfref_decoder_data {
    const float* input;
    const float* rms1_weight;
    const float* query_weight;
    const float* key_weight;
    const float* value_weight;
    const float* output_weight;
    const float* rms2_weight;
    const float* gate_weight;
    const float* up_weight;
    const float* down_weight;
    const float* router_weight;
    const float* w1;
    const float* w3;
    const float* w2;
    const float* cached_key;
    const float* cached_value;
    // optional routing trace (all three non-null to use it)
    const int* trace_expert_ids;
    const float* trace_expert_weights;
    const int* trace_counts;
};

struct sfref_attention_config {
    int batch, query_heads, kv_heads, sequence_query, sequence_kv, head_dim, head_dim_value;
    int causal;
    float scale;
};

struct sfref_moe_config {
    int tokens, hidden, intermediate, experts, top_k;
};

const char* sfref_last_error() { return g_error.c_str(); }

int sfref_hardware_threads() { return schedforge::TargetInfo::detect().logical_cpus; }

}  // extern "C"

namespace {

schedforge::DecoderConfig to_config(const sfref_decoder_config& c) {
    schedforge::DecoderConfig config;
    config.batch = c.batch;
    config.sequence = c.sequence;
    config.hidden = c.hidden;
    config.intermediate = c.intermediate;
    config.query_heads = c.query_heads;
    config.kv_heads = c.kv_heads;
    config.head_dim = c.head_dim;
    config.rms_epsilon = c.rms_epsilon;
    config.rope_theta = c.rope_theta;
    config.causal = c.causal != 0;
    config.ffn = c.ffn_moe ? schedforge::DecoderFFNKind::MoE : schedforge::DecoderFFNKind::Dense;
    config.experts = c.experts;
    config.top_k = c.top_k;
    config.context_sequence = c.context_sequence;
    return config;
}

schedforge::AttentionConfig to_config(const sfref_attention_config& c) {
    return {c.batch, c.query_heads, c.kv_heads, c.sequence_query, c.sequence_kv,
            c.head_dim, c.head_dim_value, c.causal != 0, c.scale};
}

schedforge::MoeConfig to_config(const sfref_moe_config& c) {
    return {c.tokens, c.hidden, c.intermediate, c.experts, c.top_k};
}

schedforge::DecoderData to_data(const schedforge::DecoderConfig& config,
                                const sfref_decoder_data& d) {
    using std::size_t;
    const size_t t = static_cast<size_t>(config.batch) * config.sequence;
    const size_t h = config.hidden, i = config.intermediate;
    const size_t kv = static_cast<size_t>(config.kv_heads) * config.head_dim;
    schedforge::DecoderData data;
    data.input = vec(d.input, t * h);
    data.rms1_weight = vec(d.rms1_weight, h);
    data.query_weight = vec(d.query_weight, h * h);
    data.key_weight = vec(d.key_weight, h * kv);
    data.value_weight = vec(d.value_weight, h * kv);
    data.output_weight = vec(d.output_weight, h * h);
    data.rms2_weight = vec(d.rms2_weight, h);
    if (config.ffn == schedforge::DecoderFFNKind::Dense) {
        data.gate_weight = vec(d.gate_weight, h * i);
        data.up_weight = vec(d.up_weight, h * i);
        data.down_weight = vec(d.down_weight, i * h);
    } else {
        const size_t e = config.experts;
        data.moe.input = data.input;
        data.moe.router_weight = vec(d.router_weight, h * e);
        data.moe.w1 = vec(d.w1, e * h * i);
        data.moe.w3 = vec(d.w3, e * h * i);
        data.moe.w2 = vec(d.w2, e * i * h);
        if (d.trace_expert_ids && d.trace_expert_weights && d.trace_counts) {
            schedforge::RoutingTrace trace;
            trace.tokens = static_cast<int>(t);
            trace.experts = config.experts;
            trace.top_k = config.top_k;
            trace.expert_ids.assign(d.trace_expert_ids, d.trace_expert_ids + t * config.top_k);
            trace.expert_weights.assign(d.trace_expert_weights,
                                        d.trace_expert_weights + t * config.top_k);
            trace.counts.assign(d.trace_counts, d.trace_counts + e);
            data.routing_trace = std::move(trace);
        }
    }
    if (config.context_sequence > 0) {
        const size_t cached = static_cast<size_t>(config.batch) * config.kv_heads *
                              config.context_sequence * config.head_dim;
        data.cached_key = vec(d.cached_key, cached);
        data.cached_value = vec(d.cached_value, cached);
    }
    return data;
}

schedforge::RoutingTrace to_trace(const schedforge::MoeConfig& config, int tokens,
                                  const int* ids, const float* weights, const int* counts) {
    schedforge::RoutingTrace trace;
    trace.tokens = tokens;
    trace.experts = config.experts;
    trace.top_k = config.top_k;
    const std::size_t n = static_cast<std::size_t>(tokens) * config.top_k;
    trace.expert_ids.assign(ids, ids + n);
    trace.expert_weights.assign(weights, weights + n);
    trace.counts.assign(counts, counts + config.experts);
    return trace;
}

schedforge::MoeData to_moe_data(const schedforge::MoeConfig& config, const float* router,
                                const float* w1, const float* w3, const float* w2) {
    const std::size_t h = config.hidden, i = config.intermediate, e = config.experts;
    schedforge::MoeData data;
    data.router_weight = vec(router, h * e);
    data.w1 = vec(w1, e * h * i);
    data.w3 = vec(w3, e * h * i);
    data.w2 = vec(w2, e * i * h);
    return data;
}

struct DecoderHandle {
    schedforge::DecoderConfig config;
    schedforge::DecoderData data;
    schedforge::DecoderExecutablePlan plan;
};

struct PagedHandle {
    schedforge::PagedKVCache cache;
};

}  // namespace

extern "C" {

// ---- fixtures: the reference's own seeded generators (mt19937 + uniform) ----
// Buffers that do not apply to the configuration may be null.
int sfref_make_decoder_data(const sfref_decoder_config* c, unsigned seed,
                            float* input, float* rms1, float* wq, float* wk, float* wv,
                            float* wo, float* rms2, float* wg, float* wu, float* wd,
                            float* router, float* w1, float* w3, float* w2,
                            float* cached_key, float* cached_value) {
    return guarded([&] {
        const auto data = schedforge::make_decoder_data(to_config(*c), seed);
        out(data.input, input);
        out(data.rms1_weight, rms1);
        out(data.query_weight, wq);
        out(data.key_weight, wk);
        out(data.value_weight, wv);
        out(data.output_weight, wo);
        out(data.rms2_weight, rms2);
        out(data.gate_weight, wg);
        out(data.up_weight, wu);
        out(data.down_weight, wd);
        out(data.moe.router_weight, router);
        out(data.moe.w1, w1);
        out(data.moe.w3, w3);
        out(data.moe.w2, w2);
        out(data.cached_key, cached_key);
        out(data.cached_value, cached_value);
    });
}

int sfref_make_attention_data(const sfref_attention_config* c, unsigned seed,
                              float* query, float* key, float* value) {
    return guarded([&] {
        const auto data = schedforge::make_attention_data(to_config(*c), seed);
        out(data.query, query);
        out(data.key, key);
        out(data.value, value);
    });
}

int sfref_make_moe_data(const sfref_moe_config* c, unsigned seed, float* input,
                        float* router, float* w1, float* w3, float* w2) {
    return guarded([&] {
        const auto data = schedforge::make_moe_data(to_config(*c), seed);
        out(data.input, input);
        out(data.router_weight, router);
        out(data.w1, w1);
        out(data.w3, w3);
        out(data.w2, w2);
    });
}

void sfref_round_bf16(float* values, long long count) {
    std::vector<float> input(values, values + count);
    const auto rounded = schedforge::convert_from_bf16(schedforge::convert_to_bf16(input));
    std::memcpy(values, rounded.data(), static_cast<std::size_t>(count) * sizeof(float));
}

// ---- importer + fusion pass ------------------------------------------------
// flags[0..2] = fused_qkv, fused_gate_up, fused_rope; counts[0] = operations,
// counts[1] = values, counts[2] = graph inputs, counts[3] = MatMul ops.
int sfref_import_stablehlo(const char* text, int ffn_moe, int* flags, int* counts) {
    return guarded([&] {
        const auto graph = schedforge::StableHLOImporter{}.importText(text);
        const auto fusion = schedforge::DecoderFusionPass{}.run(
            graph, ffn_moe ? schedforge::DecoderFFNKind::MoE : schedforge::DecoderFFNKind::Dense);
        flags[0] = fusion.fused_qkv;
        flags[1] = fusion.fused_gate_up;
        flags[2] = fusion.fused_rope;
        int inputs = 0, matmuls = 0;
        for (const auto& operation : graph.operations()) {
            if (operation.kind == schedforge::GraphOpKind::Input) ++inputs;
            if (operation.kind == schedforge::GraphOpKind::MatMul) ++matmuls;
        }
        counts[0] = static_cast<int>(graph.operations().size());
        counts[1] = static_cast<int>(graph.values().size());
        counts[2] = inputs;
        counts[3] = matmuls;
    });
}

// Writes the canonical decoder graph's operation names, '\n'-separated.
int sfref_canonical_graph_names(const sfref_decoder_config* c, char* buffer, int capacity) {
    return guarded([&] {
        const auto graph = schedforge::build_decoder_layer_graph(to_config(*c));
        std::string names;
        for (const auto& operation : graph.operations()) names += operation.name + "\n";
        std::snprintf(buffer, static_cast<std::size_t>(capacity), "%s", names.c_str());
    });
}

// ---- decoder layer -----------------------------------------------------------
void* sfref_decoder_create(const sfref_decoder_config* c, const sfref_decoder_data* d,
                           const char* stablehlo_text, int threads) {
    DecoderHandle* handle = nullptr;
    const int status = guarded([&] {
        auto owned = std::make_unique<DecoderHandle>();
        owned->config = to_config(*c);
        owned->data = to_data(owned->config, *d);
        const auto imported = stablehlo_text && *stablehlo_text
            ? schedforge::StableHLOImporter{}.importText(stablehlo_text)
            : schedforge::build_decoder_layer_graph(owned->config);
        schedforge::DecoderCompileOptions options;
        options.max_threads = threads > 0 ? threads : sfref_hardware_threads();
        options.emit_llvm = false;
        owned->plan = schedforge::DecoderCompiler{}.compile(imported, owned->config,
                                                            owned->data, options);
        handle = owned.release();
    });
    return status == 0 ? handle : nullptr;
}

void sfref_decoder_destroy(void* handle) { delete static_cast<DecoderHandle*>(handle); }

// One pass of the reference's native (AVX2 + threads) layer path.
// stage_ms[0..5] = total, attention, projection, norm_rope, ffn, residual.
int sfref_decoder_execute_once(void* handle, float* output, double* stage_ms) {
    return guarded([&] {
        auto* h = static_cast<DecoderHandle*>(handle);
        const auto result = schedforge::execute_once(h->plan, h->data);
        out(result.output, output);
        if (stage_ms) {
            stage_ms[0] = result.milliseconds;
            stage_ms[1] = result.attention_milliseconds;
            stage_ms[2] = result.projection_milliseconds;
            stage_ms[3] = result.norm_rope_milliseconds;
            stage_ms[4] = result.ffn_milliseconds;
            stage_ms[5] = result.residual_milliseconds;
        }
    });
}

// attention strategy selected by the plan (enum value) and its split_kv.
int sfref_decoder_plan_info(void* handle, int* strategy, int* split_kv, long long* workspace) {
    return guarded([&] {
        auto* h = static_cast<DecoderHandle*>(handle);
        *strategy = static_cast<int>(h->plan.attention.plan.strategy);
        *split_kv = h->plan.attention.plan.split_kv;
        *workspace = static_cast<long long>(h->plan.memory.workspace_bytes);
    });
}

// The scalar layer reference (ground truth of the reference's own tests).
int sfref_decoder_reference(void* handle, float* output) {
    return guarded([&] {
        auto* h = static_cast<DecoderHandle*>(handle);
        out(schedforge::reference_decoder_layer(h->config, h->data), output);
    });
}

// The reference's weight-only INT8 layer: quantize_decoder_weights + execute_quantized_decoder_layer
// (src/next_milestones.cpp:660-697), one pass; max_error is against its scalar layer reference.
int sfref_decoder_quantized(void* handle, int per_channel, float* output, double* max_error) {
    return guarded([&] {
        auto* h = static_cast<DecoderHandle*>(handle);
        const auto weights = schedforge::quantize_decoder_weights(h->config, h->data, per_channel != 0);
        const auto result = schedforge::execute_quantized_decoder_layer(h->config, h->data, weights, 0, 1);
        out(result.output, output);
        if (max_error) *max_error = result.max_error;
    });
}

// ---- pieces of the layer (anonymous-namespace functions of the reference) ---
int sfref_rms_norm(const float* input, const float* weight, int rows, int width,
                   float epsilon, float* output) {
    return guarded([&] {
        out(schedforge::rms_norm(vec(input, static_cast<std::size_t>(rows) * width),
                                 vec(weight, width), rows, width, epsilon), output);
    });
}

int sfref_split_qkv_rope(const sfref_decoder_config* c, const float* fused,
                         float* query, float* key, float* value) {
    return guarded([&] {
        const auto config = to_config(*c);
        const std::size_t count = static_cast<std::size_t>(schedforge::rows(config)) * schedforge::qkv_width(config);
        const auto split = schedforge::split_qkv(config, vec(fused, count));
        out(split.query, query);
        out(split.key, key);
        out(split.value, value);
    });
}

int sfref_swiglu(const float* gate_up, int rows, int intermediate, float* output) {
    return guarded([&] {
        out(schedforge::swiglu(vec(gate_up, static_cast<std::size_t>(rows) * 2 * intermediate),
                               rows, intermediate), output);
    });
}

// The GEMM the decoder calls: execute(LoopIR) with the decoder schedule.
int sfref_gemm_native(int m, int n, int k, const float* a, const float* b, float* c,
                      int threads) {
    return guarded([&] {
        schedforge::DecoderPlanPolicy policy;
        auto target = schedforge::TargetInfo::detect();
        policy.threads = std::clamp(threads > 0 ? threads : target.logical_cpus, 1,
                                    target.logical_cpus);
        const auto loop = schedforge::apply_schedule({m, n, k, false, false},
                                                     schedforge::decoder_schedule(target, policy));
        std::vector<float> output;
        schedforge::execute(loop, {vec(a, static_cast<std::size_t>(m) * k),
                                   vec(b, static_cast<std::size_t>(k) * n), {}, {}, {}}, output);
        out(output, c);
    });
}

int sfref_scalar_matmul(int m, int n, int k, const float* a, const float* b, float* c) {
    return guarded([&] {
        out(schedforge::scalar_matmul(vec(a, static_cast<std::size_t>(m) * k),
                                      vec(b, static_cast<std::size_t>(k) * n), m, n, k), c);
    });
}

// ---- attention ----------------------------------------------------------------
namespace {
schedforge::AttentionData attention_data(const schedforge::AttentionConfig& config,
                                         const float* q, const float* k, const float* v) {
    const std::size_t b = config.batch;
    schedforge::AttentionData data;
    data.query = vec(q, b * config.query_heads * config.sequence_query * config.head_dim);
    data.key = vec(k, b * config.kv_heads * config.sequence_kv * config.head_dim);
    data.value = vec(v, b * config.kv_heads * config.sequence_kv * config.head_dim_value);
    return data;
}
}  // namespace

int sfref_reference_attention(const sfref_attention_config* c, const float* q,
                              const float* k, const float* v, float* output) {
    return guarded([&] {
        const auto config = to_config(*c);
        out(schedforge::reference_attention(config, attention_data(config, q, k, v)), output);
    });
}

// strategy < 0: let select_attention_plan choose.  query_tile/kv_tile <= 0 keep the
// planner's choice.  Returns the strategy actually used through *used_strategy.
int sfref_execute_attention(const sfref_attention_config* c, int strategy, int query_tile,
                            int kv_tile, int threads, const float* q, const float* k,
                            const float* v, float* output, double* milliseconds,
                            int* used_strategy) {
    return guarded([&] {
        const auto config = to_config(*c);
        const auto target = schedforge::TargetInfo::detect();
        auto options = schedforge::select_attention_plan(
            config, target, threads > 0 ? threads : target.logical_cpus);
        if (strategy >= 0)
            options.strategy = static_cast<schedforge::AttentionLoweringStrategy>(strategy);
        if (query_tile > 0) options.schedule.query_tile = query_tile;
        if (kv_tile > 0) options.schedule.kv_tile = kv_tile;
        const auto plan = schedforge::AttentionCompiler{target}.compile(config, options);
        const auto result = schedforge::execute_attention(
            plan, attention_data(config, q, k, v), 0, 1, false);
        out(result.output, output);
        if (milliseconds) *milliseconds = result.p50_milliseconds;
        if (used_strategy) *used_strategy = static_cast<int>(plan.plan.strategy);
    });
}

// Contiguous KV cache decode: appends `length` cached tokens in `appends` equal
// or ragged chunks (chunk sizes in append_tokens) and runs split-KV decode.
int sfref_decode_attention(const sfref_attention_config* c, int capacity, const float* query,
                           const float* keys, const float* values, int length, int threads,
                           float* output, int* used_split_kv) {
    return guarded([&] {
        const auto config = to_config(*c);
        const auto target = schedforge::TargetInfo::detect();
        const auto options = schedforge::select_attention_plan(
            config, target, threads > 0 ? threads : target.logical_cpus);
        const auto plan = schedforge::AttentionCompiler{target}.compile(config, options);
        auto cache = schedforge::make_kv_cache(config, capacity);
        const std::size_t b = config.batch;
        schedforge::append_kv(cache, vec(keys, b * config.kv_heads * length * config.head_dim),
                              vec(values, b * config.kv_heads * length * config.head_dim_value),
                              length);
        const auto result = schedforge::execute_decode_attention(
            plan, vec(query, b * config.query_heads * config.sequence_query * config.head_dim),
            cache, 0, 1, false);
        out(result.output, output);
        if (used_split_kv)
            *used_split_kv = config.sequence_kv > 0
                ? std::clamp(std::max(2, length / 128), 2, std::max(2, plan.plan.schedule.threads))
                : 1;
    });
}

// ---- paged KV cache -------------------------------------------------------------
void* sfref_paged_create(int batch, int kv_heads, int head_dim, int head_dim_value,
                         int page_tokens, int capacity) {
    PagedHandle* handle = nullptr;
    const int status = guarded([&] {
        auto owned = std::make_unique<PagedHandle>();
        owned->cache = schedforge::make_paged_kv_cache(
            {batch, kv_heads, head_dim, head_dim_value, page_tokens, capacity});
        handle = owned.release();
    });
    return status == 0 ? handle : nullptr;
}

void sfref_paged_destroy(void* handle) { delete static_cast<PagedHandle*>(handle); }

// Overwrites the allocator's free list (public field of the reference struct);
// pages are handed out from the back.
int sfref_paged_set_free_pages(void* handle, const int* pages, int count) {
    return guarded([&] {
        static_cast<PagedHandle*>(handle)->cache.free_pages.assign(pages, pages + count);
    });
}

int sfref_paged_append(void* handle, const float* keys, const float* values, int tokens) {
    return guarded([&] {
        auto& cache = static_cast<PagedHandle*>(handle)->cache;
        const std::size_t rows = static_cast<std::size_t>(cache.config.batch) *
                                 cache.config.kv_heads * std::max(tokens, 0);
        schedforge::append_paged_kv(cache, vec(keys, rows * cache.config.head_dim),
                                    vec(values, rows * cache.config.head_dim_value), tokens);
    });
}

int sfref_paged_truncate(void* handle, int new_length) {
    return guarded([&] {
        schedforge::truncate_paged_kv(static_cast<PagedHandle*>(handle)->cache, new_length);
    });
}

int sfref_paged_release(void* handle, const int* pages, int count) {
    return guarded([&] {
        schedforge::release_paged_kv_pages(static_cast<PagedHandle*>(handle)->cache,
                                           std::vector<int>(pages, pages + count));
    });
}

// info[0] = length, info[1] = pages in table, info[2] = free pages, info[3] = total pages.
int sfref_paged_info(void* handle, int* info, int* page_table, int table_capacity,
                     int* free_pages, int free_capacity) {
    return guarded([&] {
        const auto& cache = static_cast<PagedHandle*>(handle)->cache;
        info[0] = cache.length;
        info[1] = static_cast<int>(cache.page_table.size());
        info[2] = static_cast<int>(cache.free_pages.size());
        info[3] = (cache.config.capacity + cache.config.page_tokens - 1) / cache.config.page_tokens;
        for (int i = 0; i < info[1] && i < table_capacity; ++i) page_table[i] = cache.page_table[i];
        for (int i = 0; i < info[2] && i < free_capacity; ++i) free_pages[i] = cache.free_pages[i];
    });
}

// Raw paged storage [page][batch][kv_head][page_tokens][dim].
int sfref_paged_storage(void* handle, float* keys, float* values) {
    return guarded([&] {
        const auto& cache = static_cast<PagedHandle*>(handle)->cache;
        out(cache.keys, keys);
        out(cache.values, values);
    });
}

// Contiguous [batch][kv_head][length][dim] copy of the live tokens.
int sfref_paged_gather(void* handle, float* keys, float* values) {
    return guarded([&] {
        const auto flat = schedforge::gather_paged_kv(static_cast<PagedHandle*>(handle)->cache);
        out(flat.keys, keys);
        out(flat.values, values);
    });
}

// use_reference = 0: paged_attention_online through execute_paged_decode_attention;
// use_reference = 1: the two-pass paged reference (returned via max_error trick is
// not available, so the result of the online path is validated against it and the
// error is returned through *max_error).
int sfref_paged_decode(void* handle, const sfref_attention_config* c, const float* query,
                       float* output, double* max_error, double* milliseconds) {
    return guarded([&] {
        const auto& cache = static_cast<PagedHandle*>(handle)->cache;
        const auto config = to_config(*c);
        const auto target = schedforge::TargetInfo::detect();
        const auto plan = schedforge::AttentionCompiler{target}.compile(
            config, schedforge::select_attention_plan(config, target, 1));
        const std::size_t count = static_cast<std::size_t>(config.batch) * config.query_heads *
                                  config.sequence_query * config.head_dim;
        const auto result = schedforge::execute_paged_decode_attention(
            plan, vec(query, count), cache, 0, 1, max_error != nullptr);
        out(result.output, output);
        if (max_error) *max_error = result.max_error;
        if (milliseconds) *milliseconds = result.p50_milliseconds;
    });
}

// ---- MoE ----------------------------------------------------------------------
int sfref_route_topk(const sfref_moe_config* c, const float* input, int tokens,
                     const float* router_weight, int* expert_ids, float* expert_weights,
                     int* counts) {
    return guarded([&] {
        const auto config = to_config(*c);
        schedforge::MoeData data;
        data.router_weight = vec(router_weight,
                                 static_cast<std::size_t>(config.hidden) * config.experts);
        const auto routing = schedforge::route_topk(
            config, data, vec(input, static_cast<std::size_t>(tokens) * config.hidden));
        std::memcpy(expert_ids, routing.expert_ids.data(), routing.expert_ids.size() * sizeof(int));
        std::memcpy(expert_weights, routing.expert_weights.data(),
                    routing.expert_weights.size() * sizeof(float));
        std::memcpy(counts, routing.counts.data(), routing.counts.size() * sizeof(int));
    });
}

int sfref_make_routing_trace(const sfref_moe_config* c, int distribution, unsigned seed,
                             int* expert_ids, float* expert_weights, int* counts) {
    return guarded([&] {
        const auto routing = schedforge::make_routing_trace(
            to_config(*c), static_cast<schedforge::RoutingDistribution>(distribution), seed);
        std::memcpy(expert_ids, routing.expert_ids.data(), routing.expert_ids.size() * sizeof(int));
        std::memcpy(expert_weights, routing.expert_weights.data(),
                    routing.expert_weights.size() * sizeof(float));
        std::memcpy(counts, routing.counts.data(), routing.counts.size() * sizeof(int));
    });
}

int sfref_dispatch_tokens(const sfref_moe_config* c, const float* input, int tokens,
                          const int* expert_ids, const float* expert_weights, const int* counts,
                          float* values, int* offsets, int* token_ids, int* route_slots,
                          float* routing_weights) {
    return guarded([&] {
        const auto config = to_config(*c);
        const auto trace = to_trace(config, tokens, expert_ids, expert_weights, counts);
        const auto result = schedforge::dispatch_tokens(
            config, vec(input, static_cast<std::size_t>(tokens) * config.hidden), trace);
        out(result.values, values);
        std::memcpy(offsets, result.offsets.data(), result.offsets.size() * sizeof(int));
        std::memcpy(token_ids, result.token_ids.data(), result.token_ids.size() * sizeof(int));
        std::memcpy(route_slots, result.route_slots.data(), result.route_slots.size() * sizeof(int));
        out(result.routing_weights, routing_weights);
    });
}

// tasks: rows of (expert, begin, end, bucket); returns the count through *task_count.
int sfref_plan_moe_tasks(const sfref_moe_config* c, int tokens, const int* expert_ids,
                         const float* expert_weights, const int* counts, int split_threshold,
                         int* tasks, int task_capacity, int* task_count) {
    return guarded([&] {
        const auto config = to_config(*c);
        const auto trace = to_trace(config, tokens, expert_ids, expert_weights, counts);
        schedforge::MoeExecutionSchedule schedule;
        if (split_threshold > 0) schedule.split_threshold = split_threshold;
        const auto plan = schedforge::MoeCompiler{}.compile(config, schedule);
        const auto planned = schedforge::plan_moe_tasks(trace, plan.schedule);
        *task_count = static_cast<int>(planned.size());
        for (int i = 0; i < *task_count && i < task_capacity; ++i) {
            tasks[4 * i + 0] = planned[i].expert;
            tasks[4 * i + 1] = planned[i].begin;
            tasks[4 * i + 2] = planned[i].end;
            tasks[4 * i + 3] = planned[i].bucket;
        }
    });
}

int sfref_reference_moe(const sfref_moe_config* c, const float* input, int tokens,
                        const float* router, const float* w1, const float* w3, const float* w2,
                        const int* expert_ids, const float* expert_weights, const int* counts,
                        float* output) {
    return guarded([&] {
        const auto config = to_config(*c);
        const auto data = to_moe_data(config, router, w1, w3, w2);
        const auto trace = to_trace(config, tokens, expert_ids, expert_weights, counts);
        out(schedforge::reference_moe(
                config, data, vec(input, static_cast<std::size_t>(tokens) * config.hidden), trace),
            output);
    });
}

// Native (threaded, bucketed grouped) MoE with a given trace.
// stage_ms[0..3] = total, dispatch, experts, combine.
int sfref_execute_moe(const sfref_moe_config* c, const float* input, int tokens,
                      const float* router, const float* w1, const float* w3, const float* w2,
                      const int* expert_ids, const float* expert_weights, const int* counts,
                      int threads, float* output, double* stage_ms) {
    return guarded([&] {
        const auto config = to_config(*c);
        const auto data = to_moe_data(config, router, w1, w3, w2);
        const auto trace = to_trace(config, tokens, expert_ids, expert_weights, counts);
        schedforge::MoeExecutionSchedule schedule;
        schedule.threads = threads > 0 ? threads : sfref_hardware_threads();
        const auto plan = schedforge::MoeCompiler{}.compile(config, schedule);
        const auto result = schedforge::execute_moe(
            plan, data, vec(input, static_cast<std::size_t>(tokens) * config.hidden), trace,
            0, 1, false);
        out(result.output, output);
        if (stage_ms) {
            stage_ms[0] = result.milliseconds;
            stage_ms[1] = result.dispatch_milliseconds;
            stage_ms[2] = result.expert_milliseconds;
            stage_ms[3] = result.combine_milliseconds;
        }
    });
}

// Weight-only INT8 experts: quantize_moe_weights + execute_quantized_moe with a given trace.
// max_error = against reference_moe on the unquantized weights (the reference's own bar is 0.2).
int sfref_quantized_moe(const sfref_moe_config* c, const float* input, int tokens,
                        const float* w1, const float* w3, const float* w2,
                        const int* expert_ids, const float* expert_weights, const int* counts,
                        int per_channel, float* output, double* max_error) {
    return guarded([&] {
        const auto config = to_config(*c);
        std::vector<float> router(static_cast<std::size_t>(config.hidden) * config.experts, 0.0F);
        auto data = to_moe_data(config, router.data(), w1, w3, w2);
        data.input = vec(input, static_cast<std::size_t>(tokens) * config.hidden);
        const auto trace = to_trace(config, tokens, expert_ids, expert_weights, counts);
        const auto weights = schedforge::quantize_moe_weights(config, data, per_channel != 0);
        const auto result = schedforge::execute_quantized_moe(config, data, trace, weights, 0, 1);
        out(result.output, output);
        if (max_error) *max_error = result.max_error;
    });
}

// realistic_decoder_profiles as text, one profile per line:
// name|batch|sequence|context|hidden|intermediate|q_heads|kv_heads|head_dim|ffn|experts|top_k|routing|flops|weight_bytes|activation_bytes
// followed by the header lines of the two CSV writers (written with no records) and the compile-only
// row of profile 14 as the reference's own test produces it (tests/test_schedforge.cpp:927-942).
int sfref_decoder_profiles(char* buffer, int capacity) {
    return guarded([&] {
        std::ostringstream out;
        const auto profiles = schedforge::realistic_decoder_profiles();
        for (const auto& p : profiles) {
            const auto& c = p.config;
            out << p.name << '|' << c.batch << '|' << c.sequence << '|' << c.context_sequence << '|' << c.hidden << '|'
                << c.intermediate << '|' << c.query_heads << '|' << c.kv_heads << '|' << c.head_dim << '|'
                << (c.ffn == schedforge::DecoderFFNKind::MoE ? 1 : 0) << '|' << c.experts << '|' << c.top_k << '|'
                << schedforge::routing_distribution_name(p.routing) << '|' << p.estimated_flops << '|'
                << p.estimated_weight_bytes << '|' << p.estimated_activation_bytes << '\n';
        }
        const auto dir = std::filesystem::temp_directory_path();
        const auto slurp = [](const std::filesystem::path& path) {
            std::ifstream in(path);
            return std::string((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
        };
        schedforge::write_decoder_benchmark_csv(dir / "sfref_profiles.csv", {});
        out << "#benchmark_header " << slurp(dir / "sfref_profiles.csv");
        schedforge::write_decoder_plan_candidates_csv(dir / "sfref_candidates.csv", {});
        out << "#candidates_header " << slurp(dir / "sfref_candidates.csv");
        const auto graph = schedforge::build_decoder_layer_graph(profiles[14].config);
        const auto record = schedforge::benchmark_decoder_profile(profiles[14], graph, 2, 1, 1, false, 1);
        schedforge::write_decoder_benchmark_csv(dir / "sfref_profiles.csv", {record});
        const std::string text = slurp(dir / "sfref_profiles.csv");
        out << "#compile_only_row " << text.substr(text.find('\n') + 1);
        const std::string all = out.str();
        if (static_cast<int>(all.size()) + 1 > capacity) throw std::runtime_error("profile buffer too small");
        std::memcpy(buffer, all.c_str(), all.size() + 1);
    });
}

}  // extern "C"
