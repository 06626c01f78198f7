// The decoder benchmark matrix of the reference, run on the GPU plan:
// realistic_decoder_profiles, benchmark_decoder_profile, write_decoder_benchmark_csv and
// write_decoder_plan_candidates_csv (include/schedforge/decoder_compiler.h:180-203,236-247;
// src/decoder_compiler.cpp:864-1060).  The 24 profiles, their FLOP / byte estimates, the synthetic
// data (make_decoder_data seed 101, make_routing_trace seed 103), the evidence kinds and both CSV
// schemas are the reference's; what is measured is the device plan.  Built on the C entry points
// of this library only.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <iomanip>
#include <random>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "runtime.hpp"

using namespace sfb;

namespace {

long long rows_of(const sfb_decoder_config& c) { return static_cast<long long>(c.batch) * c.sequence; }
long long kv_width_of(const sfb_decoder_config& c) { return static_cast<long long>(c.kv_heads) * c.head_dim; }

const char* routing_name(int routing) {
    return routing == 0 ? "uniform" : routing == 1 ? "moderate-skew" : "heavy-skew";
}
const char* evidence_name(int evidence) {
    return evidence == SFB_EVIDENCE_MEASURED ? "measured" : evidence == SFB_EVIDENCE_COMPILE_ONLY ? "compile-only" : "skipped";
}

// estimate_decoder_flops / estimate_decoder_weights / make_profile, src/decoder_compiler.cpp:864-905
sfb_decoder_profile make_profile(const std::string& name, const sfb_decoder_config& c, int routing) {
    sfb_decoder_profile p{};
    std::snprintf(p.name, sizeof(p.name), "%s", name.c_str());
    p.config = c;
    p.routing = routing;
    const std::uint64_t tokens = static_cast<std::uint64_t>(rows_of(c)), hidden = c.hidden, inter = c.intermediate;
    const std::uint64_t kv = static_cast<std::uint64_t>(kv_width_of(c));
    const std::uint64_t keys = c.context_sequence > 0 ? c.context_sequence : c.sequence;
    const std::uint64_t projections = 2 * tokens * hidden * (hidden + 2 * kv) + 2 * tokens * hidden * hidden;
    const std::uint64_t attention = 4 * static_cast<std::uint64_t>(c.batch) * c.query_heads * c.sequence * keys * c.head_dim;
    const std::uint64_t ffn = 6 * tokens * hidden * inter * (c.ffn_moe ? c.top_k : 1);
    p.estimated_flops = projections + attention + ffn;
    std::uint64_t values = hidden * (hidden + 2 * kv) + hidden * hidden;
    values += c.ffn_moe ? hidden * c.experts + 3 * hidden * inter * c.experts : 3 * hidden * inter;
    p.estimated_weight_bytes = values * sizeof(float);
    p.estimated_activation_bytes = tokens * (6 * hidden + 3 * inter) * sizeof(float);
    return p;
}

sfb_decoder_config base_config(int sequence, int hidden, int intermediate, int heads, int kv_heads, int dim) {
    sfb_decoder_config c{};
    c.batch = 1; c.sequence = sequence; c.hidden = hidden; c.intermediate = intermediate;
    c.query_heads = heads; c.kv_heads = kv_heads; c.head_dim = dim;
    c.rms_epsilon = 1.0e-5F; c.rope_theta = 10000.0F; c.causal = 1;  // DecoderConfig defaults
    c.experts = 4; c.top_k = 2;
    return c;
}

const std::vector<sfb_decoder_profile>& profiles() {
    static const std::vector<sfb_decoder_profile> table = [] {
        std::vector<sfb_decoder_profile> out;
        struct Scale { const char* name; int hidden, intermediate, heads, kv_heads, dim; };
        for (const Scale& s : {Scale{"tiny", 512, 1376, 8, 2, 64}, Scale{"medium", 1024, 2816, 16, 4, 64},
                               Scale{"large", 4096, 11008, 32, 8, 128}}) {
            for (const int sequence : {128, 512, 2048})
                out.push_back(make_profile(std::string(s.name) + "-prefill-s" + std::to_string(sequence),
                                           base_config(sequence, s.hidden, s.intermediate, s.heads, s.kv_heads, s.dim), 0));
            for (const int context : {128, 512, 2048, 4096}) {
                sfb_decoder_config c = base_config(1, s.hidden, s.intermediate, s.heads, s.kv_heads, s.dim);
                c.context_sequence = context;
                out.push_back(make_profile(std::string(s.name) + "-decode-kv" + std::to_string(context), c, 0));
            }
        }
        for (const int routing : {0, 1, 2}) {
            sfb_decoder_config c = base_config(32, 512, 1376, 8, 2, 64);
            c.ffn_moe = 1;
            c.experts = routing == 2 ? 16 : 8;
            c.top_k = 2;
            out.push_back(make_profile(std::string("tiny-moe-") + routing_name(routing), c, routing));
        }
        return out;
    }();
    return table;
}

// make_decoder_data (src/decoder_compiler.cpp:483-514) and make_moe_data (src/moe_compiler.cpp:393-406):
// one mt19937 stream per call, uniform in (-0.15, 0.15) resp. (-0.2, 0.2), filled in the reference's order.
struct HostData {
    std::vector<float> input, rms1, rms2, wq, wk, wv, wo, gate, up, down, router, w1, w3, w2, cached_key, cached_value;
    std::vector<int> trace_ids, trace_counts;
    std::vector<float> trace_weights;
    sfb_decoder_data view() const {
        sfb_decoder_data d{};
        d.rms1_weight = rms1.data(); d.query_weight = wq.data(); d.key_weight = wk.data(); d.value_weight = wv.data();
        d.output_weight = wo.data(); d.rms2_weight = rms2.data(); d.gate_weight = gate.data(); d.up_weight = up.data();
        d.down_weight = down.data();
        if (!router.empty()) { d.router_weight = router.data(); d.w1 = w1.data(); d.w3 = w3.data(); d.w2 = w2.data(); }
        if (!cached_key.empty()) { d.cached_key = cached_key.data(); d.cached_value = cached_value.data(); }
        return d;
    }
};

// make_routing_trace, src/moe_compiler.cpp:457-489: top_k distinct experts per token drawn from a uniform or
// power-law (exponent 0.8 / 1.6) distribution, equal weights 1 / top_k.
void routing_trace(int tokens, int experts, int top_k, int routing, std::uint32_t seed, int* ids, float* weights,
                   int* counts) {
    std::fill(counts, counts + experts, 0);
    std::mt19937 generator(seed);
    std::vector<double> probabilities(static_cast<std::size_t>(experts), 1.0);
    if (routing != 0) {
        const double exponent = routing == 1 ? 0.8 : 1.6;
        for (int x = 0; x < experts; ++x) probabilities[static_cast<std::size_t>(x)] = 1.0 / std::pow(x + 1.0, exponent);
    }
    std::discrete_distribution<int> draw(probabilities.begin(), probabilities.end());
    for (int t = 0; t < tokens; ++t) {
        std::vector<int> chosen;
        while (static_cast<int>(chosen.size()) < top_k) {
            const int expert = draw(generator);
            if (std::find(chosen.begin(), chosen.end(), expert) == chosen.end()) chosen.push_back(expert);
        }
        for (int slot = 0; slot < top_k; ++slot) {
            ids[static_cast<std::size_t>(t) * top_k + slot] = chosen[static_cast<std::size_t>(slot)];
            weights[static_cast<std::size_t>(t) * top_k + slot] = 1.0F / static_cast<float>(top_k);
            ++counts[chosen[static_cast<std::size_t>(slot)]];
        }
    }
}

HostData make_data(const sfb_decoder_config& c, std::uint32_t seed, int routing, std::uint32_t trace_seed) {
    HostData d;
    std::mt19937 generator(seed);
    std::uniform_real_distribution<float> distribution(-0.15F, 0.15F);
    const auto fill = [&](std::vector<float>& v, std::size_t n) {
        v.resize(n);
        for (float& x : v) x = distribution(generator);
    };
    const std::size_t h = c.hidden, i = c.intermediate, kv = static_cast<std::size_t>(kv_width_of(c));
    fill(d.input, static_cast<std::size_t>(rows_of(c)) * h);
    d.rms1.assign(h, 1.0F);
    d.rms2.assign(h, 1.0F);
    fill(d.wq, h * h); fill(d.wk, h * kv); fill(d.wv, h * kv); fill(d.wo, h * h);
    fill(d.gate, h * i); fill(d.up, h * i); fill(d.down, i * h);
    if (c.ffn_moe) {
        std::mt19937 moe_generator(seed + 1);
        std::uniform_real_distribution<float> moe_distribution(-0.2F, 0.2F);
        std::vector<float> moe_input(static_cast<std::size_t>(rows_of(c)) * h);  // drawn, then replaced by the layer input
        const std::size_t e = c.experts;
        d.router.resize(h * e); d.w1.resize(e * h * i); d.w3.resize(e * h * i); d.w2.resize(e * i * h);
        for (auto* v : {&moe_input, &d.router, &d.w1, &d.w3, &d.w2})
            for (float& x : *v) x = moe_distribution(moe_generator);
        const int tokens = static_cast<int>(rows_of(c));
        d.trace_ids.resize(static_cast<std::size_t>(tokens) * c.top_k);
        d.trace_weights.resize(d.trace_ids.size());
        d.trace_counts.resize(e);
        routing_trace(tokens, c.experts, c.top_k, routing, trace_seed, d.trace_ids.data(), d.trace_weights.data(),
                      d.trace_counts.data());
    }
    if (c.context_sequence > 0) {
        const std::size_t n = static_cast<std::size_t>(c.batch) * c.kv_heads * c.context_sequence * c.head_dim;
        fill(d.cached_key, n);
        fill(d.cached_value, n);
    }
    return d;
}

sfb_compile_options default_options(const sfb_compile_options* given) {
    sfb_compile_options o{};
    if (given) o = *given;
    else { o.dtype = SFB_BF16; o.token_major_attention = 1; o.fuse_epilogues = 1; }
    if (o.tp_size <= 0) o.tp_size = 1;
    return o;
}

// DecoderPlanPolicy::dump, src/decoder_compiler.cpp:312-324, for the axes a device plan has: the GEMM family
// stands for the schedule family (tensor cores = throughput, CUDA cores = latency), core placement and threads
// have no counterpart (compact, 0), attention names the kernel family.
std::string policy_text(const sfb_compile_options& o, const sfb_decoder_config& c) {
    const bool decode = c.sequence == 1 && c.context_sequence > 0;
    return std::string("decoder.policy layout=") + (o.token_major_attention ? "token_major" : "head_major") +
           " schedule=" + (o.gemm_backend == SFB_GEMM_SIMT ? "latency" : "throughput") + " placement=compact materialize=" +
           std::to_string(o.fuse_epilogues ? 0 : 1) + " reuse=" + std::to_string(o.no_workspace_reuse ? 0 : 1) +
           " threads=0 attention=" + (decode ? "split-kv-decode" : (o.attention_backend == 1 ? "io-aware-simt" : "io-aware"));
}

void check(sfb_status status) {
    if (status == SFB_OK) return;
    const std::string message = sfb_last_error();
    if (status == SFB_INVALID_ARGUMENT) throw std::invalid_argument(message);
    throw std::runtime_error(message);
}

}  // namespace

extern "C" {

sfb_status sfb_make_routing_trace(const sfb_moe_config* config, int distribution, unsigned seed, int* expert_ids,
                                  float* expert_weights, int* counts) {
    return guarded([&] {
        if (!config || !expert_ids || !expert_weights || !counts || config->tokens <= 0 || config->experts <= 0 ||
            config->top_k <= 0 || config->top_k > config->experts || distribution < 0 || distribution > 2)
            throw std::invalid_argument("invalid MoE configuration");
        routing_trace(config->tokens, config->experts, config->top_k, distribution, seed, expert_ids, expert_weights, counts);
    });
}

sfb_status sfb_make_decoder_input(const sfb_decoder_config* config, unsigned seed, float* input) {
    return guarded([&] {
        if (!config || !input || rows_of(*config) <= 0 || config->hidden <= 0) throw std::invalid_argument("invalid decoder configuration");
        std::mt19937 generator(seed);
        std::uniform_real_distribution<float> distribution(-0.15F, 0.15F);
        const std::size_t n = static_cast<std::size_t>(rows_of(*config)) * config->hidden;
        for (std::size_t i = 0; i < n; ++i) input[i] = distribution(generator);
    });
}

sfb_status sfb_make_decoder_data(const sfb_decoder_config* config, unsigned seed, float* input,
                                 const sfb_decoder_data_buffers* out) {
    return guarded([&] {
        if (!config || !out || rows_of(*config) <= 0 || config->hidden <= 0 || config->intermediate <= 0 ||
            config->kv_heads <= 0 || config->head_dim <= 0 || (config->ffn_moe && (config->experts <= 0 || config->top_k <= 0)))
            throw std::invalid_argument("invalid decoder configuration");
        // every tensor is drawn (the stream position of each one is part of the contract); a NULL destination only skips the copy
        sfb_decoder_config c = *config;
        const int top_k = c.top_k;
        if (c.ffn_moe) c.top_k = std::min(std::max(top_k, 1), c.experts);  // only sizes the (unused) routing trace
        const HostData d = make_data(c, seed, 0, 0);
        auto put = [](float* dst, const std::vector<float>& src) {
            if (dst && !src.empty()) std::memcpy(dst, src.data(), src.size() * sizeof(float));
        };
        put(input, d.input);
        put(out->rms1_weight, d.rms1); put(out->rms2_weight, d.rms2);
        put(out->query_weight, d.wq); put(out->key_weight, d.wk); put(out->value_weight, d.wv); put(out->output_weight, d.wo);
        put(out->gate_weight, d.gate); put(out->up_weight, d.up); put(out->down_weight, d.down);
        put(out->router_weight, d.router); put(out->w1, d.w1); put(out->w3, d.w3); put(out->w2, d.w2);
        put(out->cached_key, d.cached_key); put(out->cached_value, d.cached_value);
    });
}

int sfb_decoder_profile_count(void) { return static_cast<int>(profiles().size()); }

sfb_status sfb_decoder_profile_get(int index, sfb_decoder_profile* out) {
    return guarded([&] {
        if (!out || index < 0 || index >= sfb_decoder_profile_count()) throw std::invalid_argument("decoder profile index out of range");
        *out = profiles()[static_cast<std::size_t>(index)];
    });
}

sfb_status sfb_benchmark_decoder_profile(const sfb_decoder_profile* profile, const char* stablehlo_text,
                                         const sfb_compile_options* options, uint64_t max_real_flops,
                                         uint64_t max_real_weight_bytes, int optimize_plan, int repetitions,
                                         sfb_decoder_benchmark_record* record) {
    return guarded([&] {
        if (!profile || !record) throw std::invalid_argument("null decoder benchmark argument");
        *record = {};
        record->profile = *profile;
        record->optimizer_speedup = 1.0;
        const sfb_decoder_config& c = profile->config;
        const sfb_compile_options base = default_options(options);
        const bool feasible = profile->estimated_flops <= max_real_flops && profile->estimated_weight_bytes <= max_real_weight_bytes;
        if (!feasible) {
            // The reference compiles a plan without data here; a device plan owns its weights, so such a
            // record carries the profile's estimates only (no memory plan is evaluated; the policy stays empty as there).
            record->evidence = SFB_EVIDENCE_COMPILE_ONLY;
            std::snprintf(record->note, sizeof(record->note), "exceeds real-execution FLOP or weight-memory budget");
            return;
        }
        const HostData data = make_data(c, 101, profile->routing, 103);
        const sfb_decoder_data view = data.view();
        // MoE profiles use the canonical MoE graph (the reference re-imports examples/decoder_layer_moe.mlir)
        const char* text = c.ffn_moe ? nullptr : stablehlo_text;
        sfb_decoder_plan* plan = nullptr;
        sfb_compile_options chosen = base;
        if (optimize_plan) {
            sfb_optimization_result result{};
            check(sfb_decoder_optimize(&c, &view, text, &base, data.input.data(), 6, repetitions, &result,
                                       record->candidates, SFB_MAX_PLAN_CANDIDATES, &plan));
            record->candidate_count = std::min(result.candidates, static_cast<int>(SFB_MAX_PLAN_CANDIDATES));
            record->optimizer_speedup = result.speedup;
            record->optimizer_baseline_milliseconds = result.baseline.measured_milliseconds;
            record->hardware_measurements = result.hardware_measurements;
            record->plan_cost = result.winner;
            chosen = result.winner_options;
        } else {
            check(sfb_decoder_compile(&c, &view, text, &base, &plan));
        }
        struct Guard { sfb_decoder_plan* p; ~Guard() { sfb_decoder_destroy(p); } } guard{plan};
        std::snprintf(record->selected_policy, sizeof(record->selected_policy), "%s", policy_text(chosen, c).c_str());
        std::vector<float> output(data.input.size());
        // page-lock the two buffers that cross PCIe on every pass (a failed registration only costs speed)
        struct Pinned {
            void* p;
            bool ok;
            Pinned(const void* ptr, std::size_t bytes)
                : p(const_cast<void*>(ptr)), ok(cudaHostRegister(p, bytes, cudaHostRegisterDefault) == cudaSuccess) {
                if (!ok) (void)cudaGetLastError();
            }
            ~Pinned() { if (ok) cudaHostUnregister(p); }
        } pin_in(data.input.data(), data.input.size() * sizeof(float)), pin_out(output.data(), output.size() * sizeof(float));
        const int* ids = data.trace_ids.empty() ? nullptr : data.trace_ids.data();
        const float* weights = data.trace_weights.empty() ? nullptr : data.trace_weights.data();
        const int* counts = data.trace_counts.empty() ? nullptr : data.trace_counts.data();
        // execute_decoder_layer(plan, data, 1, repetitions): one warm-up, median of the repetitions
        sfb_decoder_result pass{};
        check(sfb_decoder_execute(plan, data.input.data(), output.data(), ids, weights, counts, &pass));
        std::vector<sfb_decoder_result> passes;
        for (int r = 0; r < std::max(1, repetitions); ++r) {
            check(sfb_decoder_execute(plan, data.input.data(), output.data(), ids, weights, counts, &pass));
            passes.push_back(pass);
        }
        std::sort(passes.begin(), passes.end(), [](const sfb_decoder_result& l, const sfb_decoder_result& r) {
            return l.milliseconds < r.milliseconds;
        });
        record->measured = passes[passes.size() / 2];
        record->evidence = SFB_EVIDENCE_MEASURED;
        record->plan_cost.workspace_bytes = sfb_decoder_workspace_bytes(plan);
        record->compile_milliseconds = sfb_decoder_compile_milliseconds(plan);
    });
}

sfb_status sfb_write_decoder_benchmark_csv(const char* path, const sfb_decoder_benchmark_record* records, int count) {
    return guarded([&] {
        if (!path || (!records && count > 0)) throw std::invalid_argument("null decoder benchmark CSV argument");
        const std::filesystem::path file(path);
        if (file.has_parent_path()) std::filesystem::create_directories(file.parent_path());
        std::ofstream out(file);
        if (!out) throw std::runtime_error(std::string("cannot write decoder benchmark: ") + path);
        out << "profile,evidence,ffn,batch,sequence,context,hidden,intermediate,q_heads,kv_heads,head_dim,experts,top_k,"
               "routing,estimated_flops,weight_bytes,activation_bytes,latency_ms,attention_ms,attention_pct,projection_ms,"
               "projection_pct,norm_rope_ms,norm_rope_pct,ffn_ms,ffn_pct,residual_ms,residual_pct,dispatch_ms,dispatch_pct,"
               "tokens_per_second,workspace_bytes,compile_ms,llvm_compile_ms,memory_planning_ms,memory_planning_pct,"
               "optimizer_baseline_ms,optimizer_speedup,hardware_measurements,max_error,selected_policy,note\n";
        out << std::fixed << std::setprecision(6);
        for (int r = 0; r < count; ++r) {
            const auto& rec = records[r];
            const auto& c = rec.profile.config;
            const auto& m = rec.measured;
            const auto pct = [&](double v) { return m.milliseconds > 0.0 ? v * 100.0 / m.milliseconds : 0.0; };
            const double planning_pct = rec.compile_milliseconds > 0.0
                ? rec.memory_planning_milliseconds * 100.0 / rec.compile_milliseconds : 0.0;
            // dispatch_ms: the host copies around the kernels, the part of a pass that is not a layer stage
            const double dispatch = m.h2d_milliseconds + m.d2h_milliseconds;
            out << rec.profile.name << ',' << evidence_name(rec.evidence) << ',' << (c.ffn_moe ? "moe" : "dense") << ','
                << c.batch << ',' << c.sequence << ',' << c.context_sequence << ',' << c.hidden << ',' << c.intermediate << ','
                << c.query_heads << ',' << c.kv_heads << ',' << c.head_dim << ',' << c.experts << ',' << c.top_k << ','
                << routing_name(rec.profile.routing) << ',' << rec.profile.estimated_flops << ','
                << rec.profile.estimated_weight_bytes << ',' << rec.profile.estimated_activation_bytes << ','
                << m.milliseconds << ',' << m.attention_milliseconds << ',' << pct(m.attention_milliseconds) << ','
                << m.projection_milliseconds << ',' << pct(m.projection_milliseconds) << ',' << m.norm_rope_milliseconds << ','
                << pct(m.norm_rope_milliseconds) << ',' << m.ffn_milliseconds << ',' << pct(m.ffn_milliseconds) << ','
                << m.residual_milliseconds << ',' << pct(m.residual_milliseconds) << ',' << dispatch << ',' << pct(dispatch) << ','
                << m.tokens_per_second << ',' << rec.plan_cost.workspace_bytes << ',' << rec.compile_milliseconds << ','
                << rec.llvm_compile_milliseconds << ',' << rec.memory_planning_milliseconds << ',' << planning_pct << ','
                << rec.optimizer_baseline_milliseconds << ',' << rec.optimizer_speedup << ',' << rec.hardware_measurements << ','
                << rec.max_error << ',' << rec.selected_policy << ',' << rec.note << '\n';
        }
    });
}

sfb_status sfb_write_decoder_plan_candidates_csv(const char* path, const sfb_decoder_benchmark_record* records, int count) {
    return guarded([&] {
        if (!path || (!records && count > 0)) throw std::invalid_argument("null decoder candidates CSV argument");
        const std::filesystem::path file(path);
        if (file.has_parent_path()) std::filesystem::create_directories(file.parent_path());
        std::ofstream out(file);
        if (!out) throw std::runtime_error(std::string("cannot write decoder candidates: ") + path);
        out << "profile,candidate,selected,measured,latency_ms,analytical_score,workspace_bytes,materialization_bytes,"
               "layout,schedule,placement,materialize,reuse,threads,attention\n";
        out << std::fixed << std::setprecision(6);
        for (int r = 0; r < count; ++r) {
            const auto& rec = records[r];
            const bool decode = rec.profile.config.sequence == 1 && rec.profile.config.context_sequence > 0;
            for (int i = 0; i < rec.candidate_count; ++i) {
                const auto& cand = rec.candidates[i];
                const auto& o = cand.options;
                out << rec.profile.name << ',' << i << ','
                    << (policy_text(o, rec.profile.config) == rec.selected_policy) << ',' << cand.cost.measured << ','
                    << cand.cost.measured_milliseconds << ',' << cand.cost.analytical_score << ','
                    << cand.cost.workspace_bytes << ',' << cand.cost.materialization_bytes << ','
                    << (o.token_major_attention ? "token_major" : "head_major") << ','
                    << (o.gemm_backend == SFB_GEMM_SIMT ? "latency" : "throughput") << ",compact,"
                    << (o.fuse_epilogues ? 0 : 1) << ',' << (o.no_workspace_reuse ? 0 : 1) << ",0,"
                    << (decode ? "split-kv-decode" : (o.attention_backend == 1 ? "io-aware-simt" : "io-aware")) << '\n';
            }
        }
    });
}

}  // extern "C"
