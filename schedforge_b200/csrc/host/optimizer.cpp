// Whole-layer plan optimizer on the GPU: the counterpart of ExecutablePlanOptimizer::optimize
// (include/schedforge/decoder_compiler.h:140-178, src/decoder_compiler.cpp:726-861).  Same
// procedure: enumerate policies, rank them with an analytic score, measure the baseline and the
// best-ranked `measurement_budget` candidates with equal warm-up, confirm a winner that beats
// the baseline with three interleaved baseline/winner measurements (medians), fall back to the
// baseline otherwise, report the speedup.  The policy axes are the ones that exist on this
// device: fused epilogues or materialised intermediates, tensor-core or CUDA-core GEMM family
// (the reference's Throughput / Latency schedule families), tensor-core or CUDA-core attention,
// workspace reuse on or off; thread counts and core placement have no counterpart.
#include <algorithm>
#include <cstring>
#include <limits>
#include <memory>
#include <stdexcept>
#include <vector>

#include "decoder.hpp"

namespace sfb {
struct PlanHandle;  // capi.cpp
}

using namespace sfb;

namespace {

double measure(DecoderExecutablePlan& plan, const float* input, int warmup, int repetitions) {
    plan.upload_input(input);
    cudaStream_t s = plan.stream();
    for (int i = 0; i < warmup; ++i) plan.run(s, RoutingTraceView{}, false);
    cudaEvent_t a, b;
    cuda_check(cudaEventCreate(&a), "event");
    cuda_check(cudaEventCreate(&b), "event");
    std::vector<double> times;
    for (int i = 0; i < std::max(1, repetitions); ++i) {
        cuda_check(cudaEventRecord(a, s), "event");
        plan.run(s, RoutingTraceView{}, false);
        cuda_check(cudaEventRecord(b, s), "event");
        cuda_check(cudaEventSynchronize(b), "event sync");
        float ms = 0.0F;
        cuda_check(cudaEventElapsedTime(&ms, a, b), "event time");
        times.push_back(ms);
    }
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    std::sort(times.begin(), times.end());
    return times[times.size() / 2];
}

// Analytic ranking: bytes an unfused plan writes and reads back, the workspace, and a penalty for
// running the contractions off the tensor cores (in milliseconds-like units; only the order matters).
sfb_plan_cost evaluate(const DecoderConfig& c, const sfb_compile_options& o, std::size_t workspace_bytes) {
    sfb_plan_cost cost{};
    const double rows = static_cast<double>(c.rows());
    const std::size_t elt = o.dtype == SFB_F32 ? 4 : 2;
    const double ffn_width = c.ffn == DecoderFFNKind::MoE ? 0.0 : 2.0 * c.intermediate;
    cost.workspace_bytes = workspace_bytes;
    cost.materialization_bytes = o.fuse_epilogues ? 0
        : static_cast<std::size_t>(rows * (c.qkv_width() + ffn_width + 2.0 * c.hidden)) * elt;
    const double flops = 2.0 * rows * c.hidden * (c.qkv_width() + c.hidden) +
                         6.0 * rows * c.hidden * c.intermediate * (c.ffn == DecoderFFNKind::MoE ? c.top_k : 1);
    const double gemm_penalty = (o.dtype == SFB_BF16 && o.gemm_backend == SFB_GEMM_SIMT) ? flops / 2.0e10 : 0.0;
    const double kv = c.context_sequence > 0 ? c.context_sequence : c.sequence;
    const double attention_penalty = (o.dtype == SFB_BF16 && o.attention_backend == 1)
        ? 4.0 * rows * kv * c.query_heads * c.head_dim / 2.0e10 : 0.0;
    cost.analytical_score = 2.0 * static_cast<double>(cost.materialization_bytes) / 6.0e9 * 1.0e3 +
                            static_cast<double>(workspace_bytes) / (1024.0 * 1024.0 * 1024.0) + gemm_penalty +
                            attention_penalty;
    return cost;
}

}  // namespace

namespace sfb {
std::unique_ptr<DecoderExecutablePlan> optimize_decoder_plan(
    const TensorGraph& graph, const DecoderConfig& config, const sfb_decoder_data& data, const sfb_compile_options& base,
    const float* input, int measurement_budget, int repetitions, sfb_optimization_result* result,
    sfb_plan_candidate* candidates_out, int capacity) {
    if (!input || !result) throw std::invalid_argument("optimizer: null input or result");
    std::vector<sfb_plan_candidate> candidates;
    for (const int fuse : {1, 0})
        for (const int gemm : {static_cast<int>(SFB_GEMM_AUTO), static_cast<int>(SFB_GEMM_SIMT)})
            for (const int attention : {0, 1})
                for (const int no_reuse : {0, 1}) {
                    sfb_plan_candidate cand{};
                    cand.options = base;
                    cand.options.fuse_epilogues = fuse;
                    cand.options.gemm_backend = gemm;
                    cand.options.attention_backend = attention;
                    cand.options.no_workspace_reuse = no_reuse;
                    candidates.push_back(cand);
                }
    *result = {};
    DecoderCompiler compiler;
    auto baseline_plan = compiler.compile(graph, config, data, base);
    result->baseline = evaluate(config, base, baseline_plan->workspace_bytes);
    result->baseline.measured = 1;
    result->baseline.measured_milliseconds = measure(*baseline_plan, input, 3, repetitions);
    ++result->hardware_measurements;

    // workspace sizes come from compiled plans; candidates that differ only in kernels share them
    std::size_t workspace_reuse = baseline_plan->workspace_bytes, workspace_no_reuse = baseline_plan->naive_bytes;
    for (auto& cand : candidates)
        cand.cost = evaluate(config, cand.options, cand.options.no_workspace_reuse ? workspace_no_reuse : workspace_reuse);
    std::stable_sort(candidates.begin(), candidates.end(), [](const sfb_plan_candidate& l, const sfb_plan_candidate& r) {
        return l.cost.analytical_score < r.cost.analytical_score;
    });

    const int budget = std::clamp(measurement_budget, 1, static_cast<int>(candidates.size()));
    double best = std::numeric_limits<double>::infinity();
    std::unique_ptr<DecoderExecutablePlan> winner_plan;
    sfb_compile_options winner_options = base;
    for (int i = 0; i < budget; ++i) {
        auto plan = compiler.compile(graph, config, data, candidates[i].options);
        candidates[i].cost.workspace_bytes = plan->workspace_bytes;
        candidates[i].cost.measured = 1;
        candidates[i].cost.measured_milliseconds = measure(*plan, input, 3, repetitions);
        ++result->hardware_measurements;
        if (candidates[i].cost.measured_milliseconds < best) {
            best = candidates[i].cost.measured_milliseconds;
            result->winner = candidates[i].cost;
            winner_options = candidates[i].options;
            winner_plan = std::move(plan);
        }
    }
    if (result->baseline.measured_milliseconds > best) {  // three interleaved confirmations, medians
        std::vector<double> base_times, win_times;
        for (int k = 0; k < 3; ++k) {
            base_times.push_back(measure(*baseline_plan, input, k == 0 ? 1 : 0, repetitions));
            win_times.push_back(measure(*winner_plan, input, k == 0 ? 1 : 0, repetitions));
            result->hardware_measurements += 2;
        }
        std::sort(base_times.begin(), base_times.end());
        std::sort(win_times.begin(), win_times.end());
        result->baseline.measured_milliseconds = base_times[1];
        result->winner.measured_milliseconds = win_times[1];
        best = win_times[1];
    }
    const double confirmed_baseline = result->baseline.measured_milliseconds;
    if (confirmed_baseline <= best) {
        winner_plan = std::move(baseline_plan);
        result->winner = result->baseline;
        winner_options = base;
        best = confirmed_baseline;
    }
    result->winner_options = winner_options;
    result->candidates = static_cast<int>(candidates.size()) + 1;
    result->speedup = best > 0.0 ? confirmed_baseline / best : 1.0;
    if (candidates_out && capacity > 0) {
        sfb_plan_candidate first{};
        first.options = base;
        first.cost = result->baseline;
        candidates_out[0] = first;
        for (int i = 0; i + 1 < capacity && i < static_cast<int>(candidates.size()); ++i) candidates_out[i + 1] = candidates[i];
    }
    return winner_plan;
}
}  // namespace sfb
