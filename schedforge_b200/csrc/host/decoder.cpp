#include "decoder.hpp"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <numeric>
#include <random>
#include <sstream>

#include "../common.cuh"

namespace sfb {

void validate(const DecoderConfig& c) {
    if (c.batch <= 0 || c.sequence <= 0 || c.hidden <= 0 || c.intermediate <= 0 || c.query_heads <= 0 ||
        c.kv_heads <= 0 || c.head_dim <= 0 || c.hidden != c.query_heads * c.head_dim ||
        c.query_heads % c.kv_heads != 0 || c.rms_epsilon <= 0.0F)
        throw std::invalid_argument("invalid decoder configuration");
    if (c.ffn == DecoderFFNKind::MoE && (c.experts <= 0 || c.top_k <= 0 || c.top_k > c.experts))
        throw std::invalid_argument("invalid decoder MoE configuration");
    if (c.context_sequence < 0) throw std::invalid_argument("invalid decoder context sequence");
}

TensorGraph build_decoder_layer_graph(const DecoderConfig& c) {
    validate(c);
    auto dims = [](std::initializer_list<int> extents) {
        GraphTensorType type;
        for (const int e : extents) type.shape.push_back(Dimension::fixed(e));
        return type;
    };
    TensorGraph g;
    const int T = c.rows();
    const auto hidden = dims({T, c.hidden});
    const auto q_type = dims({c.batch, c.query_heads, c.sequence, c.head_dim});
    const auto kv_type = dims({c.batch, c.kv_heads, c.sequence, c.head_dim});
    const int x = g.addInput("x", hidden);
    const int rms1 = g.addInput("rms1_weight", dims({c.hidden}), true);
    const int n1 = g.addOperation(GraphOpKind::RmsNorm, "attention_rms_norm", {x, rms1}, hidden);
    const int wqkv = g.addInput("packed_qkv_weight", dims({c.hidden, c.qkv_width()}), true);
    const int qkv = g.addOperation(GraphOpKind::FusedQKVProjection, "fused_qkv_projection", {n1, wqkv},
                                   dims({T, c.qkv_width()}));
    const int q = g.addOperation(GraphOpKind::Split, "split_query", {qkv}, q_type);
    const int k = g.addOperation(GraphOpKind::Split, "split_key", {qkv}, kv_type);
    const int v = g.addOperation(GraphOpKind::Split, "split_value", {qkv}, kv_type);
    const int rq = g.addOperation(GraphOpKind::RoPE, "rope_query", {q}, q_type);
    const int rk = g.addOperation(GraphOpKind::RoPE, "rope_key", {k}, kv_type);
    const int attn = g.addOperation(GraphOpKind::AttentionSdpa, "flash_attention", {rq, rk, v}, q_type);
    const int merged = g.addOperation(GraphOpKind::Concat, "merge_heads", {attn}, hidden);
    const int wo = g.addInput("output_weight", dims({c.hidden, c.hidden}), true);
    const int proj = g.addOperation(GraphOpKind::MatMul, "output_projection", {merged, wo}, hidden);
    const int r1 = g.addOperation(GraphOpKind::Add, "attention_residual", {proj, x}, hidden);
    const int rms2 = g.addInput("rms2_weight", dims({c.hidden}), true);
    const int n2 = g.addOperation(GraphOpKind::RmsNorm, "ffn_rms_norm", {r1, rms2}, hidden);
    int ffn = -1;
    if (c.ffn == DecoderFFNKind::Dense) {
        const int wgu = g.addInput("packed_gate_up_weight", dims({c.hidden, 2 * c.intermediate}), true);
        const int gu = g.addOperation(GraphOpKind::FusedGateUpProjection, "fused_gate_up_projection", {n2, wgu},
                                      dims({T, 2 * c.intermediate}));
        const int act = g.addOperation(GraphOpKind::SwiGLU, "swiglu", {gu}, dims({T, c.intermediate}));
        const int wd = g.addInput("down_weight", dims({c.intermediate, c.hidden}), true);
        ffn = g.addOperation(GraphOpKind::MatMul, "down_projection", {act, wd}, hidden);
    } else {
        const int wr = g.addInput("router_weight", dims({c.hidden, c.experts}), true);
        const int logits = g.addOperation(GraphOpKind::MatMul, "router_projection", {n2, wr}, dims({T, c.experts}));
        const int topk = g.addOperation(GraphOpKind::TopK, "router_topk", {logits});
        const int dispatch = g.addOperation(GraphOpKind::MoeDispatch, "token_dispatch", {n2, topk});
        const int expert = g.addOperation(GraphOpKind::MoeGroupedMatMul, "expert_grouped_ffn", {dispatch});
        ffn = g.addOperation(GraphOpKind::MoeCombine, "expert_combine", {expert, topk}, hidden);
    }
    g.setReturn(g.addOperation(GraphOpKind::Add, "ffn_residual", {ffn, r1}, hidden));
    ShapeInferencePass{}.run(g);
    return g;
}

std::string DecoderPlanPolicy::dump() const {
    return std::string("decoder.policy layout=") + (token_major_attention ? "token_major" : "head_major") +
           " schedule=throughput placement=compact materialize=" + std::to_string(!fuse_epilogues) +
           " reuse=" + std::to_string(reuse_workspace) + " threads=0";
}

std::string DecoderConstant::dump() const {
    std::ostringstream out;
    auto list = [&](const std::vector<int>& v) {
        for (std::size_t i = 0; i < v.size(); ++i) out << (i ? "," : "") << v[i];
    };
    out << "constant @" << name << " logical=[";
    list(logical_shape);
    out << "] packed=[";
    list(packed_shape);
    out << "] layout=" << layout << " bytes=" << bytes;
    return out.str();
}

// ---------------------------------------------------------------------------------------

struct DecoderExecutablePlan::Impl {
    // local (this shard's) extents
    int T = 0, H = 0, D = 0, hq = 0, hkv = 0, hidden_l = 0, kvw_l = 0, qkv_l = 0, I_l = 0;
    int E = 0, E_l = 0, e_begin = 0, K = 0;
    int rank = 0, size = 1;
    int dtype = SFB_BF16;
    int swiglu_block = 0;       // dense gate/up interleave block (bf16)
    int moe_swiglu_block = 0;   // expert W3|W1 interleave block (bf16)
    bool decode = false, paged = false;
    int page_tokens = 16, max_blocks = 0, num_blocks = 0, splits = 1;
    bool append_new = false;        // autoregressive step: append the new token's K/V, attend over context + 1
    // RMSNorm folded into the following GEMM: norm weight inside the packed weight, 1/rms applied to accumulator rows
    bool fold1 = false, fold2 = false;
    float rms_eps = 1.0e-5F;
    // where the sums of squares of the current pass live (workspace, or the gathered copies of a two-shot plan)
    const float* cur_ss1 = nullptr;
    const void* cur_ss2 = nullptr;
    bool cur_ss2_fixed = false;     // 64-bit fixed-point sums left by the O projection's epilogue (single shard)
    bool kv_in_epilogue = false;    // the QKV epilogue writes the new token's K/V into the paged cache itself
    // Paged cache accounting of a decode plan, kept like the reference's PagedKVCache (one page table and one
    // length for the whole batch, pages taken from the back of the free list; src/next_milestones.cpp:486-550).
    // Page p of sequence b is physical block block_ids[p * batch + b] of the pool.
    int kv_length = 0, kv_capacity = 0;
    std::vector<int> page_table, free_pages, block_ids;
    std::vector<int> trace_counts;  // expert-parallel plan with a caller's trace: this rank's histogram of it
    int* len_pinned = nullptr;      // start lengths for the stand-alone append kernel (plans without the fused append)
    int len_uploaded = -1;
    // Device block table for ALL logical blocks: the pages in use, then the free pages in the order they will be
    // handed out, so that a step that crosses a page boundary finds its entry already there.
    void sync_table(int batch, cudaStream_t s) {
        std::vector<int> order(page_table);
        for (auto it = free_pages.rbegin(); it != free_pages.rend(); ++it) order.push_back(*it);
        std::vector<int> table(static_cast<std::size_t>(batch) * max_blocks, 0);
        for (int b = 0; b < batch; ++b)
            for (std::size_t i = 0; i < order.size() && i < static_cast<std::size_t>(max_blocks); ++i)
                table[static_cast<std::size_t>(b) * max_blocks + i] = block_ids[static_cast<std::size_t>(order[i]) * batch + b];
        cuda_check(cudaMemcpyAsync(block_table, table.data(), table.size() * sizeof(int), cudaMemcpyHostToDevice, s), "block table");
        cuda_check(cudaStreamSynchronize(s), "block table sync");
    }

    DeviceBuffer weights, workspace, kv_pool;
    WorkspacePlanner planner{true};
    // weight pointers inside `weights`
    float *rms1 = nullptr, *rms2 = nullptr, *rope_cos = nullptr, *rope_sin = nullptr;
    void *wqkv = nullptr, *wo = nullptr, *wgu = nullptr, *wd = nullptr;
    float *router = nullptr, *router_bias = nullptr;
    void *w13 = nullptr, *w2 = nullptr;       // bf16: [E_l][2I][H], [E_l][H][I]
    float *w1f = nullptr, *w3f = nullptr, *w2f = nullptr;  // f32: reference layouts
    void *k_pool = nullptr, *v_pool = nullptr;
    int *block_table = nullptr, *context_len = nullptr;
    void *kc = nullptr, *vc = nullptr;         // contiguous cached K/V (decode with sequence > 1)
    cudaEvent_t events[16] = {};
    int pipeline_chunks = 1;      // host copies overlap compute in this many row chunks (1 = off)
    std::vector<std::pair<int, int>> pipeline_ranges;  // (first row, rows) of every chunk: whole sequences or part of one
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    // "chunk landed" words: the copy stream copies upload_epoch_host (pinned) into chunk_flags[c] behind the rows of
    // chunk c and the kernel stream waits for the word with a kernel.  An event from the copy stream would do, but
    // beside saturated PCIe traffic every cross-stream event wait held the kernels up by tens of microseconds.
    uint32_t* chunk_flags = nullptr;
    uint32_t* upload_epoch_host = nullptr;
    uint32_t upload_epoch = 0;
    std::vector<cudaEvent_t> chunk_events;   // per chunk: input landed, compute done, + 4 stage marks
    bool has_input = false;
    void* output_bf16 = nullptr;    // where the last pass left the bf16 output
    bool output_f32_valid = true;   // false: "output_f32" has to be converted from output_bf16 before the host reads it
    // fp32 copy of output rows [first, first + rows) for a host read (no-op when the pass already produced it)
    void materialize_output(int first, int rows, cudaStream_t s) {
        if (output_f32_valid || !output_bf16) return;
        const std::size_t at = static_cast<std::size_t>(first) * H;
        throw_on(sfb_k_convert(static_cast<char*>(output_bf16) + at * 2, SFB_BF16, ws<float>("output_f32") + at, SFB_F32,
                               static_cast<int64_t>(rows) * H, s));
        if (first == 0 && rows == T) output_f32_valid = true;
    }
    // Device status word (bounded waits that gave up) of the plan's device and a pinned host copy that every
    // host-synchronising call refreshes in stream order, so a timed-out wait surfaces as SFB_DEVICE_TIMEOUT.
    uint32_t* status_device = nullptr;
    uint32_t* status_host = nullptr;
    void queue_status_read(cudaStream_t s) {
        if (status_device && status_host)
            cuda_check(cudaMemcpyAsync(status_host, status_device, sizeof(uint32_t), cudaMemcpyDeviceToHost, s), "status read");
    }
    // after the stream has been synchronised: a non-zero word means that some kernel of the pass gave up waiting,
    // so the output is not the layer's; the word is cleared and the split-K scratch (sums and tile counters that an
    // aborted few-row GEMM leaves behind) is zeroed again so that the next pass starts clean
    void check_status(cudaStream_t s) {
        if (!status_host || *status_host == 0) return;
        const uint32_t word = *status_host;
        *status_host = 0;
        cuda_check(cudaMemsetAsync(status_device, 0, sizeof(uint32_t), s), "status clear");
        if (has("gemm_partials"))
            cuda_check(cudaMemsetAsync(ws("gemm_partials"), 0, planner.bytes(planner.find("gemm_partials")), s), "scratch clear");
        if (peer_local)  // the block counters of the two-shot kernels must start at zero again
            cuda_check(cudaMemsetAsync(peer_local + counters_offset(), 0, 64, s), "counter clear");
        cuda_check(cudaStreamSynchronize(s), "status clear sync");
        char text[96];
        std::snprintf(text, sizeof(text), "a bounded device-side wait gave up (status word 0x%x)", word);
        throw DeviceError(SFB_DEVICE_TIMEOUT, text);
    }
    // dense fused bf16 plan on one rank: the last GEMM writes the fp32 result itself, "output" is skipped
    bool direct_f32_output = false;
    // fused all-reduce over peer memory: [2 slot sets][size slots][slot_bytes] + flags [2][size]
    char* peer_local = nullptr;
    char* peer_remote[SFB_MAX_PEERS] = {};
    uint32_t peer_epoch[2] = {0, 0};
    std::size_t peer_slot_bytes() const { return (static_cast<std::size_t>(T) * H * 2 + 255) / 256 * 256; }
    std::size_t peer_flags_offset() const { return 2 * static_cast<std::size_t>(size) * peer_slot_bytes(); }
    // this rank's slot of slot set `set` in every other rank's receive buffer, `offset` elements in
    void fill_peer_out(sfb_gemm_args& g, int set, std::size_t offset) const {
        for (int r = 0; r < size; ++r)
            if (r != rank)
                g.peer_out[g.peer_count++] =
                    peer_remote[r] + (static_cast<std::size_t>(set) * size + rank) * peer_slot_bytes() + offset * 2;
    }
    // ---- two-shot form (reduce-scatter under the GEMM, sum + all-gather by the row owners), see peer_allreduce.cu.
    // Behind the one-shot slots and their flags the peer buffer holds: two-shot flags and counters, this rank's
    // partial tensors [2 sets][T rows] (written by its own O / Down GEMM with the ordinary epilogue; every owner
    // fetches its rows from them with wide peer loads, which use NVLink far better than 64-byte stores out of a
    // GEMM epilogue), three gathered tensors (layer input, attention_residual, output) that every rank's finish
    // kernel fills on every rank, and the gathered sums of squares of the first two.
    int peer_mode = 0;             // 0 = hook, 1 = one-shot fused all-reduce, 2 = two-shot, 3 = two-shot with the all-gather on copy engines
    // mode 3: after the owner kernel (sum, no gather) the finished rows, their sums of squares and a "rows sent" word
    // go to every peer with peer-to-peer copies on a side stream, i.e. on copy engines, while the next GEMM already
    // runs on the rows it has (it waits per owner, sfb_gemm_args.owner_flags); the pass ends with a wait for the
    // peers' last rows and for this rank's own copies
    cudaStream_t ce_stream = nullptr;
    cudaEvent_t ce_ready = nullptr, ce_done = nullptr;
    bool ce_pending = false;
    bool ce_gather() const { return two_shot() && peer_mode == 3; }
    uint32_t* ce_epoch_word(int coll) const { return reinterpret_cast<uint32_t*>(peer_local + counters_offset()) + 8 + coll; }
    uint32_t* ce_flags(int r, int coll) const {
        return reinterpret_cast<uint32_t*>(peer_base(r) + flags2_offset()) + (5 + coll) * 2 * SFB_MAX_PEERS;
    }
    void ce_push(int coll, bool with_ss, cudaStream_t s) {
        const std::size_t rows_own = static_cast<std::size_t>(T / size);
        const std::size_t row_bytes = rows_own * H * 2, first = static_cast<std::size_t>(rank) * row_bytes;
        cuda_check(cudaEventRecord(ce_ready, s), "event");
        cuda_check(cudaStreamWaitEvent(ce_stream, ce_ready, 0), "stream wait");
        for (int step = 1; step < size; ++step) {
            const int r = (rank - step + size) % size;  // the rank that reaches this owner's rows first is served first
            cuda_check(cudaMemcpyAsync(peer_remote[r] + gathered_offset(coll) + first, peer_local + gathered_offset(coll) + first,
                                       row_bytes, cudaMemcpyDeviceToDevice, ce_stream), "peer copy");
            if (with_ss)
                cuda_check(cudaMemcpyAsync(peer_remote[r] + ss_offset(coll) + rank * rows_own * 4,
                                           peer_local + ss_offset(coll) + rank * rows_own * 4, rows_own * 4,
                                           cudaMemcpyDeviceToDevice, ce_stream), "peer copy");
            cuda_check(cudaMemcpyAsync(ce_flags(r, coll) + rank, ce_epoch_word(coll), sizeof(uint32_t), cudaMemcpyDeviceToDevice,
                                       ce_stream), "peer flag copy");
        }
        ce_pending = true;
    }
    bool input_in_peer = false;    // the resident input is the gathered copy (sfb_decoder_execute_rows on a two-shot plan)
    uint32_t gather_epoch[6] = {0, 0, 0, 0, 0, 0};  // collectives 0-2: gathers; 3-5: expert-parallel plan / send / return
    std::size_t th_bytes() const { return (static_cast<std::size_t>(T) * H * 2 + 1023) / 1024 * 1024; }
    std::size_t flags2_offset() const { return peer_flags_offset() + 256; }
    std::size_t counters_offset() const { return peer_flags_offset() + 1024; }
    std::size_t recv2_offset() const { return peer_flags_offset() + 2048; }
    std::size_t partial_offset(int set) const { return recv2_offset() + set * th_bytes(); }
    std::size_t gathered_offset(int which) const { return recv2_offset() + 2 * th_bytes() + which * th_bytes(); }
    std::size_t ss_offset(int which) const { return gathered_offset(3) + which * ((static_cast<std::size_t>(T) * 4 + 255) / 256 * 256); }
    // expert-parallel MoE plans add: the table of every rank's per-expert histogram, the receive buffer for dispatched
    // rows (any split of the T * top_k assignments may land here) with their token ids and slots, and the buffer the
    // experts' owners return this rank's rows to (its local dispatched order)
    std::size_t ep_counts_offset() const { return ss_offset(2); }
    std::size_t ep_recv_rows_offset() const { return ep_counts_offset() + 4096; }
    std::size_t ep_capacity() const { return static_cast<std::size_t>(T) * std::max(1, K); }
    std::size_t ep_recv_tokens_offset() const { return ep_recv_rows_offset() + (ep_capacity() * H * 2 + 1023) / 1024 * 1024; }
    std::size_t ep_recv_slots_offset() const { return ep_recv_tokens_offset() + (ep_capacity() * 4 + 1023) / 1024 * 1024; }
    std::size_t ep_back_offset() const { return ep_recv_slots_offset() + (ep_capacity() * 4 + 1023) / 1024 * 1024; }
    std::size_t ep_end_offset() const { return ep_back_offset() + (ep_capacity() / size * H * 2 + 1023) / 1024 * 1024; }
    std::size_t peer_total_bytes() const { return (E > 0 ? ep_end_offset() : ss_offset(2)) + 256; }
    sfb_ep_sync ep_sync(int coll) {
        sfb_ep_sync y{};
        y.local_flags = reinterpret_cast<uint32_t*>(peer_local + flags2_offset()) + coll * 2 * SFB_MAX_PEERS;
        for (int r = 0; r < size; ++r)
            if (r != rank)
                y.peer_flags[r] = reinterpret_cast<uint32_t*>(peer_remote[r] + flags2_offset()) + coll * 2 * SFB_MAX_PEERS + rank;
        y.done_counter = reinterpret_cast<uint32_t*>(peer_local + counters_offset()) + coll;
        y.epoch = ++gather_epoch[coll];
        y.rank = rank; y.size = size;
        return y;
    }
    char* peer_base(int r) const { return r == rank ? peer_local : peer_remote[r]; }
    template <class P = void> P* gathered(int which) const { return reinterpret_cast<P*>(peer_local + gathered_offset(which)); }
    float* gathered_ss(int which) const { return reinterpret_cast<float*>(peer_local + ss_offset(which)); }
    bool two_shot() const { return size > 1 && peer_local != nullptr && peer_mode >= 2; }
    void* partial(int set) const { return peer_local + partial_offset(set); }
    // Owner side of collective `coll` (0 = all-gather of the input rows, 1 = after O, 2 = after Down): sums the slots of
    // set coll - 1 (+ residual rows), writes gathered tensor `coll` and optionally its sums of squares on every rank.
    sfb_status reduce_gather(int coll, const void* source, const float* source_ss, const void* residual, bool with_ss, cudaStream_t s,
                             int gather = 1, uint32_t* epoch_out = nullptr) {
        sfb_peer_gather_args a{};
        const int rows_own = T / size;
        if (coll > 0 && !source) {  // this owner's rows inside every rank's partial tensor of set coll - 1
            a.slots = size;
            for (int r = 0; r < size; ++r)
                a.pull[r] = peer_base(r) + partial_offset(coll - 1) + static_cast<std::size_t>(rank) * rows_own * H * 2;
        }
        a.source = source; a.source_ss = source_ss; a.residual = residual;
        for (int r = 0; r < size; ++r) {
            a.gathered[r] = peer_base(r) + gathered_offset(coll);
            a.ss[r] = with_ss ? reinterpret_cast<float*>(peer_base(r) + ss_offset(coll)) : nullptr;
            if (r != rank)
                a.peer_flags[r] = reinterpret_cast<uint32_t*>(peer_remote[r] + flags2_offset()) + coll * 2 * SFB_MAX_PEERS + rank;
        }
        a.local_flags = reinterpret_cast<uint32_t*>(peer_local + flags2_offset()) + coll * 2 * SFB_MAX_PEERS;
        a.done_counter = reinterpret_cast<uint32_t*>(peer_local + counters_offset()) + coll;
        a.rank = rank; a.size = size; a.epoch = ++gather_epoch[coll];
        a.rows_own = rows_own; a.width = H; a.gather = gather; a.epoch_out = epoch_out;
        return sfb_k_peer_reduce_gather(&a, s);
    }
    // completes the all-reduce whose data the preceding GEMM pushed: `count` elements starting `offset` elements in
    sfb_status peer_finish(int set, void* data, std::size_t offset, int64_t count, cudaStream_t s) {
        sfb_peer_allreduce_args a{};
        a.data = data;
        a.recv = peer_local + static_cast<std::size_t>(set) * size * peer_slot_bytes() + offset * 2;
        uint32_t* flags = reinterpret_cast<uint32_t*>(peer_local + peer_flags_offset());
        a.local_flags = flags + set * SFB_MAX_PEERS;
        for (int r = 0; r < size; ++r)
            if (r != rank)
                a.peer_flags[r] = reinterpret_cast<uint32_t*>(peer_remote[r] + peer_flags_offset()) + set * SFB_MAX_PEERS + rank;
        a.rank = rank; a.size = size; a.epoch = ++peer_epoch[set];
        a.count = count; a.slot_elems = static_cast<int64_t>(peer_slot_bytes() / 2);
        return sfb_k_peer_allreduce_finish(&a, s);
    }
    // weight-only INT8: per projection the int8 blocked copy and its per-column scales
    struct Int8Weight { const void* weight; void* q; float* scales; };
    std::vector<Int8Weight> int8_weights;
    DeviceBuffer int8_arena;
    const Int8Weight* int8(const void* w) const {
        for (const auto& entry : int8_weights)
            if (entry.weight == w) return &entry;
        return nullptr;
    }
    std::vector<const void*> blocked_weights;  // weights re-laid in 64x64 blocks (decode-shaped plans)
    bool blocked(const void* w) const {
        return std::find(blocked_weights.begin(), blocked_weights.end(), w) != blocked_weights.end();
    }

    std::size_t esz() const { return dtype == SFB_BF16 ? 2 : 4; }
    template <class P = void> P* ws(const char* name) {
        const int id = planner.find(name);
        if (id < 0) throw std::runtime_error(std::string("unknown workspace tensor: ") + name);
        return reinterpret_cast<P*>(workspace.as<char>() + planner.offset(id));
    }
    bool has(const char* name) const { return planner.find(name) >= 0; }
};

DecoderExecutablePlan::~DecoderExecutablePlan() {
    if (impl_) {
        for (auto& e : impl_->events)
            if (e) cudaEventDestroy(e);
        for (auto& e : impl_->chunk_events)
            if (e) cudaEventDestroy(e);
        if (impl_->copy_in) cudaStreamDestroy(impl_->copy_in);
        if (impl_->chunk_flags) cudaFree(impl_->chunk_flags);
        if (impl_->upload_epoch_host) cudaFreeHost(impl_->upload_epoch_host);
        if (impl_->copy_out) cudaStreamDestroy(impl_->copy_out);
        if (impl_->status_host) cudaFreeHost(impl_->status_host);
        if (impl_->len_pinned) cudaFreeHost(impl_->len_pinned);
        if (impl_->ce_stream) cudaStreamDestroy(impl_->ce_stream);
        if (impl_->ce_ready) cudaEventDestroy(impl_->ce_ready);
        if (impl_->ce_done) cudaEventDestroy(impl_->ce_done);
    }
    if (stream_) cudaStreamDestroy(stream_);
}

namespace {

struct WeightArena {
    std::size_t total = 0;
    std::size_t reserve(std::size_t bytes) {
        const std::size_t offset = total;
        total += (bytes + 1023) / 1024 * 1024;
        return offset;
    }
};

const float* need(const float* p, const char* name) {
    if (!p) throw std::invalid_argument(std::string("constant weight shape mismatch: missing ") + name);
    return p;
}

}  // namespace

// Row chunks of the pipelined host-buffer pass, in blocks of 128 rows (empty: the shape takes no row chunks).
// Chunks are sized for the GEMMs whose output is `hidden` wide (O and Down: 128 x 256 tiles, hidden / 256 per row
// block): a multiple of `unit` row blocks fills whole rounds of the SMs (9 row blocks x 16 = 144 tiles on 148 SMs at
// hidden = 4096, where 1536 rows were 192 tiles = two rounds of which the second is a third full).  Nothing overlaps
// the first upload and the last download, so the first and the last chunk are short; the chunks between them grow
// and shrink again (the copies run a little faster than the kernels).
std::vector<int> pipelined_row_blocks(int rows, int hidden, int sms) {
    if (rows <= 0 || hidden <= 0 || sms <= 0 || rows % 128 != 0 || hidden % 256 != 0) return {};
    const int unit = sms / (hidden / 256), blocks = rows / 128;
    if (unit < 2 || blocks < 8 + unit) return {};
    const int first = 4, last = 4 + (blocks - 8) % unit;
    const int units = (blocks - first - last) / unit;
    std::vector<int> sizes{first};
    if (units <= 2) {
        for (int i = 0; i < units; ++i) sizes.push_back(unit);
    } else {
        sizes.push_back(unit);
        int left = units - 2;
        const int group = std::max(2, (left + 5) / 6);
        for (; left > 0; left -= std::min(group, left)) sizes.push_back(std::min(group, left) * unit);
        sizes.push_back(unit);
    }
    sizes.push_back(last);
    return sizes;
}

std::unique_ptr<DecoderExecutablePlan> DecoderCompiler::compile(const TensorGraph& imported,
                                                                const DecoderConfig& c,
                                                                const sfb_decoder_data& data,
                                                                const sfb_compile_options& opt) const {
    const auto t0 = std::chrono::steady_clock::now();
    validate(c);
    auto plan = std::make_unique<DecoderExecutablePlan>();
    plan->config = c;
    plan->options = opt;
    plan->policy.token_major_attention = opt.token_major_attention != 0;
    plan->policy.fuse_epilogues = opt.fuse_epilogues != 0 && opt.dtype == SFB_BF16;
    plan->policy.gemm_backend = opt.gemm_backend;
    plan->policy.attention_backend = opt.attention_backend;
    plan->imported_graph = imported;
    plan->fusion = DecoderFusionPass{}.run(imported, c.ffn);
    if (!plan->fusion.fused_qkv || !plan->fusion.fused_rope ||
        (c.ffn == DecoderFFNKind::Dense && !plan->fusion.fused_gate_up))
        throw std::invalid_argument("decoder graph is missing required fusion patterns");
    plan->graph = build_decoder_layer_graph(c);

    const int G = opt.tp_size > 0 ? opt.tp_size : 1, r = opt.tp_rank;
    if (r < 0 || r >= G || c.query_heads % G != 0 || c.kv_heads % G != 0 || c.intermediate % G != 0 ||
        (c.ffn == DecoderFFNKind::MoE && c.experts % G != 0))
        throw std::invalid_argument("tensor-parallel size does not divide heads / FFN columns / experts");
    if (opt.dtype != SFB_F32 && opt.dtype != SFB_BF16) throw std::invalid_argument("unknown plan dtype");

    plan->impl_ = std::make_unique<DecoderExecutablePlan::Impl>();
    auto& m = *plan->impl_;
    m.T = c.rows(); m.H = c.hidden; m.D = c.head_dim;
    m.hq = c.query_heads / G; m.hkv = c.kv_heads / G;
    m.hidden_l = m.hq * m.D; m.kvw_l = m.hkv * m.D; m.qkv_l = m.hidden_l + 2 * m.kvw_l;
    m.rank = r; m.size = G; m.dtype = opt.dtype;
    const bool moe = c.ffn == DecoderFFNKind::MoE;
    // MoE under sharding: every rank holds E/G whole experts (full intermediate width).
    m.I_l = moe ? c.intermediate : c.intermediate / G;
    m.E = moe ? c.experts : 0; m.E_l = moe ? c.experts / G : 0; m.e_begin = r * m.E_l; m.K = moe ? c.top_k : 0;
    m.decode = c.context_sequence > 0;
    m.paged = m.decode && c.sequence == 1;
    m.page_tokens = opt.page_tokens > 0 ? opt.page_tokens : 16;
    m.append_new = m.paged && opt.append_new_token != 0;
    plan->policy.reuse_workspace = opt.no_workspace_reuse == 0;
    m.planner = WorkspacePlanner(plan->policy.reuse_workspace);
    const bool bf = m.dtype == SFB_BF16;
    const bool fused = plan->policy.fuse_epilogues;
    // A dense FFN width that is no multiple of 64 would send gate/up (no SwiGLU block the tensor-core epilogue
    // accepts) to the CUDA-core GEMM: the packed weights get zero columns up to the next multiple instead.
    // SiLU(0) * 0 = 0 in the padded activation columns meets zero rows of the padded down projection.
    const bool pad_ffn = bf && fused && !moe && G == 1 && c.intermediate % 64 != 0 && opt.gemm_backend != SFB_GEMM_SIMT;
    if (pad_ffn) m.I_l = (c.intermediate + 63) / 64 * 64;
    const int T = m.T, H = m.H, I = m.I_l, D = m.D;
    auto pick_block = [&](int width) {  // gate/up interleave that the tensor-core epilogue accepts
        if (T > 128 && width % 128 == 0) return 128;
        if (width % 64 == 0) return 64;
        return width;                   // one block: plain [gate | up] concatenation (CUDA-core GEMM)
    };
    m.swiglu_block = fused ? pick_block(I) : I;  // unfused: plain [gate | up] halves
    m.moe_swiglu_block = pick_block(c.intermediate);
    {
        // Both RMSNorms can be folded into the GEMM behind them when that GEMM (and, for the second norm, the O
        // projection that leaves the sums of squares) runs on the tensor-core kernel.  INT8 plans keep the
        // stand-alone norm: the reference quantizes the plain weights (src/next_milestones.cpp:660-675).
        auto on_tensor_cores = [&](int epilogue, int n, int k, int block) {
            sfb_gemm_args g{};
            void* aligned = reinterpret_cast<void*>(std::uintptr_t{1024});
            g.a = g.bt = aligned; g.out = aligned; g.residual = aligned;
            g.q = g.key = g.value = aligned;
            g.rope_cos = g.rope_sin = static_cast<const float*>(aligned);
            g.m = T; g.n = n; g.k = k; g.epilogue = epilogue; g.swiglu_block = block;
            g.batch = c.batch; g.seq = c.sequence; g.q_heads = m.hq; g.kv_heads = m.hkv; g.head_dim = D;
            return gemm_bf16_tcgen05_supported(g);
        };
        const bool eligible = bf && fused && opt.gemm_backend != SFB_GEMM_SIMT && opt.weight_int8 == 0 &&
                              D % 2 == 0 && (opt.norm_fusion > 0 || (opt.norm_fusion == 0 && G > 1));
        m.fold1 = eligible && on_tensor_cores(SFB_EPI_ROPE_SPLIT, m.qkv_l, H, 0);
        m.fold2 = eligible && !moe && on_tensor_cores(SFB_EPI_SWIGLU, 2 * I, H, m.swiglu_block) &&
                  on_tensor_cores(SFB_EPI_RESIDUAL, H, m.hidden_l, 0);
        m.kv_in_epilogue = m.append_new && bf && fused && opt.gemm_backend != SFB_GEMM_SIMT && D % 2 == 0 &&
                           on_tensor_cores(SFB_EPI_ROPE_SPLIT, m.qkv_l, H, 0);
    }
    // a single-shard dense plan on the tensor-core GEMM lets the down projection write the fp32 result itself
    m.direct_f32_output = bf && fused && !moe && G == 1 && opt.gemm_backend != SFB_GEMM_SIMT && H % 8 == 0 && I % 8 == 0;
    const int ctx = c.context_sequence;
    m.kv_capacity = m.append_new ? std::max(opt.kv_capacity, ctx + 1) : ctx;
    const int rope_positions = m.append_new ? m.kv_capacity : c.sequence;

    cuda_check(cudaStreamCreateWithFlags(&plan->stream_, cudaStreamNonBlocking), "cudaStreamCreate");
    cudaStream_t s = plan->stream_;

    // ---- weights: one arena ----------------------------------------------------------------
    const std::size_t wsz = bf ? 2 : 4;
    WeightArena arena;
    const std::size_t o_rms1 = arena.reserve(sizeof(float) * H), o_rms2 = arena.reserve(sizeof(float) * H);
    const std::size_t o_cos = arena.reserve(sizeof(float) * rope_positions * std::max(1, D / 2));
    const std::size_t o_sin = arena.reserve(sizeof(float) * rope_positions * std::max(1, D / 2));
    const std::size_t o_wqkv = arena.reserve(wsz * H * m.qkv_l), o_wo = arena.reserve(wsz * m.hidden_l * H);
    std::size_t o_wgu = 0, o_wd = 0, o_router = 0, o_bias = 0, o_w13 = 0, o_w2 = 0, o_w1f = 0, o_w3f = 0, o_w2f = 0;
    const std::size_t expert_elems = static_cast<std::size_t>(H) * c.intermediate;
    if (!moe) {
        o_wgu = arena.reserve(wsz * H * 2 * I);
        o_wd = arena.reserve(wsz * I * H);
    } else {
        o_router = arena.reserve(sizeof(float) * H * m.E);
        o_bias = arena.reserve(sizeof(float) * m.E);
        if (bf) {
            o_w13 = arena.reserve(2 * m.E_l * 2 * expert_elems);
            o_w2 = arena.reserve(2 * m.E_l * expert_elems);
        } else {
            o_w1f = arena.reserve(4 * m.E_l * expert_elems);
            o_w3f = arena.reserve(4 * m.E_l * expert_elems);
            o_w2f = arena.reserve(4 * m.E_l * expert_elems);
        }
    }
    m.weights.allocate(arena.total);
    plan->weight_bytes = arena.total;
    char* wb = m.weights.as<char>();
    m.rms1 = reinterpret_cast<float*>(wb + o_rms1); m.rms2 = reinterpret_cast<float*>(wb + o_rms2);
    m.rope_cos = reinterpret_cast<float*>(wb + o_cos); m.rope_sin = reinterpret_cast<float*>(wb + o_sin);
    m.wqkv = wb + o_wqkv; m.wo = wb + o_wo;
    auto h2d = [&](void* dst, const void* src, std::size_t bytes) {
        cuda_check(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, s), "weight upload");
        cuda_check(cudaStreamSynchronize(s), "weight upload sync");  // the host source may be a temporary
    };
    h2d(m.rms1, need(data.rms1_weight, "rms1_weight"), sizeof(float) * H);
    h2d(m.rms2, need(data.rms2_weight, "rms2_weight"), sizeof(float) * H);
    {
        // positions 0..sequence-1; an appending decode plan rotates its one token at the position it is appended
        // at, anywhere below the cache capacity (the run passes the table advanced by that many rows)
        const std::size_t row = static_cast<std::size_t>(std::max(1, D / 2));
        std::vector<float> cs(static_cast<std::size_t>(rope_positions) * row), sn(cs.size());
        if (D >= 2) throw_on(sfb_rope_table(rope_positions, D, c.rope_theta, cs.data(), sn.data()));
        h2d(m.rope_cos, cs.data(), cs.size() * 4);
        h2d(m.rope_sin, sn.data(), sn.size() * 4);
    }
    // fp32 staging buffer on the device for the transpose/convert packer
    std::size_t staging_elems = static_cast<std::size_t>(H) * std::max({H, c.intermediate, m.I_l, m.qkv_l});
    DeviceBuffer staging;
    if (bf) staging.allocate(staging_elems * 4);
    const int whole = 1 << 30;
    auto pack = [&](const float* host, int rows_k, int cols, int k_begin, int k_count, int c_begin, int c_count,
                    void* dst, int block, int stride, int offset, const float* norm_weight = nullptr) {
        h2d(staging.get(), host, static_cast<std::size_t>(rows_k) * cols * 4);
        pack_weight_transposed(staging.as<float>(), cols, k_begin, k_count, c_begin, c_count, dst, block, stride,
                               offset, s, norm_weight);
        cuda_check(cudaStreamSynchronize(s), "weight pack");
    };
    const float* wq = need(data.query_weight, "query_weight");
    const float* wk = need(data.key_weight, "key_weight");
    const float* wv = need(data.value_weight, "value_weight");
    const float* wo_h = need(data.output_weight, "output_weight");
    const int kvw = c.kv_width();
    if (bf) {
        const float* n1 = m.fold1 ? m.rms1 : nullptr;  // folded: W'[k, n] = rms1_weight[k] * W[k, n]
        pack(wq, H, H, 0, H, r * m.hidden_l, m.hidden_l, m.wqkv, whole, 0, 0, n1);
        pack(wk, H, kvw, 0, H, r * m.kvw_l, m.kvw_l, m.wqkv, whole, 0, m.hidden_l, n1);
        pack(wv, H, kvw, 0, H, r * m.kvw_l, m.kvw_l, m.wqkv, whole, 0, m.hidden_l + m.kvw_l, n1);
        pack(wo_h, H, H, r * m.hidden_l, m.hidden_l, 0, H, m.wo, whole, 0, 0);
    } else {
        std::vector<float> packed(static_cast<std::size_t>(H) * m.qkv_l);
        for (int row = 0; row < H; ++row) {
            float* dst = packed.data() + static_cast<std::size_t>(row) * m.qkv_l;
            std::memcpy(dst, wq + static_cast<std::size_t>(row) * H + r * m.hidden_l, sizeof(float) * m.hidden_l);
            std::memcpy(dst + m.hidden_l, wk + static_cast<std::size_t>(row) * kvw + r * m.kvw_l, sizeof(float) * m.kvw_l);
            std::memcpy(dst + m.hidden_l + m.kvw_l, wv + static_cast<std::size_t>(row) * kvw + r * m.kvw_l, sizeof(float) * m.kvw_l);
        }
        h2d(m.wqkv, packed.data(), packed.size() * 4);
        h2d(m.wo, wo_h + static_cast<std::size_t>(r) * m.hidden_l * H, static_cast<std::size_t>(m.hidden_l) * H * 4);
    }
    plan->constants.push_back({"packed_qkv_weight", {H, c.hidden, kvw, kvw}, {H, c.qkv_width()},
                               bf ? (m.fold1 ? "qkv_transposed_bf16_k_major_rms_folded" : "qkv_transposed_bf16_k_major") : "qkv_concat_f32",
                               static_cast<std::size_t>(H) * m.qkv_l * wsz});
    if (!moe) {
        m.wgu = wb + o_wgu; m.wd = wb + o_wd;
        const float* wg = need(data.gate_weight, "gate_weight");
        const float* wu = need(data.up_weight, "up_weight");
        const float* wd_h = need(data.down_weight, "down_weight");
        int Ifull = c.intermediate;
        std::vector<float> wg_padded, wu_padded, wd_padded;
        if (pad_ffn) {
            wg_padded.assign(static_cast<std::size_t>(H) * I, 0.0F);
            wu_padded.assign(static_cast<std::size_t>(H) * I, 0.0F);
            wd_padded.assign(static_cast<std::size_t>(I) * H, 0.0F);
            for (int row = 0; row < H; ++row) {
                std::memcpy(wg_padded.data() + static_cast<std::size_t>(row) * I, wg + static_cast<std::size_t>(row) * Ifull, sizeof(float) * Ifull);
                std::memcpy(wu_padded.data() + static_cast<std::size_t>(row) * I, wu + static_cast<std::size_t>(row) * Ifull, sizeof(float) * Ifull);
            }
            std::memcpy(wd_padded.data(), wd_h, sizeof(float) * static_cast<std::size_t>(Ifull) * H);
            wg = wg_padded.data(); wu = wu_padded.data(); wd_h = wd_padded.data();
            Ifull = I;
        }
        if (bf) {
            const float* n2 = m.fold2 ? m.rms2 : nullptr;
            pack(wg, H, Ifull, 0, H, r * I, I, m.wgu, m.swiglu_block, 2 * m.swiglu_block, 0, n2);
            pack(wu, H, Ifull, 0, H, r * I, I, m.wgu, m.swiglu_block, 2 * m.swiglu_block, m.swiglu_block, n2);
            pack(wd_h, Ifull, H, r * I, I, 0, H, m.wd, whole, 0, 0);
        } else {
            std::vector<float> packed(static_cast<std::size_t>(H) * 2 * I);
            for (int row = 0; row < H; ++row) {
                std::memcpy(packed.data() + static_cast<std::size_t>(row) * 2 * I, wg + static_cast<std::size_t>(row) * Ifull + r * I, sizeof(float) * I);
                std::memcpy(packed.data() + static_cast<std::size_t>(row) * 2 * I + I, wu + static_cast<std::size_t>(row) * Ifull + r * I, sizeof(float) * I);
            }
            h2d(m.wgu, packed.data(), packed.size() * 4);
            h2d(m.wd, wd_h + static_cast<std::size_t>(r) * I * H, static_cast<std::size_t>(I) * H * 4);
        }
        plan->constants.push_back({"packed_gate_up_weight", {H, c.intermediate, c.intermediate}, {H, 2 * Ifull},
                                   bf ? "gate_up_interleaved_" + std::to_string(m.swiglu_block) + (m.fold2 ? "_rms_folded" : "") : "gate_up_concat_f32",
                                   static_cast<std::size_t>(H) * 2 * I * wsz});
    } else {
        m.router = reinterpret_cast<float*>(wb + o_router);
        m.router_bias = data.router_bias ? reinterpret_cast<float*>(wb + o_bias) : nullptr;
        h2d(m.router, need(data.router_weight, "router_weight"), sizeof(float) * H * m.E);
        if (data.router_bias) h2d(m.router_bias, data.router_bias, sizeof(float) * m.E);
        const float* w1 = need(data.w1, "w1");
        const float* w3 = need(data.w3, "w3");
        const float* w2 = need(data.w2, "w2");
        const int Ifull = c.intermediate;
        const int first_expert = opt.local_expert_weights != 0 ? 0 : m.e_begin;  // index into the caller's arrays
        if (bf) {
            m.w13 = wb + o_w13; m.w2 = wb + o_w2;
            for (int e = 0; e < m.E_l; ++e) {
                const std::size_t src = static_cast<std::size_t>(first_expert + e) * expert_elems;
                char* d13 = static_cast<char*>(m.w13) + static_cast<std::size_t>(e) * 2 * expert_elems * 2;
                // SiLU applies to the W3 product, which multiplies the raw W1 product: [W3 | W1] = [gate | up]
                pack(w3 + src, H, Ifull, 0, H, 0, Ifull, d13, m.moe_swiglu_block, 2 * m.moe_swiglu_block, 0);
                pack(w1 + src, H, Ifull, 0, H, 0, Ifull, d13, m.moe_swiglu_block, 2 * m.moe_swiglu_block, m.moe_swiglu_block);
                pack(w2 + src, Ifull, H, 0, Ifull, 0, H, static_cast<char*>(m.w2) + static_cast<std::size_t>(e) * expert_elems * 2, whole, 0, 0);
            }
        } else {
            m.w1f = reinterpret_cast<float*>(wb + o_w1f); m.w3f = reinterpret_cast<float*>(wb + o_w3f);
            m.w2f = reinterpret_cast<float*>(wb + o_w2f);
            const std::size_t src = static_cast<std::size_t>(first_expert) * expert_elems, n = static_cast<std::size_t>(m.E_l) * expert_elems;
            h2d(m.w1f, w1 + src, n * 4);
            h2d(m.w3f, w3 + src, n * 4);
            h2d(m.w2f, w2 + src, n * 4);
        }
    }
    staging.release();
    if (opt.weight_int8 != 0) {
        if (!bf) throw std::invalid_argument("INT8 weights need a bf16 plan");
        if (moe) throw std::invalid_argument("INT8 decoder currently requires dense FFN weights");
        struct Item { void* w; int n, k; };
        const Item items[4] = {{m.wqkv, m.qkv_l, H}, {m.wo, H, m.hidden_l}, {m.wgu, 2 * I, H}, {m.wd, H, I}};
        const bool keep_int8 = T <= 128 && plan->policy.gemm_backend != SFB_GEMM_SIMT && fused && m.swiglu_block == 64;
        std::size_t bytes = 0;
        for (const auto& item : items)
            bytes += (static_cast<std::size_t>(sfb_tiled_weight_elems(item.n, item.k)) + 255) / 256 * 256 +
                     static_cast<std::size_t>(ceil_div(item.n, 128)) * 128 * sizeof(float);
        m.int8_arena.allocate(bytes);
        char* cursor = m.int8_arena.as<char>();
        for (const auto& item : items) {
            void* q = cursor;
            cursor += (static_cast<std::size_t>(sfb_tiled_weight_elems(item.n, item.k)) + 255) / 256 * 256;
            float* scales = reinterpret_cast<float*>(cursor);
            cursor += static_cast<std::size_t>(ceil_div(item.n, 128)) * 128 * sizeof(float);
            cuda_check(cudaMemsetAsync(scales, 0, static_cast<std::size_t>(ceil_div(item.n, 128)) * 128 * sizeof(float), s), "scale clear");
            throw_on(sfb_k_quantize_weight_int8(item.w, q, scales, item.n, item.k, s));
            if (keep_int8) m.int8_weights.push_back({item.w, q, scales});
            else throw_on(sfb_k_dequantize_weight_int8(q, scales, item.w, item.n, item.k, s));  // q * scale, bf16
        }
        cuda_check(cudaStreamSynchronize(s), "weight quantization");
        if (!keep_int8) m.int8_arena.release();
        for (auto& constant : plan->constants) constant.layout += keep_int8 ? "_int8_blocked64" : "_int8_values";
    }
    // Plans with few rows stream every weight once per pass: store the dense weights in 64x64
    // blocks so that the GEMM reads 8 KB contiguous runs instead of 128-byte row pieces.
    if (bf && T <= 128 && plan->policy.gemm_backend != SFB_GEMM_SIMT && m.int8_weights.empty()) {
        auto reblock = [&](void* w, int n, int k) {
            if (!w || n % 64 != 0 || k % 64 != 0) return;
            const std::size_t bytes = static_cast<std::size_t>(n) * k * 2;
            DeviceBuffer blocked(bytes);
            throw_on(sfb_k_tile_weight_bf16(w, blocked.get(), n, k, s));
            cuda_check(cudaMemcpyAsync(w, blocked.get(), bytes, cudaMemcpyDeviceToDevice, s), "weight reblock");
            cuda_check(cudaStreamSynchronize(s), "weight reblock");
            m.blocked_weights.push_back(w);
        };
        reblock(m.wqkv, m.qkv_l, H);
        reblock(m.wo, H, m.hidden_l);
        if (!moe) {
            if (!fused || m.swiglu_block == 64) reblock(m.wgu, 2 * I, H);  // the SwiGLU epilogue of the few-row kernel pairs 64-column blocks
            reblock(m.wd, H, I);
        }
        for (auto& constant : plan->constants)
            if ((constant.name == "packed_qkv_weight" && m.blocked(m.wqkv)) ||
                (constant.name == "packed_gate_up_weight" && m.blocked(m.wgu)))
                constant.layout += "_blocked64";
    }

    // ---- KV cache for decode plans ------------------------------------------------------------
    if (m.decode) {
        const float* ck = need(data.cached_key, "cached_key");
        const float* cv = need(data.cached_value, "cached_value");
        // this shard's KV heads, [B, hkv_l, ctx, D]
        const std::size_t per_head = static_cast<std::size_t>(ctx) * D;
        std::vector<float> lk(static_cast<std::size_t>(c.batch) * m.hkv * per_head), lv(lk.size());
        for (int b = 0; b < c.batch; ++b)
            for (int h = 0; h < m.hkv; ++h) {
                const std::size_t src = (static_cast<std::size_t>(b) * c.kv_heads + r * m.hkv + h) * per_head;
                const std::size_t dst = (static_cast<std::size_t>(b) * m.hkv + h) * per_head;
                std::memcpy(lk.data() + dst, ck + src, per_head * 4);
                std::memcpy(lv.data() + dst, cv + src, per_head * 4);
            }
        const std::size_t cache_bytes = lk.size() * m.esz();
        DeviceBuffer f32_stage(lk.size() * 4 * 2);
        float* dk = f32_stage.as<float>();
        float* dv = dk + lk.size();
        h2d(dk, lk.data(), lk.size() * 4);
        h2d(dv, lv.data(), lv.size() * 4);
        if (m.paged) {
            m.max_blocks = ceil_div(m.kv_capacity, m.page_tokens);
            m.num_blocks = c.batch * m.max_blocks;
            const std::size_t pool_elems = static_cast<std::size_t>(m.num_blocks) * m.hkv * m.page_tokens * D;
            const std::size_t table_bytes = sizeof(int) * m.num_blocks, len_bytes = sizeof(int) * c.batch;
            const std::size_t pool_bytes = (pool_elems * m.esz() + 1023) / 1024 * 1024;
            m.kv_pool.allocate(2 * pool_bytes + table_bytes + 2 * len_bytes + 1024);
            DeviceBuffer converted(bf ? 2 * cache_bytes : 0);
            char* kb = m.kv_pool.as<char>();
            m.k_pool = kb; m.v_pool = kb + pool_bytes;
            m.block_table = reinterpret_cast<int*>(kb + 2 * pool_bytes);
            m.context_len = m.block_table + m.num_blocks;
            char* tmp = converted.as<char>();
            std::vector<int> lens(c.batch, 0);
            m.block_ids.resize(m.num_blocks);
            std::iota(m.block_ids.begin(), m.block_ids.end(), 0);
            if (opt.seed_block_table != 0) {
                std::mt19937 generator(static_cast<unsigned>(opt.seed_block_table));
                std::shuffle(m.block_ids.begin(), m.block_ids.end(), generator);
            }
            // make_paged_kv_cache + append_paged_kv of the cached context: the free list starts as 0..pages-1 and
            // every page comes from its back (src/next_milestones.cpp:472-500)
            m.free_pages.resize(m.max_blocks);
            std::iota(m.free_pages.begin(), m.free_pages.end(), 0);
            for (int page = 0; page < ceil_div(ctx, m.page_tokens); ++page) {
                m.page_table.push_back(m.free_pages.back());
                m.free_pages.pop_back();
            }
            m.kv_length = ctx;
            m.sync_table(c.batch, s);
            cuda_check(cudaHostAlloc(reinterpret_cast<void**>(&m.len_pinned), len_bytes, cudaHostAllocDefault), "length staging");
            h2d(m.context_len, lens.data(), len_bytes);  // start lengths for the append kernel
            cuda_check(cudaMemsetAsync(m.k_pool, 0, 2 * pool_bytes, s), "pool clear");
            void *ak = dk, *av = dv;
            if (bf) {
                throw_on(sfb_k_convert(dk, SFB_F32, tmp, SFB_BF16, static_cast<int64_t>(lk.size()), s));
                throw_on(sfb_k_convert(dv, SFB_F32, tmp + cache_bytes, SFB_BF16, static_cast<int64_t>(lv.size()), s));
                ak = tmp; av = tmp + cache_bytes;
            }
            throw_on(sfb_k_paged_kv_append(ak, av, m.k_pool, m.v_pool, m.block_table, m.context_len, c.batch, m.hkv,
                                           ctx, D, D, m.page_tokens, m.max_blocks, m.num_blocks, static_cast<sfb_dtype>(m.dtype), s));
            cuda_check(cudaStreamSynchronize(s), "paged cache build");
            m.splits = sfb_attention_decode_default_splits(c.batch, m.hkv, m.kv_capacity);
            plan->attention_strategy = "split_kv_decode";
        } else {
            m.kv_pool.allocate(2 * cache_bytes + 1024);
            m.kc = m.kv_pool.get();
            m.vc = m.kv_pool.as<char>() + cache_bytes;
            if (bf) {
                throw_on(sfb_k_convert(dk, SFB_F32, m.kc, SFB_BF16, static_cast<int64_t>(lk.size()), s));
                throw_on(sfb_k_convert(dv, SFB_F32, m.vc, SFB_BF16, static_cast<int64_t>(lv.size()), s));
            } else {
                cuda_check(cudaMemcpyAsync(m.kc, dk, cache_bytes, cudaMemcpyDeviceToDevice, s), "cache copy");
                cuda_check(cudaMemcpyAsync(m.vc, dv, cache_bytes, cudaMemcpyDeviceToDevice, s), "cache copy");
            }
            cuda_check(cudaStreamSynchronize(s), "cache build");
            plan->attention_strategy = "io_aware";
        }
    } else {
        plan->attention_strategy = "io_aware";
    }

    // ---- activations: one workspace with lifetime-based reuse --------------------------------
    const auto plan_start = std::chrono::steady_clock::now();
    const std::size_t e = m.esz();
    auto& wp = m.planner;
    const std::size_t TH = static_cast<std::size_t>(T) * H;
    // The layer input stays resident for the whole pass so that the plan can be re-run.
    m.pipeline_chunks = 1;
    // Causal attention of rows [r0, r1) of a sequence needs its keys [0, r1), which the chunks before have
    // produced, so a chunk may be any row range; only the tensor-core attention kernel takes such slices.
    const bool row_chunks = c.causal && D == 128 && c.sequence % 128 == 0 && plan->policy.attention_backend != 1;
    const std::vector<int> row_blocks = pipelined_row_blocks(T, H, sm_count());
    if (bf && fused && !moe && !m.decode && opt.no_pipeline == 0 && G == 1 && row_chunks && !row_blocks.empty()) {
        int row = 0;
        for (int size : row_blocks) {
            m.pipeline_ranges.push_back({row, size * 128});
            row += size * 128;
        }
        m.pipeline_chunks = static_cast<int>(m.pipeline_ranges.size());
    } else if (bf && fused && !moe && !m.decode && c.batch >= 2 && opt.no_pipeline == 0) {
        m.pipeline_chunks = c.batch;
        while (m.pipeline_chunks > 8 || c.batch % m.pipeline_chunks != 0) --m.pipeline_chunks;
        const int per_chunk = c.batch / m.pipeline_chunks * c.sequence;
        for (int i = 0; i < m.pipeline_chunks; ++i) m.pipeline_ranges.push_back({i * per_chunk, per_chunk});
        // the first and the last chunk cut short: 512 rows at the head of the first sequence and at the tail
        // of the last one
        const int edge = 512;
        if (row_chunks && per_chunk == c.sequence && c.sequence >= 2 * edge && c.sequence % 256 == 0) {
            std::vector<std::pair<int, int>> ranges;
            ranges.push_back({0, edge});
            ranges.push_back({edge, c.sequence - edge});
            for (int i = 1; i + 1 < m.pipeline_chunks; ++i) ranges.push_back(m.pipeline_ranges[i]);
            const int last = (m.pipeline_chunks - 1) * c.sequence;
            ranges.push_back({last, c.sequence - edge});
            ranges.push_back({last + c.sequence - edge, edge});
            m.pipeline_ranges = ranges;
            m.pipeline_chunks = static_cast<int>(ranges.size());
        }
    }
    const bool piped = m.pipeline_chunks > 1;  // host copies overlap compute: I/O staging must not alias anything
    wp.add("input_f32", TH * 4, 0, (bf && !piped) ? 0 : 13);
    if (bf) wp.add("input", TH * e, 0, 13);
    if (!m.fold1) wp.add("normalized1", TH * e, 1, 2);
    // sums of squares per row for the folded norms; they live for the whole pass (the first one as long as the
    // resident input, the second one keeps the zeros that a ragged column group never overwrites)
    if (m.fold1) wp.add("ss1", static_cast<std::size_t>(T) * 4, 0, 13);
    if (m.fold2) wp.add("ss2", static_cast<std::size_t>(T) * 8, 0, 13);  // 64-bit fixed point (one shard) or float (sharded)
    if (!fused) wp.add("fused_qkv", static_cast<std::size_t>(T) * m.qkv_l * e, 2, 3);
    wp.add("query", static_cast<std::size_t>(T) * m.hidden_l * e, 2, 4);
    // chunks that are part of a sequence attend to the keys and values of the chunks before them
    bool sliced = false;
    for (const auto& range : m.pipeline_ranges)
        sliced = sliced || range.first % c.sequence != 0 || range.second % c.sequence != 0;
    wp.add("key", static_cast<std::size_t>(T) * m.kvw_l * e, 2, sliced ? 13 : 4);
    wp.add("value", static_cast<std::size_t>(T) * m.kvw_l * e, 2, sliced ? 13 : 4);
    if (m.paged)
        wp.add("decode_partials", sfb_attention_decode_workspace(c.batch, m.hq, D, m.splits), 4, 4);
    wp.add("attention", static_cast<std::size_t>(T) * m.hidden_l * e, 4, 5);
    if (!fused) wp.add("projected", TH * e, 5, 6);
    wp.add("attention_residual", TH * e, 5, 12);
    if (!m.fold2) wp.add("normalized2", TH * e, 7, 9);
    if (!moe) {
        if (!fused) wp.add("gate_up", static_cast<std::size_t>(T) * 2 * I * e, 8, 9);
        // the fused down projection reads it while it writes "output" (step 11): the two must not share bytes
        wp.add("activation", static_cast<std::size_t>(T) * I * e, 8, fused ? 11 : 10);
        if (!fused) wp.add("down", TH * e, 10, 11);
    } else {
        const std::size_t A = static_cast<std::size_t>(T) * m.K;
        wp.add("expert_ids", A * 4, 8, 12);
        wp.add("expert_weights", A * 4, 8, 12);
        wp.add("counts", static_cast<std::size_t>(m.E) * 4, 8, 12);
        wp.add("offsets", static_cast<std::size_t>(m.E + 1) * 4, 8, 12);
        wp.add("token_ids", A * 4, 8, 12);
        wp.add("route_slots", A * 4, 8, 12);
        wp.add("routing_weights", A * 4, 8, 12);
        wp.add("dest_of", A * 4, 8, 12);
        wp.add("dispatch_scratch", sfb_moe_dispatch_scratch_bytes(T, m.E, m.K), 8, 9);
        if (G > 1) {  // expert-parallel tables (see moe_ep.cu)
            wp.add("ep_send_base", static_cast<std::size_t>(m.E) * 4, 8, 12);
            wp.add("ep_recv_offsets", static_cast<std::size_t>(m.E_l + 1) * 4, 8, 12);
            wp.add("ep_return_table", static_cast<std::size_t>(m.E_l) * G * 16, 8, 12);
        }
        wp.add("tile_table", sizeof(int) * 4 * (A / 128 + m.E + 2), 9, 11);
        wp.add("dispatched", A * H * e, 8, 10);
        if (bf) {
            wp.add("expert_activation", A * I * e, 9, 10);
        } else {
            wp.add("expert_first", A * I * e, 9, 10);
            wp.add("expert_gate", A * I * e, 9, 10);
        }
        wp.add("expert_output", A * H * e, 10, 11);
    }
    if (bf && T <= 128 && opt.fixed_order == 0)  // partial tile sums of the weight-streaming GEMMs; zero between kernels
        wp.add("gemm_partials", sfb_gemm_stream_workspace_bytes(std::max({m.qkv_l, H, 2 * I})), 0, 13);
    wp.add("output", TH * e, 11, 13);
    if (bf) wp.add("output_f32", TH * 4, piped ? 0 : (m.direct_f32_output ? 10 : 12), 13);  // written by the last GEMM when direct
    m.workspace.allocate(wp.total_bytes());
    if (m.has("gemm_partials"))
        cuda_check(cudaMemsetAsync(m.ws("gemm_partials"), 0, wp.bytes(wp.find("gemm_partials")), s), "scratch clear");
    if (m.fold2) cuda_check(cudaMemsetAsync(m.ws("ss2"), 0, wp.bytes(wp.find("ss2")), s), "sums clear");
    plan->naive_bytes = wp.naive_bytes();
    plan->workspace_bytes = wp.total_bytes();
    (void)plan_start;
    for (auto& ev : m.events) cuda_check(cudaEventCreate(&ev), "cudaEventCreate");
    m.status_device = device_status_word();
    cuda_check(cudaHostAlloc(reinterpret_cast<void**>(&m.status_host), sizeof(uint32_t), cudaHostAllocDefault), "status word");
    *m.status_host = 0;
    if (piped) {
        cuda_check(cudaStreamCreateWithFlags(&m.copy_in, cudaStreamNonBlocking), "cudaStreamCreate");
        cuda_check(cudaMalloc(reinterpret_cast<void**>(&m.chunk_flags), sizeof(uint32_t) * m.pipeline_chunks), "chunk flags");
        cuda_check(cudaMemset(m.chunk_flags, 0, sizeof(uint32_t) * m.pipeline_chunks), "chunk flags");
        cuda_check(cudaHostAlloc(reinterpret_cast<void**>(&m.upload_epoch_host), sizeof(uint32_t), cudaHostAllocDefault), "epoch word");
        cuda_check(cudaStreamCreateWithFlags(&m.copy_out, cudaStreamNonBlocking), "cudaStreamCreate");
        m.chunk_events.resize(static_cast<std::size_t>(m.pipeline_chunks) * 7);
        for (auto& ev : m.chunk_events) cuda_check(cudaEventCreate(&ev), "cudaEventCreate");
    }
    plan->compile_milliseconds =
        std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    return plan;
}

std::size_t DecoderExecutablePlan::peer_bytes() const {
    const auto& m = *impl_;
    return m.size > 1 ? m.peer_total_bytes() : 0;
}

void DecoderExecutablePlan::set_peer_allreduce(void* local_base, void* const* peer_bases, int mode) {
    auto& m = *impl_;
    m.input_in_peer = false;
    if (!local_base) {  // back to the hook
        m.peer_local = nullptr;
        m.peer_mode = 0;
        return;
    }
    if (mode < 0 || mode > 3) throw std::invalid_argument("peer all-reduce: unknown mode");
    const bool can_two_shot = m.T % std::max(1, m.size) == 0 && m.H % 8 == 0;
    if (mode >= 2 && !can_two_shot) throw std::invalid_argument("two-shot peer all-reduce needs rows divisible by the rank count");
    // the copy-engine all-gather needs whole 128-row tiles per owner (the GEMM that consumes the rows waits per owner)
    const bool can_overlap = can_two_shot && config.ffn == DecoderFFNKind::Dense && (m.T / std::max(1, m.size)) % 128 == 0;
    if (mode == 3 && !can_overlap) throw std::invalid_argument("the overlapped all-gather needs a dense plan with 128-row multiples per rank");
    // one-shot pushes (size - 1) x the tensor per rank: right for the small outputs of decode plans and for two ranks
    // of a dense layer; an MoE layer wants the row ownership of the two-shot form at any rank count (its experts then
    // see only the tokens routed to them instead of every rank's replica of all tokens)
    const bool moe_rows = config.ffn != DecoderFFNKind::Dense;
    if (mode == 0) mode = (can_two_shot && m.T > 128 && (m.size > 2 || moe_rows)) ? (can_overlap ? 3 : 2) : 1;
    if (mode == 3 && !m.ce_stream) {
        cuda_check(cudaStreamCreateWithFlags(&m.ce_stream, cudaStreamNonBlocking), "cudaStreamCreate");
        cuda_check(cudaEventCreateWithFlags(&m.ce_ready, cudaEventDisableTiming), "cudaEventCreate");
        cuda_check(cudaEventCreateWithFlags(&m.ce_done, cudaEventDisableTiming), "cudaEventCreate");
    }
    if (m.size < 2 || m.size > SFB_MAX_PEERS) throw std::invalid_argument("peer all-reduce needs a sharded plan of 2..8 ranks");
    if (m.dtype != SFB_BF16 || !policy.fuse_epilogues || policy.gemm_backend == SFB_GEMM_SIMT || m.H % 8 != 0 ||
        m.hidden_l % 8 != 0 || m.I_l % 8 != 0)
        throw std::invalid_argument("peer all-reduce needs a bf16 plan with fused epilogues on the tcgen05 GEMM");
    if (!peer_bases) throw std::invalid_argument("peer all-reduce: null peer table");
    for (int s = 0; s < m.size; ++s) {
        if (s != m.rank && !peer_bases[s]) throw std::invalid_argument("peer all-reduce: null peer buffer");
        m.peer_remote[s] = static_cast<char*>(peer_bases[s]);
    }
    m.peer_local = static_cast<char*>(local_base);
    m.peer_mode = mode;
    m.peer_epoch[0] = m.peer_epoch[1] = 0;
    for (auto& epoch : m.gather_epoch) epoch = 0;
}

void DecoderExecutablePlan::upload_input(const float* input) {
    if (!input) throw std::invalid_argument("decoder input is null");
    auto& m = *impl_;
    m.input_in_peer = false;
    cuda_check(cudaMemcpyAsync(m.ws<float>("input_f32"), input, static_cast<std::size_t>(m.T) * m.H * 4,
                               cudaMemcpyHostToDevice, stream_), "input upload");
    if (m.dtype == SFB_BF16) {
        if (m.fold1)  // the conversion also leaves the sums of squares of the rounded rows for the folded first norm
            throw_on(sfb_k_convert_rows_sumsq(m.ws<float>("input_f32"), m.ws("input"), m.ws<float>("ss1"), m.T, m.H, stream_));
        else
            throw_on(sfb_k_convert(m.ws("input_f32"), SFB_F32, m.ws("input"), SFB_BF16,
                                   static_cast<int64_t>(m.T) * m.H, stream_));
    }
    m.has_input = true;
}

void DecoderExecutablePlan::download_output(float* output) {
    if (!output) throw std::invalid_argument("decoder output is null");
    auto& m = *impl_;
    const float* src = m.dtype == SFB_BF16 ? m.ws<float>("output_f32") : m.ws<float>("output");
    m.materialize_output(0, m.T, stream_);
    m.queue_status_read(stream_);
    cuda_check(cudaMemcpyAsync(output, src, static_cast<std::size_t>(m.T) * m.H * 4, cudaMemcpyDeviceToHost, stream_),
               "output download");
    cuda_check(cudaStreamSynchronize(stream_), "output download sync");
    m.check_status(stream_);
}

void DecoderExecutablePlan::run(cudaStream_t s, RoutingTraceView trace, bool stage_events) {
    auto& m = *impl_;
    if (!m.has_input) throw std::invalid_argument("decoder input has not been uploaded");
    const DecoderConfig& c = config;
    const bool bf = m.dtype == SFB_BF16, fused = policy.fuse_epilogues, moe = c.ffn == DecoderFFNKind::MoE;
    const auto dt = static_cast<sfb_dtype>(m.dtype);
    const int T = m.T, H = m.H, I = m.I_l, D = m.D;
    int ev = 0;
    auto mark = [&] { if (stage_events) cuda_check(cudaEventRecord(m.events[ev++], s), "event"); };
    // the rotary table advanced to the position of the (one) new token of an appending decode plan
    const int position = m.append_new ? m.kv_length : 0;
    const std::size_t rope_shift = static_cast<std::size_t>(position) * static_cast<std::size_t>(std::max(1, D / 2));
    using Tweak = void (*)(sfb_gemm_args&, DecoderExecutablePlan::Impl&, int);
    auto gemm = [&](const void* a, const void* w, void* out, int mm, int n, int k, int epi, const void* res = nullptr,
                    int sb = 0, const int* offsets = nullptr, int groups = 0, bool f32_out = false, int peer_set = -1,
                    Tweak tweak = nullptr) {
        if (!bf) {
            throw_on(sfb_k_gemm_f32(static_cast<const float*>(a), static_cast<const float*>(w),
                                    static_cast<float*>(out), mm, n, k, s));
            return;
        }
        sfb_gemm_args g{};
        g.a = a; g.bt = w; g.out = out; g.m = mm; g.n = n; g.k = k; g.epilogue = epi;
        g.backend = policy.gemm_backend; g.residual = res; g.swiglu_block = sb; g.out_f32 = f32_out ? 1 : 0;
        if (epi == SFB_EPI_ROPE_SPLIT) {
            g.q = m.ws("query"); g.key = m.ws("key"); g.value = m.ws("value");
            g.rope_cos = m.rope_cos + rope_shift; g.rope_sin = m.rope_sin + rope_shift;
            g.batch = c.batch; g.seq = c.sequence; g.q_heads = m.hq; g.kv_heads = m.hkv; g.head_dim = D;
        }
        if (tweak) tweak(g, m, T);
        if (offsets) { g.group_offsets = offsets; g.groups = groups; g.tile_table = m.ws("tile_table"); }
        if (m.has("gemm_partials")) {
            g.split_workspace = m.ws("gemm_partials");
            g.split_workspace_bytes = m.planner.bytes(m.planner.find("gemm_partials"));
        }
        g.bt_tiled = m.blocked(w) ? 1 : 0;
        if (const auto* quantized = m.int8(w)) {
            g.bt = quantized->q;
            g.bt_scales = quantized->scales;
        }
        if (peer_set >= 0) m.fill_peer_out(g, peer_set, 0);
        throw_on(sfb_k_gemm_bf16(&g, s));
    };
    auto allreduce = [&](void* buffer, int64_t count) {
        if (m.size > 1 && allreduce_) allreduce_(allreduce_user_, buffer, count, m.dtype, s);
    };
    const bool peer = m.size > 1 && m.peer_local != nullptr;
    auto peer_finish = [&](int peer_set, void* buffer, int64_t count) { throw_on(m.peer_finish(peer_set, buffer, 0, count, s)); };

    // QKV GEMM with the first RMSNorm folded in (1/rms from the sums of squares the input conversion left) and, in an
    // appending decode plan, the new token's K/V written into the paged cache by the same epilogue
    const Tweak qkv_tweak = [](sfb_gemm_args& g, DecoderExecutablePlan::Impl& im, int rows) {
        if (im.fold1) {
            g.row_ss = im.cur_ss1; g.rms_epsilon = im.rms_eps;
        }
        if (im.fold2 && im.size == 1) {  // the sums the O projection of this pass will add to start at zero
            g.clear = im.ws("ss2"); g.clear_bytes = static_cast<std::size_t>(rows) * 8;
        }
        if (im.kv_in_epilogue) {
            g.kv_k_pool = im.k_pool; g.kv_v_pool = im.v_pool; g.kv_table = im.block_table;
            g.kv_position = im.kv_length; g.kv_block_tokens = im.page_tokens; g.kv_max_blocks = im.max_blocks;
            g.kv_num_blocks = im.num_blocks;
        }
    };
    m.rms_eps = c.rms_epsilon;
    const bool two = m.two_shot();
    mark();  // 0
    void* x = bf ? m.ws("input") : m.ws("input_f32");
    if (two && m.input_in_peer) x = m.gathered(0);  // the rows every rank contributed, gathered by peer stores
    m.cur_ss1 = m.fold1 ? (two && m.input_in_peer ? m.gathered_ss(0) : m.ws<float>("ss1")) : nullptr;
    void* a1 = x;
    if (!m.fold1) {
        a1 = m.ws("normalized1");
        throw_on(sfb_k_rms_norm(x, m.rms1, a1, T, H, c.rms_epsilon, dt, s));
    }
    mark();  // 1: norm
    const bool rope_fused = fused && D % 2 == 0;
    if (rope_fused) {
        gemm(a1, m.wqkv, nullptr, T, m.qkv_l, H, SFB_EPI_ROPE_SPLIT, nullptr, 0, nullptr, 0, false, -1, qkv_tweak);
        mark(); mark();  // 2: projection, 3: (rope inside)
    } else {
        gemm(a1, m.wqkv, m.ws("fused_qkv"), T, m.qkv_l, H, SFB_EPI_STORE);
        mark();  // 2
        throw_on(sfb_k_rope_split(m.ws("fused_qkv"), m.ws("query"), m.ws("key"), m.ws("value"), m.rope_cos + rope_shift,
                                  m.rope_sin + rope_shift, c.batch, c.sequence, m.hq, m.hkv, D, dt, s));
        mark();  // 3
    }
    if (m.paged) {
        if (m.append_new && !(m.kv_in_epilogue && rope_fused)) {
            // the rotated key and the value of the new token go to position kv_length of every sequence
            if (m.len_uploaded != m.kv_length) {
                for (int b = 0; b < c.batch; ++b) m.len_pinned[b] = m.kv_length;
                cuda_check(cudaMemcpyAsync(m.context_len, m.len_pinned, sizeof(int) * c.batch, cudaMemcpyHostToDevice, s), "lengths");
                m.len_uploaded = m.kv_length;
            }
            throw_on(sfb_k_paged_kv_append(m.ws("key"), m.ws("value"), m.k_pool, m.v_pool, m.block_table, m.context_len,
                                           c.batch, m.hkv, 1, D, D, m.page_tokens, m.max_blocks, m.num_blocks, dt, s));
        }
        sfb_decode_args a{};
        a.q = m.ws("query"); a.k_pool = m.k_pool; a.v_pool = m.v_pool; a.block_table = m.block_table;
        a.context_len = nullptr; a.uniform_context = m.kv_length + (m.append_new ? 1 : 0);  // the batch decodes in lock step
        a.out = m.ws("attention"); a.partials = m.ws("decode_partials");
        a.batch = c.batch; a.q_heads = m.hq; a.kv_heads = m.hkv; a.head_dim = D; a.head_dim_value = D;
        a.block_tokens = m.page_tokens; a.max_blocks = m.max_blocks; a.num_blocks = m.num_blocks;
        a.max_context = m.kv_capacity; a.splits = m.splits; a.scale = 0.0F; a.dtype = m.dtype;
        throw_on(sfb_k_attention_decode_paged(&a, s));
    } else {
        sfb_attention_args a{};
        a.q = m.ws("query");
        a.key = m.decode ? m.kc : m.ws("key");
        a.value = m.decode ? m.vc : m.ws("value");
        a.out = m.ws("attention");
        a.batch = c.batch; a.q_heads = m.hq; a.kv_heads = m.hkv; a.seq_q = c.sequence;
        a.seq_kv = m.decode ? c.context_sequence : c.sequence; a.head_dim = D; a.head_dim_value = D;
        a.causal = c.causal; a.scale = 0.0F; a.token_major = 1; a.dtype = m.dtype;
        a.backend = policy.attention_backend;
        throw_on(sfb_k_attention_prefill(&a, s));
    }
    mark();  // 4: attention
    void* r1 = two ? m.gathered(1) : m.ws("attention_residual");
    const bool add_residual_here = m.rank == 0;  // under sharding the residual enters the sum once
    const std::size_t own_rows_offset = two ? static_cast<std::size_t>(m.rank) * (T / m.size) * H * 2 : 0;
    // second fold: a single shard collects the sums of squares of attention_residual in the O epilogue; a
    // sharded plan sums the squares of the reduced rows after its all-reduce
    const Tweak o_tweak = [](sfb_gemm_args& g, DecoderExecutablePlan::Impl& im, int rows) {
        if (im.fold2 && im.size == 1) g.ss_out = im.ws("ss2");
    };
    m.cur_ss2 = m.fold2 ? (two ? static_cast<const void*>(m.gathered_ss(1)) : m.ws("ss2")) : nullptr;
    m.cur_ss2_fixed = m.size == 1;
    const Tweak gate_up_tweak = [](sfb_gemm_args& g, DecoderExecutablePlan::Impl& im, int rows) {
        if (im.fold2) {
            g.row_ss = im.cur_ss2; g.row_ss_fixed = im.cur_ss2_fixed ? 1 : 0; g.rms_epsilon = im.rms_eps;
        }
        if (im.ce_gather()) {  // rows of the other owners may still be on their way: wait per owner, own rows first
            g.owner_flags = im.ce_flags(im.rank, 1); g.owner_epoch = im.gather_epoch[1];
            g.owner_rows = rows / im.size; g.owner_self = im.rank;
        }
    };
    if (fused) {
        if (two) {
            // the partial tensor stays in this rank's peer-visible memory; every owner fetches its rows from all ranks,
            // adds them up with its rows of the residual stream, takes the sums of squares and hands the finished
            // rows to everybody
            gemm(m.ws("attention"), m.wo, m.partial(0), T, H, m.hidden_l, SFB_EPI_STORE);
            // (an expert-parallel MoE layer keeps the reduced rows with their owner: its FFN half is token sharded)
            const bool ce = m.ce_gather();
            throw_on(m.reduce_gather(1, nullptr, nullptr, static_cast<const char*>(x) + own_rows_offset, m.fold2, s,
                                     moe || ce ? 0 : 1, ce ? m.ce_epoch_word(1) : nullptr));
            if (ce) m.ce_push(1, m.fold2, s);  // the other ranks' rows arrive while the gate/up GEMM runs
        } else if (peer) {
            gemm(m.ws("attention"), m.wo, r1, T, H, m.hidden_l, add_residual_here ? SFB_EPI_RESIDUAL : SFB_EPI_STORE, x, 0,
                 nullptr, 0, false, 0);
            peer_finish(0, r1, static_cast<int64_t>(T) * H);
        } else {
            gemm(m.ws("attention"), m.wo, r1, T, H, m.hidden_l, add_residual_here ? SFB_EPI_RESIDUAL : SFB_EPI_STORE, x, 0,
                 nullptr, 0, false, -1, o_tweak);
            allreduce(r1, static_cast<int64_t>(T) * H);
        }
        if (m.fold2 && m.size > 1 && !two) throw_on(sfb_k_row_sumsq(r1, m.ws<float>("ss2"), T, H, s));
        mark(); mark();  // 5: projection, 6: (residual inside)
    } else {
        gemm(m.ws("attention"), m.wo, m.ws("projected"), T, H, m.hidden_l, SFB_EPI_STORE);
        allreduce(m.ws("projected"), static_cast<int64_t>(T) * H);
        mark();  // 5
        throw_on(sfb_k_add(m.ws("projected"), x, r1, static_cast<int64_t>(T) * H, dt, s));
        mark();  // 6
    }
    const bool ep = two && moe;   // token-sharded expert parallelism (all-to-all dispatch / combine over peer stores)
    void* a2 = r1;
    if (!m.fold2 && !ep) {
        a2 = m.ws("normalized2");
        throw_on(sfb_k_rms_norm(r1, m.rms2, a2, T, H, c.rms_epsilon, dt, s));
    }
    mark();  // 7: norm
    void* out = two ? m.gathered(2) : m.ws("output");
    if (!moe) {
        if (fused) {
            gemm(a2, m.wgu, m.ws("activation"), T, 2 * I, H, SFB_EPI_SWIGLU, nullptr, m.swiglu_block, nullptr, 0, false, -1,
                 gate_up_tweak);
            if (m.direct_f32_output) {
                gemm(m.ws("activation"), m.wd, m.ws("output_f32"), T, H, I, SFB_EPI_RESIDUAL, r1, 0, nullptr, 0, true);
            } else if (two) {
                gemm(m.ws("activation"), m.wd, m.partial(1), T, H, I, SFB_EPI_STORE);
                const bool ce = m.ce_gather();
                throw_on(m.reduce_gather(2, nullptr, nullptr, static_cast<const char*>(r1) + own_rows_offset, false, s, ce ? 0 : 1,
                                         ce ? m.ce_epoch_word(2) : nullptr));
                if (ce) {  // nothing in this layer reads the gathered output: send it and wait for the peers' rows
                    m.ce_push(2, false, s);
                    throw_on(sfb_k_peer_wait(m.ce_flags(m.rank, 2), m.rank, m.size, m.gather_epoch[2], s));
                }
            } else if (peer) {
                gemm(m.ws("activation"), m.wd, out, T, H, I, add_residual_here ? SFB_EPI_RESIDUAL : SFB_EPI_STORE, r1, 0,
                     nullptr, 0, false, 1);
                peer_finish(1, out, static_cast<int64_t>(T) * H);
            } else {
                gemm(m.ws("activation"), m.wd, out, T, H, I, add_residual_here ? SFB_EPI_RESIDUAL : SFB_EPI_STORE, r1);
                allreduce(out, static_cast<int64_t>(T) * H);
            }
            mark(); mark();  // 8: ffn, 9: (residual inside)
        } else {
            gemm(a2, m.wgu, m.ws("gate_up"), T, 2 * I, H, SFB_EPI_STORE);
            throw_on(sfb_k_swiglu(m.ws("gate_up"), m.ws("activation"), T, I, dt, s));
            gemm(m.ws("activation"), m.wd, m.ws("down"), T, H, I, SFB_EPI_STORE);
            allreduce(m.ws("down"), static_cast<int64_t>(T) * H);
            mark();  // 8
            throw_on(sfb_k_add(r1, m.ws("down"), out, static_cast<int64_t>(T) * H, dt, s));
            mark();  // 9
        }
    } else if (ep) {
        // This rank's tokens only: norm, router, stable local dispatch; the histograms go round, every dispatched row
        // travels to the owner of its expert, the grouped GEMMs run on what arrived, the outputs travel back, the
        // owner of the token combines them with the residual, and the finished rows are gathered on every rank.
        const int rows_own = T / m.size, A_own = rows_own * m.K, Ifull = c.intermediate;
        const int capacity = static_cast<int>(m.ep_capacity());
        char* r1_own = static_cast<char*>(r1) + own_rows_offset;
        char* n2_own = static_cast<char*>(m.ws("normalized2")) + own_rows_offset;
        throw_on(sfb_k_rms_norm(r1_own, m.rms2, n2_own, rows_own, H, c.rms_epsilon, dt, s));
        int* ids = m.ws<int>("expert_ids");
        float* wts = m.ws<float>("expert_weights");
        int* counts = m.ws<int>("counts");
        if (trace) {  // the caller's trace covers all tokens: this rank takes its rows of it
            validate_routing_trace(T, m.K, m.E, trace.expert_ids, trace.expert_weights, trace.counts);
            const std::size_t first = static_cast<std::size_t>(m.rank) * A_own;
            m.trace_counts.assign(static_cast<std::size_t>(m.E), 0);
            for (int i = 0; i < A_own; ++i) ++m.trace_counts[static_cast<std::size_t>(trace.expert_ids[first + i])];
            cuda_check(cudaMemcpyAsync(ids, trace.expert_ids + first, sizeof(int) * A_own, cudaMemcpyHostToDevice, s), "trace upload");
            cuda_check(cudaMemcpyAsync(wts, trace.expert_weights + first, sizeof(float) * A_own, cudaMemcpyHostToDevice, s), "trace upload");
            cuda_check(cudaMemcpyAsync(counts, m.trace_counts.data(), sizeof(int) * m.E, cudaMemcpyHostToDevice, s), "trace upload");
            cuda_check(cudaStreamSynchronize(s), "trace upload sync");  // the host vector is reused by the next pass
        } else {
            throw_on(sfb_k_moe_route(n2_own, dt, m.router, m.router_bias, rows_own, H, m.E, m.K, ids, wts, counts, s));
        }
        int* offsets = m.ws<int>("offsets");
        throw_on(sfb_k_moe_dispatch(nullptr, dt, ids, wts, counts, rows_own, H, m.E, m.K, nullptr, offsets,
                                    m.ws<int>("token_ids"), m.ws<int>("route_slots"), m.ws<float>("routing_weights"),
                                    m.ws<int>("dest_of"), m.ws<int>("dispatch_scratch"), s));
        sfb_moe_ep_plan_args plan_args{};
        plan_args.counts = counts;
        for (int r = 0; r < m.size; ++r) plan_args.counts_all[r] = reinterpret_cast<int*>(m.peer_base(r) + m.ep_counts_offset());
        plan_args.experts = m.E;
        plan_args.send_base = m.ws<int>("ep_send_base");
        plan_args.recv_offsets = m.ws<int>("ep_recv_offsets");
        plan_args.return_table = m.ws<int>("ep_return_table");
        plan_args.sync = m.ep_sync(3);
        throw_on(sfb_k_moe_ep_plan(&plan_args, s));
        sfb_moe_ep_send_args send{};
        send.rows = n2_own; send.offsets = offsets; send.token_ids = m.ws<int>("token_ids"); send.route_slots = m.ws<int>("route_slots");
        send.send_base = plan_args.send_base;
        for (int r = 0; r < m.size; ++r) {
            send.recv_rows[r] = m.peer_base(r) + m.ep_recv_rows_offset();
            send.recv_tokens[r] = reinterpret_cast<int*>(m.peer_base(r) + m.ep_recv_tokens_offset());
            send.recv_slots[r] = reinterpret_cast<int*>(m.peer_base(r) + m.ep_recv_slots_offset());
        }
        send.assignments = A_own; send.hidden = H; send.experts = m.E; send.first_token = m.rank * rows_own;
        send.sync = m.ep_sync(4);
        throw_on(sfb_k_moe_ep_send(&send, s));
        void* received = m.peer_local + m.ep_recv_rows_offset();
        void* y = m.ws("expert_output");
        gemm(received, m.w13, m.ws("expert_activation"), capacity, 2 * Ifull, H, SFB_EPI_SWIGLU, nullptr, m.moe_swiglu_block,
             plan_args.recv_offsets, m.E_l);
        gemm(m.ws("expert_activation"), m.w2, y, capacity, H, Ifull, SFB_EPI_STORE, nullptr, 0, plan_args.recv_offsets, m.E_l);
        sfb_moe_ep_return_args back{};
        back.rows = y; back.recv_offsets = plan_args.recv_offsets; back.return_table = plan_args.return_table;
        for (int r = 0; r < m.size; ++r) back.back[r] = m.peer_base(r) + m.ep_back_offset();
        back.hidden = H; back.experts_local = m.E_l; back.max_rows = capacity;
        back.sync = m.ep_sync(5);
        throw_on(sfb_k_moe_ep_return(&back, s));
        char* out_own = static_cast<char*>(out) + own_rows_offset;
        throw_on(sfb_k_moe_combine(m.peer_local + m.ep_back_offset(), m.ws<int>("dest_of"), m.ws<float>("routing_weights"), r1_own,
                                   out_own, rows_own, H, m.K, dt, s));
        throw_on(m.reduce_gather(2, out_own, nullptr, nullptr, false, s));  // all-gather of the finished rows
        mark(); mark();  // 8: ffn, 9
    } else {
        const int A = T * m.K, Ifull = c.intermediate;
        int* ids = m.ws<int>("expert_ids");
        float* wts = m.ws<float>("expert_weights");
        int* counts = m.ws<int>("counts");
        if (trace) {
            validate_routing_trace(T, m.K, m.E, trace.expert_ids, trace.expert_weights, trace.counts);
            cuda_check(cudaMemcpyAsync(ids, trace.expert_ids, sizeof(int) * A, cudaMemcpyHostToDevice, s), "trace upload");
            cuda_check(cudaMemcpyAsync(wts, trace.expert_weights, sizeof(float) * A, cudaMemcpyHostToDevice, s), "trace upload");
            cuda_check(cudaMemcpyAsync(counts, trace.counts, sizeof(int) * m.E, cudaMemcpyHostToDevice, s), "trace upload");
        } else {
            throw_on(sfb_k_moe_route(m.ws("normalized2"), dt, m.router, m.router_bias, T, H, m.E, m.K, ids, wts, counts, s));
        }
        int* offsets = m.ws<int>("offsets");
        throw_on(sfb_k_moe_dispatch(m.ws("normalized2"), dt, ids, wts, counts, T, H, m.E, m.K, m.ws("dispatched"), offsets,
                                    m.ws<int>("token_ids"), m.ws<int>("route_slots"), m.ws<float>("routing_weights"),
                                    m.ws<int>("dest_of"), m.ws<int>("dispatch_scratch"), s));
        void* y = m.ws("expert_output");
        if (m.size > 1) cuda_check(cudaMemsetAsync(y, 0, static_cast<std::size_t>(A) * H * m.esz(), s), "expert output clear");
        if (bf) {
            gemm(m.ws("dispatched"), m.w13, m.ws("expert_activation"), A, 2 * Ifull, H, SFB_EPI_SWIGLU, nullptr,
                 m.moe_swiglu_block, offsets + m.e_begin, m.E_l);
            gemm(m.ws("expert_activation"), m.w2, y, A, H, Ifull, SFB_EPI_STORE, nullptr, 0, offsets + m.e_begin, m.E_l);
        } else {
            // fp32 plan: exact-order GEMM per expert segment; the segment bounds come back to the host.
            std::vector<int> host_offsets(m.E + 1);
            cuda_check(cudaMemcpyAsync(host_offsets.data(), offsets, sizeof(int) * (m.E + 1), cudaMemcpyDeviceToHost, s), "offsets");
            cuda_check(cudaStreamSynchronize(s), "offsets sync");
            float* xs = m.ws<float>("dispatched");
            float* first = m.ws<float>("expert_first");
            float* gate = m.ws<float>("expert_gate");
            const std::size_t ee = static_cast<std::size_t>(H) * Ifull;
            for (int e = 0; e < m.E_l; ++e) {
                const int lo = host_offsets[m.e_begin + e], rows = host_offsets[m.e_begin + e + 1] - lo;
                if (rows <= 0) continue;
                throw_on(sfb_k_gemm_f32(xs + static_cast<std::size_t>(lo) * H, m.w1f + e * ee, first + static_cast<std::size_t>(lo) * Ifull, rows, Ifull, H, s));
                throw_on(sfb_k_gemm_f32(xs + static_cast<std::size_t>(lo) * H, m.w3f + e * ee, gate + static_cast<std::size_t>(lo) * Ifull, rows, Ifull, H, s));
            }
            // first *= silu(gate) over every dispatched row (src/moe_compiler.cpp:146-149)
            moe_silu_mul_f32(first, gate, static_cast<int64_t>(A) * Ifull, s);
            for (int e = 0; e < m.E_l; ++e) {
                const int lo = host_offsets[m.e_begin + e], rows = host_offsets[m.e_begin + e + 1] - lo;
                if (rows <= 0) continue;
                throw_on(sfb_k_gemm_f32(first + static_cast<std::size_t>(lo) * Ifull, m.w2f + e * ee,
                                        static_cast<float*>(y) + static_cast<std::size_t>(lo) * H, rows, H, Ifull, s));
            }
        }
        throw_on(sfb_k_moe_combine(y, m.ws<int>("dest_of"), m.ws<float>("routing_weights"),
                                   add_residual_here ? r1 : nullptr, out, T, H, m.K, dt, s));
        allreduce(out, static_cast<int64_t>(T) * H);
        mark(); mark();  // 8: ffn, 9
    }
    // The layer's product on the device is the bf16 output (what a next layer would read).  A single shard also
    // leaves the fp32 copy the host calls hand out; a sharded plan converts only the rows a host call asks for,
    // instead of every rank converting the whole replicated tensor on every pass.
    if (m.ce_pending) {  // the pass is over when this rank's outgoing copies are, too
        cuda_check(cudaEventRecord(m.ce_done, m.ce_stream), "event");
        cuda_check(cudaStreamWaitEvent(s, m.ce_done, 0), "stream wait");
        m.ce_pending = false;
    }
    m.output_bf16 = out;
    m.output_f32_valid = !bf || m.direct_f32_output || m.size == 1;
    if (bf && !m.direct_f32_output && m.size == 1)
        throw_on(sfb_k_convert(out, SFB_BF16, m.ws("output_f32"), SFB_F32, static_cast<int64_t>(T) * H, s));
    mark();  // 10
}

void DecoderExecutablePlan::execute(const float* input, float* output, RoutingTraceView trace,
                                    sfb_decoder_result* result) {
    auto& m = *impl_;
    cudaStream_t s = stream_;
    const uint64_t launches_before = sfb_launch_count();
    if (m.pipeline_chunks > 1 && !trace) {
        execute_pipelined(input, output, result);
        if (result) result->kernel_launches = sfb_launch_count() - launches_before;
        return;
    }
    cudaEvent_t h0 = m.events[12], h1 = m.events[13], d0 = m.events[14], d1 = m.events[15];
    cuda_check(cudaEventRecord(h0, s), "event");
    upload_input(input);
    cuda_check(cudaEventRecord(h1, s), "event");
    run(s, trace, true);
    cuda_check(cudaEventRecord(d0, s), "event");
    download_output(output);
    cuda_check(cudaEventRecord(d1, s), "event");
    cuda_check(cudaEventSynchronize(d1), "event sync");
    if (!result) return;
    auto span = [&](cudaEvent_t a, cudaEvent_t b) {
        float ms = 0.0F;
        cuda_check(cudaEventElapsedTime(&ms, a, b), "event time");
        return static_cast<double>(ms);
    };
    auto* e = m.events;
    *result = {};
    result->h2d_milliseconds = span(h0, h1);
    result->d2h_milliseconds = span(d0, d1);
    result->norm_rope_milliseconds = span(e[0], e[1]) + span(e[2], e[3]) + span(e[6], e[7]);
    result->projection_milliseconds = span(e[1], e[2]) + span(e[4], e[5]);
    result->attention_milliseconds = span(e[3], e[4]);
    result->residual_milliseconds = span(e[5], e[6]) + span(e[8], e[9]);
    result->ffn_milliseconds = span(e[7], e[8]);
    result->milliseconds = span(h0, d1);
    result->tokens_per_second = result->milliseconds > 0.0 ? m.T * 1000.0 / result->milliseconds : 0.0;
    result->kernel_launches = sfb_launch_count() - launches_before;
}

void DecoderExecutablePlan::step(const float* input, float* output, sfb_decoder_result* result) {
    auto& m = *impl_;
    if (!m.paged || !m.append_new) throw std::invalid_argument("decoder step needs a decode plan compiled with append_new_token");
    if (m.kv_length + 1 > m.kv_capacity) throw std::invalid_argument("paged KV capacity exceeded");
    // append_paged_kv: a token that opens a new page takes it from the back of the free list; the device table
    // already holds that entry (sync_table lays the free pages out in hand-out order)
    const int last_page = m.kv_length / m.page_tokens;
    std::vector<int> taken;
    while (static_cast<int>(m.page_table.size()) <= last_page) {
        if (m.free_pages.empty()) {
            for (auto it = taken.rbegin(); it != taken.rend(); ++it) { m.free_pages.push_back(*it); m.page_table.pop_back(); }
            throw std::runtime_error("paged KV page allocator exhausted");
        }
        taken.push_back(m.free_pages.back());
        m.page_table.push_back(m.free_pages.back());
        m.free_pages.pop_back();
    }
    execute(input, output, RoutingTraceView{}, result);  // appends at kv_length, attends over kv_length + 1
    m.kv_length += 1;
}

void DecoderExecutablePlan::kv_info(int* info, int* page_table, int table_capacity, int* free_pages, int free_capacity) const {
    const auto& m = *impl_;
    if (!m.paged || !info) throw std::invalid_argument("plan has no paged KV cache");
    info[0] = m.kv_length;
    info[1] = static_cast<int>(m.page_table.size());
    info[2] = static_cast<int>(m.free_pages.size());
    info[3] = m.max_blocks;
    for (int i = 0; page_table && i < info[1] && i < table_capacity; ++i) page_table[i] = m.page_table[i];
    for (int i = 0; free_pages && i < info[2] && i < free_capacity; ++i) free_pages[i] = m.free_pages[i];
}

void DecoderExecutablePlan::kv_truncate(int new_length) {
    auto& m = *impl_;
    if (!m.paged) throw std::invalid_argument("plan has no paged KV cache");
    if (new_length < 0 || new_length > m.kv_length) throw std::invalid_argument("invalid paged KV truncation length");
    const int keep = new_length == 0 ? 0 : ceil_div(new_length, m.page_tokens);
    while (static_cast<int>(m.page_table.size()) > keep) {
        m.free_pages.push_back(m.page_table.back());
        m.page_table.pop_back();
    }
    m.kv_length = new_length;
    m.sync_table(config.batch, stream_);
}

void DecoderExecutablePlan::kv_release(const int* pages, int count) {
    auto& m = *impl_;
    if (!m.paged || (!pages && count > 0)) throw std::invalid_argument("plan has no paged KV cache");
    for (int i = 0; i < count; ++i) {
        const int page = pages[i];
        if (page < 0 || page >= m.max_blocks) throw std::invalid_argument("invalid physical KV page");
        if (std::find(m.page_table.begin(), m.page_table.end(), page) != m.page_table.end())
            throw std::invalid_argument("cannot release an active paged KV page");
        if (std::find(m.free_pages.begin(), m.free_pages.end(), page) == m.free_pages.end()) m.free_pages.push_back(page);
    }
    m.sync_table(config.batch, stream_);
}

// One pass of a sharded plan where every rank brings and takes only ITS rows over its own PCIe link:
// the rows are uploaded into a zeroed input tensor, the sum all-reduce of the hook then acts as the
// all-gather (every row is non-zero on exactly one rank, so the sum is exact), the layer runs on the
// replicated input and the rank downloads its rows of the replicated output.
void DecoderExecutablePlan::execute_rows(const float* input_rows, float* output_rows, int row_begin, int row_count,
                                         sfb_decoder_result* result) {
    auto& m = *impl_;
    if (!input_rows || !output_rows) throw std::invalid_argument("decoder input is null");
    if (row_begin < 0 || row_count <= 0 || row_begin + row_count > m.T)
        throw std::invalid_argument("decoder row range lies outside the plan");
    const bool whole = row_begin == 0 && row_count == m.T;
    // a two-shot plan gathers the rows with peer stores when every rank brings exactly the rows it owns
    const bool peer_gather = !whole && m.two_shot() && row_count == m.T / m.size && row_begin == m.rank * row_count;
    if (!whole && !peer_gather && (m.dtype != SFB_BF16 || !allreduce_))
        throw std::invalid_argument("a row range needs a bf16 plan with an all-reduce hook");
    cudaStream_t s = stream_;
    const uint64_t launches_before = sfb_launch_count();
    const std::size_t first = static_cast<std::size_t>(row_begin) * m.H, count = static_cast<std::size_t>(row_count) * m.H;
    cudaEvent_t h0 = m.events[12], h1 = m.events[13], d0 = m.events[14], d1 = m.events[15];
    cuda_check(cudaEventRecord(h0, s), "event");
    cuda_check(cudaMemcpyAsync(m.ws<float>("input_f32") + first, input_rows, count * 4, cudaMemcpyHostToDevice, s), "input upload");
    m.input_in_peer = false;
    if (peer_gather) {
        // own rows -> bf16 (+ sums of squares) straight into this rank's gathered input, then out to every peer
        char* mine = m.gathered<char>(0) + first * 2;
        float* mine_ss = m.gathered_ss(0) + row_begin;
        if (m.fold1)
            throw_on(sfb_k_convert_rows_sumsq(m.ws<float>("input_f32") + first, mine, mine_ss, row_count, m.H, s));
        else
            throw_on(sfb_k_convert(m.ws<float>("input_f32") + first, SFB_F32, mine, SFB_BF16, static_cast<int64_t>(count), s));
        throw_on(m.reduce_gather(0, mine, m.fold1 ? mine_ss : nullptr, nullptr, m.fold1, s));
        m.input_in_peer = true;
    } else if (m.dtype == SFB_BF16) {
        char* input = static_cast<char*>(m.ws("input"));
        if (!whole) cuda_check(cudaMemsetAsync(input, 0, static_cast<std::size_t>(m.T) * m.H * 2, s), "input clear");
        throw_on(sfb_k_convert(m.ws<float>("input_f32") + first, SFB_F32, input + first * 2, SFB_BF16, static_cast<int64_t>(count), s));
        if (!whole) allreduce_(allreduce_user_, input, static_cast<int64_t>(m.T) * m.H, SFB_BF16, s);
        if (m.fold1) throw_on(sfb_k_row_sumsq(input, m.ws<float>("ss1"), m.T, m.H, s));
    }
    m.has_input = true;
    cuda_check(cudaEventRecord(h1, s), "event");
    run(s, RoutingTraceView{}, true);
    cuda_check(cudaEventRecord(d0, s), "event");
    const float* src = m.dtype == SFB_BF16 ? m.ws<float>("output_f32") : m.ws<float>("output");
    m.materialize_output(row_begin, row_count, s);
    m.queue_status_read(s);
    cuda_check(cudaMemcpyAsync(output_rows, src + first, count * 4, cudaMemcpyDeviceToHost, s), "output download");
    cuda_check(cudaEventRecord(d1, s), "event");
    cuda_check(cudaEventSynchronize(d1), "event sync");
    m.check_status(s);
    if (!result) return;
    auto span = [&](cudaEvent_t a, cudaEvent_t b) {
        float ms = 0.0F;
        cuda_check(cudaEventElapsedTime(&ms, a, b), "event time");
        return static_cast<double>(ms);
    };
    auto* e = m.events;
    *result = {};
    result->h2d_milliseconds = span(h0, h1);
    result->d2h_milliseconds = span(d0, d1);
    result->norm_rope_milliseconds = span(e[0], e[1]) + span(e[2], e[3]) + span(e[6], e[7]);
    result->projection_milliseconds = span(e[1], e[2]) + span(e[4], e[5]);
    result->attention_milliseconds = span(e[3], e[4]);
    result->residual_milliseconds = span(e[5], e[6]) + span(e[8], e[9]);
    result->ffn_milliseconds = span(e[7], e[8]);
    result->milliseconds = span(h0, d1);
    result->tokens_per_second = result->milliseconds > 0.0 ? m.T * 1000.0 / result->milliseconds : 0.0;
    result->kernel_launches = sfb_launch_count() - launches_before;
}

// Dense bf16 prefill with fused epilogues, one chunk of rows at a time: the host->device copy of
// chunk c+1 and the device->host copy of chunk c-1 run on their own streams while chunk c computes.
// Every stage but attention is row-wise, and causal attention of a row needs only the rows of its
// sequence before it, which earlier chunks hold: the result equals the unchunked pass.
void DecoderExecutablePlan::execute_pipelined(const float* input, float* output, sfb_decoder_result* result) {
    auto& m = *impl_;
    if (!input || !output) throw std::invalid_argument("decoder input or output is null");
    const DecoderConfig& c = config;
    cudaStream_t s = stream_;
    m.input_in_peer = false;
    const int chunks = m.pipeline_chunks, S = c.sequence;
    int rows = 0;  // rows of the chunk at hand
    const int H = m.H, I = m.I_l, D = m.D;
    const std::size_t row_f32 = static_cast<std::size_t>(H) * 4, row_bf = static_cast<std::size_t>(H) * 2;
    auto at = [](void* base, std::size_t bytes) { return static_cast<void*>(static_cast<char*>(base) + bytes); };
    const bool peer = m.size > 1 && m.peer_local != nullptr;
    // which folded-norm role a GEMM of the chunk plays: 1 = QKV (scaled by ss1), 2 = O (leaves ss2), 3 = gate/up (scaled by ss2)
    auto gemm = [&](const void* a, const void* w, void* out, int n, int k, int epi, const void* res, int sb, int g0,
                    bool f32_out = false, int peer_set = -1, int fold_role = 0) {
        sfb_gemm_args g{};
        g.a = a; g.bt = w; g.out = out; g.m = rows; g.n = n; g.k = k; g.epilogue = epi;
        g.backend = policy.gemm_backend; g.residual = res; g.swiglu_block = sb; g.out_f32 = f32_out ? 1 : 0;
        if (epi == SFB_EPI_ROPE_SPLIT) {
            g.q = m.ws("query"); g.key = m.ws("key"); g.value = m.ws("value");  // the full tensors: row g0 + r is token (b, t)
            g.rope_cos = m.rope_cos; g.rope_sin = m.rope_sin;
            g.batch = c.batch; g.seq = S; g.q_heads = m.hq; g.kv_heads = m.hkv; g.head_dim = D;
            g.rope_row_offset = g0;
        }
        if (fold_role == 1 && m.fold1) {
            g.row_ss = m.ws<float>("ss1") + g0; g.rms_epsilon = c.rms_epsilon;
        } else if (fold_role == 2 && m.fold2 && m.size == 1) {
            g.ss_out = m.ws<unsigned long long>("ss2") + g0;
        } else if (fold_role == 3 && m.fold2) {  // 64-bit fixed-point sums from the O epilogue, or floats summed after the all-reduce
            g.row_ss = m.size == 1 ? static_cast<const void*>(m.ws<unsigned long long>("ss2") + g0)
                                   : static_cast<const void*>(m.ws<float>("ss2") + g0);
            g.row_ss_fixed = m.size == 1 ? 1 : 0; g.rms_epsilon = c.rms_epsilon;
        }
        if (fold_role == 1 && m.fold2 && m.size == 1) {  // this chunk's sums start at zero
            g.clear = m.ws<unsigned long long>("ss2") + g0; g.clear_bytes = static_cast<std::size_t>(rows) * 8;
        }
        g.bt_tiled = m.blocked(w) ? 1 : 0;
        if (const auto* quantized = m.int8(w)) {
            g.bt = quantized->q;
            g.bt_scales = quantized->scales;
        }
        if (peer_set >= 0) m.fill_peer_out(g, peer_set, static_cast<std::size_t>(g0) * H);
        throw_on(sfb_k_gemm_bf16(&g, s));
    };
    // sum over the ranks of `rows` x H partial sums: fused peer form, or the caller's hook
    auto reduce = [&](int peer_set, void* buffer, int g0) {
        if (peer) throw_on(m.peer_finish(peer_set, buffer, static_cast<std::size_t>(g0) * H,
                                         static_cast<int64_t>(rows) * H, s));
        else if (m.size > 1 && allreduce_) allreduce_(allreduce_user_, buffer, static_cast<int64_t>(rows) * H, m.dtype, s);
    };
    cudaEvent_t t0 = m.events[12], t1 = m.events[15];
    // Stage marks between the kernels of a chunk cost about 10 us each and keep a kernel from starting under the
    // tail of the one before: they are recorded only for a caller that asks for the stage times.
    const bool stage_marks = result != nullptr;
    cuda_check(cudaEventRecord(t0, s), "event");
    cuda_check(cudaStreamWaitEvent(m.copy_in, t0, 0), "stream wait");
    *m.upload_epoch_host = ++m.upload_epoch;  // (the call before has ended: it waits for its last event)
    const bool add_residual_here = m.rank == 0;
    for (int ch = 0; ch < chunks; ++ch) {
        cudaEvent_t* ev = &m.chunk_events[static_cast<std::size_t>(ch) * 7];
        const int g0 = m.pipeline_ranges[ch].first;      // first row of the chunk in the [T, H] input
        rows = m.pipeline_ranges[ch].second;
        const std::size_t r0 = static_cast<std::size_t>(g0);
        cuda_check(cudaMemcpyAsync(at(m.ws("input_f32"), r0 * row_f32), input + r0 * H, rows * row_f32,
                                   cudaMemcpyHostToDevice, m.copy_in), "input upload");
        cuda_check(cudaMemcpyAsync(m.chunk_flags + ch, m.upload_epoch_host, sizeof(uint32_t), cudaMemcpyHostToDevice, m.copy_in),
                   "chunk flag");
        if (ch == 0) cuda_check(cudaEventRecord(ev[0], m.copy_in), "event");  // end of the exposed upload, for the result
        throw_on(sfb_k_flag_wait(m.chunk_flags + ch, m.upload_epoch, s));
        void* x = at(m.ws("input"), r0 * row_bf);
        void* n1 = m.fold1 ? x : at(m.ws("normalized1"), r0 * row_bf);
        void* attn = at(m.ws("attention"), r0 * static_cast<std::size_t>(m.hidden_l) * 2);
        void* r1 = at(m.ws("attention_residual"), r0 * row_bf);
        void* n2 = m.fold2 ? r1 : at(m.ws("normalized2"), r0 * row_bf);
        void* act = at(m.ws("activation"), r0 * static_cast<std::size_t>(I) * 2);
        void* out = at(m.ws("output"), r0 * row_bf);
        void* out32 = at(m.ws("output_f32"), r0 * row_f32);
        if (stage_marks) cuda_check(cudaEventRecord(ev[2], s), "event");
        if (m.fold1) {
            throw_on(sfb_k_convert_rows_sumsq(static_cast<const float*>(at(m.ws("input_f32"), r0 * row_f32)), x,
                                              m.ws<float>("ss1") + g0, rows, H, s));
        } else {
            throw_on(sfb_k_convert(at(m.ws("input_f32"), r0 * row_f32), SFB_F32, x, SFB_BF16, static_cast<int64_t>(rows) * H, s));
            throw_on(sfb_k_rms_norm(x, m.rms1, n1, rows, H, c.rms_epsilon, SFB_BF16, s));
        }
        gemm(n1, m.wqkv, nullptr, m.qkv_l, H, SFB_EPI_ROPE_SPLIT, nullptr, 0, g0, false, -1, 1);
        if (stage_marks) cuda_check(cudaEventRecord(ev[3], s), "event");
        // one attention launch per run of whole sequences and per part of a sequence that the chunk holds
        for (int r = g0; r < g0 + rows;) {
            const int b0 = r / S, begin = r % S;                       // sequence and position of row r
            const int left = g0 + rows - r;
            const bool part = begin != 0 || left < S;                  // rows [begin, end) of sequence b0
            const int end = part ? std::min(S, begin + left) : S;
            const int nb = part ? 1 : left / S;
            sfb_attention_args a{};
            a.q = at(m.ws("query"), (static_cast<std::size_t>(b0) * m.hq * S + begin) * D * 2);
            a.key = at(m.ws("key"), static_cast<std::size_t>(b0) * m.hkv * S * D * 2);
            a.value = at(m.ws("value"), static_cast<std::size_t>(b0) * m.hkv * S * D * 2);
            a.out = at(m.ws("attention"), static_cast<std::size_t>(r) * m.hidden_l * 2);
            a.batch = nb; a.q_heads = m.hq; a.kv_heads = m.hkv;
            a.seq_q = end - begin;
            a.seq_kv = end;  // rows [begin, end) of a sequence attend to its keys [0, end)
            if (part) { a.q_head_rows = S; a.kv_head_rows = S; }
            a.head_dim = D; a.head_dim_value = D; a.causal = c.causal; a.scale = 0.0F; a.token_major = 1;
            a.dtype = SFB_BF16; a.backend = policy.attention_backend;
            throw_on(sfb_k_attention_prefill(&a, s));
            r += part ? end - begin : nb * S;
        }
        if (stage_marks) cuda_check(cudaEventRecord(ev[4], s), "event");
        gemm(attn, m.wo, r1, H, m.hidden_l, add_residual_here ? SFB_EPI_RESIDUAL : SFB_EPI_STORE, x, 0, g0, false, peer ? 0 : -1, 2);
        reduce(0, r1, g0);
        if (!m.fold2) throw_on(sfb_k_rms_norm(r1, m.rms2, n2, rows, H, c.rms_epsilon, SFB_BF16, s));
        else if (m.size > 1) throw_on(sfb_k_row_sumsq(r1, m.ws<float>("ss2") + g0, rows, H, s));
        if (stage_marks) cuda_check(cudaEventRecord(ev[5], s), "event");
        gemm(n2, m.wgu, act, 2 * I, H, SFB_EPI_SWIGLU, nullptr, m.swiglu_block, g0, false, -1, 3);
        if (m.direct_f32_output) {
            gemm(act, m.wd, out32, H, I, SFB_EPI_RESIDUAL, r1, 0, g0, true);
            if (stage_marks) cuda_check(cudaEventRecord(ev[6], s), "event");
        } else {
            gemm(act, m.wd, out, H, I, add_residual_here ? SFB_EPI_RESIDUAL : SFB_EPI_STORE, r1, 0, g0, false, peer ? 1 : -1);
            reduce(1, out, g0);
            if (stage_marks) cuda_check(cudaEventRecord(ev[6], s), "event");
            throw_on(sfb_k_convert(out, SFB_BF16, out32, SFB_F32, static_cast<int64_t>(rows) * H, s));
        }
        cuda_check(cudaEventRecord(ev[1], s), "event");
        cuda_check(cudaStreamWaitEvent(m.copy_out, ev[1], 0), "stream wait");
        cuda_check(cudaMemcpyAsync(output + r0 * H, out32, rows * row_f32, cudaMemcpyDeviceToHost, m.copy_out), "output download");
    }
    cuda_check(cudaEventRecord(m.events[14], m.copy_out), "event");
    cuda_check(cudaStreamWaitEvent(s, m.events[14], 0), "stream wait");
    m.queue_status_read(s);
    cuda_check(cudaEventRecord(t1, s), "event");
    cuda_check(cudaEventSynchronize(t1), "event sync");
    m.has_input = true;  // the whole input is resident (as bf16) for later resident runs
    m.check_status(s);
    if (!result) return;
    auto span = [&](cudaEvent_t a, cudaEvent_t b) {
        float ms = 0.0F;
        cuda_check(cudaEventElapsedTime(&ms, a, b), "event time");
        return static_cast<double>(ms);
    };
    *result = {};
    for (int ch = 0; ch < chunks; ++ch) {
        cudaEvent_t* ev = &m.chunk_events[static_cast<std::size_t>(ch) * 7];
        result->projection_milliseconds += span(ev[2], ev[3]) + span(ev[4], ev[5]);  // incl. the fused norms
        result->attention_milliseconds += span(ev[3], ev[4]);
        result->ffn_milliseconds += span(ev[5], ev[6]);
    }
    result->h2d_milliseconds = span(t0, m.chunk_events[0]);                       // exposed part: first chunk
    result->d2h_milliseconds = span(m.chunk_events[static_cast<std::size_t>(chunks - 1) * 7 + 1], t1);  // last chunk
    result->milliseconds = span(t0, t1);
    result->tokens_per_second = result->milliseconds > 0.0 ? m.T * 1000.0 / result->milliseconds : 0.0;
}

int64_t DecoderExecutablePlan::read_tensor(const std::string& name, float* host_out, int64_t capacity) {
    auto& m = *impl_;
    if (name == "output" && m.direct_f32_output) return read_tensor("output_f32", host_out, capacity);
    if (name == "output_f32") m.materialize_output(0, m.T, stream_);
    if (name == "ep_recv_tokens" || name == "ep_recv_slots") {  // expert-parallel receive side (peer-visible buffer), int32
        if (!m.two_shot() || m.E == 0) throw std::invalid_argument("unknown decoder tensor: " + name);
        const int64_t n = static_cast<int64_t>(m.ep_capacity());
        if (!host_out) return n;
        if (capacity < n) throw std::invalid_argument("read_tensor: buffer too small");
        cuda_check(cudaStreamSynchronize(stream_), "sync");
        const char* src = m.peer_local + (name == "ep_recv_tokens" ? m.ep_recv_tokens_offset() : m.ep_recv_slots_offset());
        cuda_check(cudaMemcpy(host_out, src, static_cast<std::size_t>(n) * 4, cudaMemcpyDeviceToHost), "read tensor");
        return n;
    }
    if (m.two_shot() && host_out && (name == "output" || name == "attention_residual")) {
        // a two-shot plan keeps these two in its peer-visible buffer (every rank's owners fill them on every rank)
        const int64_t n = static_cast<int64_t>(m.T) * m.H;
        if (capacity < n) throw std::invalid_argument("read_tensor: buffer too small");
        DeviceBuffer tmp(static_cast<std::size_t>(n) * 4);
        const void* src = name == "output" ? (m.output_bf16 ? m.output_bf16 : m.ws("output")) : m.gathered(1);
        throw_on(sfb_k_convert(src, SFB_BF16, tmp.get(), SFB_F32, n, stream_));
        cuda_check(cudaStreamSynchronize(stream_), "sync");
        cuda_check(cudaMemcpy(host_out, tmp.get(), static_cast<std::size_t>(n) * 4, cudaMemcpyDeviceToHost), "read tensor");
        return n;
    }
    const int id = m.planner.find(name);
    if (id < 0) throw std::invalid_argument("unknown decoder tensor: " + name);
    cuda_check(cudaStreamSynchronize(stream_), "sync");
    const bool is_int = name == "expert_ids" || name == "counts" || name == "offsets" || name == "token_ids" ||
                        name == "route_slots" || name == "dest_of" || name == "ep_send_base" || name == "ep_recv_offsets" ||
                        name == "ep_return_table";
    const bool is_f32 = is_int || name == "expert_weights" || name == "routing_weights" || name == "input_f32" ||
                        name == "output_f32" || name == "decode_partials" || name == "ss1" || name == "ss2" || m.dtype == SFB_F32;
    std::size_t bytes = m.planner.bytes(id);
    int64_t count;
    const int A = m.T * std::max(1, m.K);
    if (name == "counts") count = m.E;
    else if (name == "offsets") count = m.E + 1;
    else if (name == "ep_send_base") count = m.E;
    else if (name == "ep_recv_offsets") count = m.E_l + 1;
    else if (name == "ep_return_table") count = static_cast<int64_t>(m.E_l) * m.size * 4;
    else if (is_int || name == "expert_weights" || name == "routing_weights") count = A;
    else if (name == "query" || name == "attention") count = static_cast<int64_t>(m.T) * m.hidden_l;
    else if (name == "key" || name == "value") count = static_cast<int64_t>(m.T) * m.kvw_l;
    else if (name == "activation") count = static_cast<int64_t>(m.T) * m.I_l;
    else if (name == "gate_up") count = static_cast<int64_t>(m.T) * 2 * m.I_l;
    else if (name == "fused_qkv") count = static_cast<int64_t>(m.T) * m.qkv_l;
    else if (name == "dispatched" || name == "expert_output") count = static_cast<int64_t>(A) * m.H;
    else if (name == "expert_activation" || name == "expert_first" || name == "expert_gate") count = static_cast<int64_t>(A) * config.intermediate;
    else if (name == "decode_partials" || name == "dispatch_scratch" || name == "tile_table" || name == "gemm_partials" ||
             name == "ss1" || name == "ss2") count = static_cast<int64_t>(bytes / 4);
    else count = static_cast<int64_t>(m.T) * m.H;
    if (!host_out) return count;
    if (capacity < count) throw std::invalid_argument("read_tensor: buffer too small");
    char* src = m.workspace.as<char>() + m.planner.offset(id);
    if (is_f32) {
        cuda_check(cudaMemcpy(host_out, src, static_cast<std::size_t>(count) * 4, cudaMemcpyDeviceToHost), "read tensor");
    } else {
        DeviceBuffer tmp(static_cast<std::size_t>(count) * 4);
        throw_on(sfb_k_convert(src, SFB_BF16, tmp.get(), SFB_F32, count, stream_));
        cuda_check(cudaStreamSynchronize(stream_), "sync");
        cuda_check(cudaMemcpy(host_out, tmp.get(), static_cast<std::size_t>(count) * 4, cudaMemcpyDeviceToHost), "read tensor");
    }
    return count;
}

std::string DecoderExecutablePlan::dump() const {
    const auto& m = *impl_;
    const bool bf = m.dtype == SFB_BF16, moe = config.ffn == DecoderFFNKind::MoE;
    int device = 0;
    cudaDeviceProp prop{};
    std::string hardware = "sm_100a";
    if (cudaGetDevice(&device) == cudaSuccess && cudaGetDeviceProperties(&prop, device) == cudaSuccess)
        hardware = std::string(prop.name) + " sm_" + std::to_string(prop.major) + std::to_string(prop.minor) +
                   " sms=" + std::to_string(prop.multiProcessorCount);
    std::ostringstream out;
    out << "sfe.decoder_executable version=0.9.0 ffn=" << (moe ? "moe" : "dense") << " hardware=\"" << hardware
        << "\" {\nimported {\n" << imported_graph.dump() << "}\ncanonical {\n" << graph.dump() << "}\n"
        << fusion.dump() << '\n' << policy.dump() << " attention=" << attention_strategy
        << "\ncompile_ms=" << compile_milliseconds << " llvm_compile_ms=0 memory_planning_ms=0"
        << "\nconstants {\n";
    for (const auto& constant : constants) out << "  " << constant.dump() << '\n';
    const char* gemm_kind = bf ? "gemm.bf16.tcgen05_tma" : "gemm.f32.fma_chain";
    out << "}\ndecoder.memory naive=" << naive_bytes << " workspace=" << workspace_bytes << " weights=" << weight_bytes
        << "\ndecoder.shard rank=" << m.rank << " size=" << m.size << " dtype=" << (bf ? "bf16" : "f32") << " collective="
        << (m.size == 1 ? "none" : !m.peer_local ? "hook" : m.peer_mode == 1 ? "peer_one_shot" : m.peer_mode == 2
                ? "peer_two_shot" : "peer_two_shot_copy_engine_gather")
        << "\nkernels {\n"
        << "  qkv {\n    " << gemm_kind << " m=" << m.T << " n=" << m.qkv_l << " k=" << m.H
        << " epilogue=" << (policy.fuse_epilogues ? "rope_split" : "store") << (m.fold1 ? " prologue=rms_norm_folded" : "")
        << (m.kv_in_epilogue ? " kv_append=paged_cache" : "") << "\n  }\n"
        << "  attention {\n    strategy=" << attention_strategy << "\n"
        << "    attention.qk attention.scale attention.causal_mask reduce.max vector.exp reduce.sum\n"
        << "    attention.rescale attention.online_softmax attention.pv vector.div\n";
    if (m.paged)
        out << "    paged_kv page_tokens=" << m.page_tokens << " blocks=" << m.num_blocks << " split_kv=" << m.splits << "\n";
    out << "  }\n  output_projection {\n    " << gemm_kind << " m=" << m.T << " n=" << m.H << " k=" << m.hidden_l
        << " epilogue=" << (policy.fuse_epilogues ? "residual" : "store") << "\n  }\n";
    if (!moe) {
        out << "  gate_up {\n    " << gemm_kind << " m=" << m.T << " n=" << 2 * m.I_l << " k=" << m.H << " epilogue="
            << (policy.fuse_epilogues ? "swiglu" : "store") << (m.fold2 ? " prologue=rms_norm_folded" : "") << "\n  }\n"
            << "  down {\n    " << gemm_kind << " m=" << m.T << " n=" << m.H << " k=" << m.I_l << " epilogue="
            << (policy.fuse_epilogues ? "residual" : "store") << "\n  }\n";
    } else {
        out << "  moe {\n    moe.router_matmul tensor.softmax tensor.topk moe.histogram moe.prefix_sum moe.dispatch\n"
            << "    moe.grouped_matmul.w1 moe.grouped_matmul.w3 tensor.swiglu moe.grouped_matmul.w2 moe.weighted_combine\n"
            << "    experts=" << m.E << " local_experts=" << m.E_l << " top_k=" << m.K << " token_buckets=[4,16,64," << m.T
            << "]\n  }\n";
    }
    out << "}\nllvm_kernels=0\n}\n";
    return out.str();
}

}  // namespace sfb
