// Host-buffer entry points for the attention, paged-KV and MoE sub-APIs that the
// reference exposes next to the decoder compiler (execute_attention,
// execute_decode_attention, PagedKVCache functions, route_topk, dispatch_tokens,
// execute_moe, plan_moe_tasks).  Each call stages float32 host data on the device,
// runs the CUDA kernels through the kernel ABI and copies the result back.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <memory>
#include <numeric>
#include <vector>

#include "../common.cuh"
#include "runtime.hpp"

using namespace sfb;

namespace {

struct Timer {
    cudaEvent_t a = nullptr, b = nullptr;
    Timer() { cudaEventCreate(&a); cudaEventCreate(&b); }
    ~Timer() { if (a) cudaEventDestroy(a); if (b) cudaEventDestroy(b); }
    void start(cudaStream_t s) { cudaEventRecord(a, s); }
    double stop(cudaStream_t s) {
        cudaEventRecord(b, s);
        cudaEventSynchronize(b);
        float ms = 0.0F;
        cudaEventElapsedTime(&ms, a, b);
        return ms;
    }
};

// Device tensor of `count` elements of `dtype`, filled from host float32.
struct Staged {
    DeviceBuffer buffer, f32;
    void* get() const { return buffer.get(); }
    Staged(const float* host, size_t count, int dtype, cudaStream_t s) {
        buffer.allocate(count * dtype_size(dtype));
        if (!host) return;
        if (dtype == SFB_F32) {
            cuda_check(cudaMemcpyAsync(buffer.get(), host, count * 4, cudaMemcpyHostToDevice, s), "upload");
        } else {
            f32.allocate(count * 4);
            cuda_check(cudaMemcpyAsync(f32.get(), host, count * 4, cudaMemcpyHostToDevice, s), "upload");
            throw_on(sfb_k_convert(f32.get(), SFB_F32, buffer.get(), SFB_BF16, static_cast<int64_t>(count), s));
        }
    }
};

void fetch(const void* device, size_t count, int dtype, float* host, cudaStream_t s) {
    if (dtype == SFB_F32) {
        cuda_check(cudaMemcpyAsync(host, device, count * 4, cudaMemcpyDeviceToHost, s), "download");
        cuda_check(cudaStreamSynchronize(s), "download sync");
    } else {
        DeviceBuffer f32(count * 4);
        throw_on(sfb_k_convert(device, SFB_BF16, f32.get(), SFB_F32, static_cast<int64_t>(count), s));
        cuda_check(cudaMemcpyAsync(host, f32.get(), count * 4, cudaMemcpyDeviceToHost, s), "download");
        cuda_check(cudaStreamSynchronize(s), "download sync");
    }
}

void validate_attention(const sfb_attention_config& c) {
    if (c.batch <= 0 || c.query_heads <= 0 || c.kv_heads <= 0 || c.sequence_query <= 0 || c.sequence_kv <= 0 ||
        c.head_dim <= 0 || c.head_dim_value <= 0 || c.query_heads % c.kv_heads != 0 ||
        (c.causal && c.sequence_query > c.sequence_kv))
        throw std::invalid_argument("invalid attention configuration");
}

void validate_moe(const sfb_moe_config& c) {
    if (c.tokens <= 0 || c.hidden <= 0 || c.intermediate <= 0 || c.experts <= 0 || c.top_k <= 0 ||
        c.top_k > c.experts)
        throw std::invalid_argument("invalid MoE configuration");
}

}  // namespace

// PagedKVCache on the device.  Page p of the reference holds [batch][kv_head][page_tokens][dim];
// here that is physical block p*batch + b of a [block][kv_head][page_tokens][dim] pool, so
// sequence b's block table is page_table[i]*batch + b.
struct sfb_paged_kv {
    int batch, kv_heads, dim, dim_v, page_tokens, capacity, dtype;
    int length = 0;
    std::vector<int> page_table, free_pages;
    DeviceBuffer k_pool, v_pool, table, lens;
    int pages() const { return (capacity + page_tokens - 1) / page_tokens; }
    void sync_table(cudaStream_t s, int start_length) {
        const int max_blocks = pages();
        std::vector<int> host(static_cast<size_t>(batch) * max_blocks, 0), len(batch, start_length);
        for (int b = 0; b < batch; ++b)
            for (size_t i = 0; i < page_table.size(); ++i) host[static_cast<size_t>(b) * max_blocks + i] = page_table[i] * batch + b;
        cuda_check(cudaMemcpyAsync(table.get(), host.data(), host.size() * 4, cudaMemcpyHostToDevice, s), "table upload");
        cuda_check(cudaMemcpyAsync(lens.get(), len.data(), len.size() * 4, cudaMemcpyHostToDevice, s), "length upload");
        cuda_check(cudaStreamSynchronize(s), "table sync");
    }
};

extern "C" {

sfb_status sfb_attention_execute(const sfb_attention_config* config, const float* q, const float* key,
                                 const float* value, float* out, int dtype, int backend, double* milliseconds) {
    return guarded([&] {
        if (!config || !q || !key || !value || !out) throw std::invalid_argument("attention data shape mismatch");
        validate_attention(*config);
        const auto& c = *config;
        cudaStream_t s = nullptr;
        const size_t nq = static_cast<size_t>(c.batch) * c.query_heads * c.sequence_query * c.head_dim;
        const size_t nk = static_cast<size_t>(c.batch) * c.kv_heads * c.sequence_kv * c.head_dim;
        const size_t nv = static_cast<size_t>(c.batch) * c.kv_heads * c.sequence_kv * c.head_dim_value;
        const size_t no = static_cast<size_t>(c.batch) * c.query_heads * c.sequence_query * c.head_dim_value;
        Staged dq(q, nq, dtype, s), dk(key, nk, dtype, s), dv(value, nv, dtype, s), dout(nullptr, no, dtype, s);
        sfb_attention_args a{};
        a.q = dq.get(); a.key = dk.get(); a.value = dv.get(); a.out = dout.get();
        a.batch = c.batch; a.q_heads = c.query_heads; a.kv_heads = c.kv_heads; a.seq_q = c.sequence_query;
        a.seq_kv = c.sequence_kv; a.head_dim = c.head_dim; a.head_dim_value = c.head_dim_value;
        a.causal = c.causal; a.scale = c.scale; a.token_major = 0; a.dtype = dtype; a.backend = backend;
        Timer timer;
        timer.start(s);
        throw_on(sfb_k_attention_prefill(&a, s));
        const double ms = timer.stop(s);
        if (milliseconds) *milliseconds = ms;
        fetch(dout.get(), no, dtype, out, s);
    });
}

sfb_status sfb_attention_decode(const sfb_attention_config* config, const float* q, const float* keys,
                                const float* values, int length, float* out, int dtype, double* milliseconds) {
    return guarded([&] {
        if (!config || !q || !keys || !values || !out) throw std::invalid_argument("KV append shape mismatch");
        validate_attention(*config);
        const auto& c = *config;
        if (length <= 0 || length > c.sequence_kv) throw std::invalid_argument("KV cache length violates compiled guard");
        if (c.sequence_query != 1) throw std::invalid_argument("decode attention expects one query token per sequence");
        // The contiguous cache [B,Hkv,length,D] is a paged cache with one block per (sequence, 16 tokens).
        sfb_paged_kv* cache = nullptr;
        throw_on(sfb_paged_create(c.batch, c.kv_heads, c.head_dim, c.head_dim_value, 16, length, dtype, &cache));
        std::unique_ptr<sfb_paged_kv> owner(cache);
        throw_on(sfb_paged_append(cache, keys, values, length));
        sfb_attention_config runtime = c;
        runtime.sequence_kv = length;
        throw_on(sfb_paged_decode(cache, &runtime, q, out, milliseconds));
    });
}

sfb_status sfb_paged_create(int batch, int kv_heads, int head_dim, int head_dim_value, int page_tokens,
                            int capacity, int dtype, sfb_paged_kv** cache) {
    return guarded([&] {
        if (!cache) throw std::invalid_argument("null cache pointer");
        *cache = nullptr;
        if (batch <= 0 || kv_heads <= 0 || head_dim <= 0 || head_dim_value <= 0 || page_tokens <= 0 || capacity <= 0)
            throw std::invalid_argument("invalid paged KV configuration");
        auto owned = std::make_unique<sfb_paged_kv>();
        owned->batch = batch; owned->kv_heads = kv_heads; owned->dim = head_dim; owned->dim_v = head_dim_value;
        owned->page_tokens = page_tokens; owned->capacity = capacity; owned->dtype = dtype;
        const int pages = owned->pages();
        owned->free_pages.resize(pages);
        std::iota(owned->free_pages.begin(), owned->free_pages.end(), 0);
        const size_t rows = static_cast<size_t>(pages) * batch * kv_heads * page_tokens;
        owned->k_pool.allocate(rows * head_dim * dtype_size(dtype));
        owned->v_pool.allocate(rows * head_dim_value * dtype_size(dtype));
        owned->table.allocate(static_cast<size_t>(batch) * pages * 4);
        owned->lens.allocate(static_cast<size_t>(batch) * 4);
        cuda_check(cudaMemset(owned->k_pool.get(), 0, owned->k_pool.bytes()), "pool clear");
        cuda_check(cudaMemset(owned->v_pool.get(), 0, owned->v_pool.bytes()), "pool clear");
        *cache = owned.release();
    });
}

void sfb_paged_destroy(sfb_paged_kv* cache) { delete cache; }

sfb_status sfb_paged_set_free_pages(sfb_paged_kv* cache, const int* pages, int count) {
    return guarded([&] {
        if (!cache || (!pages && count > 0)) throw std::invalid_argument("null paged KV cache");
        cache->free_pages.assign(pages, pages + count);
    });
}

sfb_status sfb_paged_append(sfb_paged_kv* cache, const float* keys, const float* values, int tokens) {
    return guarded([&] {
        if (!cache) throw std::invalid_argument("null paged KV cache");
        auto& c = *cache;
        if (tokens <= 0 || c.length + tokens > c.capacity) throw std::invalid_argument("paged KV capacity exceeded");
        if (!keys || !values) throw std::invalid_argument("paged KV append shape mismatch");
        const int last_page = (c.length + tokens - 1) / c.page_tokens;
        while (static_cast<int>(c.page_table.size()) <= last_page) {
            if (c.free_pages.empty()) throw std::runtime_error("paged KV page allocator exhausted");
            c.page_table.push_back(c.free_pages.back());
            c.free_pages.pop_back();
        }
        cudaStream_t s = nullptr;
        c.sync_table(s, c.length);
        const size_t rows = static_cast<size_t>(c.batch) * c.kv_heads * tokens;
        Staged dk(keys, rows * c.dim, c.dtype, s), dv(values, rows * c.dim_v, c.dtype, s);
        throw_on(sfb_k_paged_kv_append(dk.get(), dv.get(), c.k_pool.get(), c.v_pool.get(), c.table.as<int>(),
                                       c.lens.as<int>(), c.batch, c.kv_heads, tokens, c.dim, c.dim_v, c.page_tokens,
                                       c.pages(), c.pages() * c.batch, static_cast<sfb_dtype>(c.dtype), s));
        cuda_check(cudaStreamSynchronize(s), "append sync");
        c.length += tokens;
    });
}

sfb_status sfb_paged_truncate(sfb_paged_kv* cache, int new_length) {
    return guarded([&] {
        if (!cache) throw std::invalid_argument("null paged KV cache");
        auto& c = *cache;
        if (new_length < 0 || new_length > c.length) throw std::invalid_argument("invalid paged KV truncation length");
        const int keep = new_length == 0 ? 0 : (new_length + c.page_tokens - 1) / c.page_tokens;
        while (static_cast<int>(c.page_table.size()) > keep) {
            c.free_pages.push_back(c.page_table.back());
            c.page_table.pop_back();
        }
        c.length = new_length;
    });
}

sfb_status sfb_paged_release(sfb_paged_kv* cache, const int* pages, int count) {
    return guarded([&] {
        if (!cache || (!pages && count > 0)) throw std::invalid_argument("null paged KV cache");
        auto& c = *cache;
        for (int i = 0; i < count; ++i) {
            const int page = pages[i];
            if (page < 0 || page >= c.pages()) throw std::invalid_argument("invalid physical KV page");
            if (std::find(c.page_table.begin(), c.page_table.end(), page) != c.page_table.end())
                throw std::invalid_argument("cannot release an active paged KV page");
            if (std::find(c.free_pages.begin(), c.free_pages.end(), page) == c.free_pages.end())
                c.free_pages.push_back(page);
        }
    });
}

sfb_status sfb_paged_info(const sfb_paged_kv* cache, int* info, int* page_table, int table_capacity,
                          int* free_pages, int free_capacity) {
    return guarded([&] {
        if (!cache || !info) throw std::invalid_argument("null paged KV cache");
        info[0] = cache->length;
        info[1] = static_cast<int>(cache->page_table.size());
        info[2] = static_cast<int>(cache->free_pages.size());
        info[3] = cache->pages();
        for (int i = 0; page_table && i < info[1] && i < table_capacity; ++i) page_table[i] = cache->page_table[i];
        for (int i = 0; free_pages && i < info[2] && i < free_capacity; ++i) free_pages[i] = cache->free_pages[i];
    });
}

sfb_status sfb_paged_gather(sfb_paged_kv* cache, float* keys, float* values) {
    return guarded([&] {
        if (!cache || !keys || !values) throw std::invalid_argument("null paged KV cache");
        auto& c = *cache;
        if (c.length <= 0) throw std::invalid_argument("cannot gather empty paged KV cache");
        cudaStream_t s = nullptr;
        c.sync_table(s, c.length);
        const size_t rows = static_cast<size_t>(c.batch) * c.kv_heads * c.length;
        DeviceBuffer dk(rows * c.dim * dtype_size(c.dtype)), dv(rows * c.dim_v * dtype_size(c.dtype));
        throw_on(sfb_k_paged_kv_gather(c.k_pool.get(), c.v_pool.get(), dk.get(), dv.get(), c.table.as<int>(), c.batch,
                                       c.kv_heads, c.length, c.dim, c.dim_v, c.page_tokens, c.pages(),
                                       static_cast<sfb_dtype>(c.dtype), s));
        fetch(dk.get(), rows * c.dim, c.dtype, keys, s);
        fetch(dv.get(), rows * c.dim_v, c.dtype, values, s);
    });
}

sfb_status sfb_paged_decode(sfb_paged_kv* cache, const sfb_attention_config* config, const float* q,
                            float* out, double* milliseconds) {
    return guarded([&] {
        if (!cache || !config || !q || !out) throw std::invalid_argument("paged attention query shape mismatch");
        auto& c = *cache;
        const auto& a = *config;
        if (c.length <= 0 || c.length > a.sequence_kv) throw std::invalid_argument("paged KV length violates compiled guard");
        if (a.causal && a.sequence_query > c.length) throw std::invalid_argument("paged causal query exceeds available KV length");
        if (c.batch != a.batch || c.kv_heads != a.kv_heads || c.dim != a.head_dim || c.dim_v != a.head_dim_value)
            throw std::invalid_argument("paged KV shape violates compiled guard");
        if (a.query_heads <= 0 || a.query_heads % a.kv_heads != 0)
            throw std::invalid_argument("invalid grouped-query attention configuration");
        if (static_cast<int>(c.page_table.size()) < (c.length + c.page_tokens - 1) / c.page_tokens)
            throw std::invalid_argument("paged KV page table is incomplete");
        cudaStream_t s = nullptr;
        c.sync_table(s, c.length);
        const size_t nq = static_cast<size_t>(a.batch) * a.query_heads * a.sequence_query * a.head_dim;
        const size_t no = static_cast<size_t>(a.batch) * a.query_heads * a.sequence_query * a.head_dim_value;
        Staged dq(q, nq, c.dtype, s), dout(nullptr, no, c.dtype, s);
        Timer timer;
        if (a.sequence_query == 1) {
            const int splits = sfb_attention_decode_default_splits(a.batch, a.kv_heads, c.length);
            DeviceBuffer partials(sfb_attention_decode_workspace(a.batch, a.query_heads, a.head_dim_value, splits));
            sfb_decode_args d{};
            d.q = dq.get(); d.k_pool = c.k_pool.get(); d.v_pool = c.v_pool.get(); d.block_table = c.table.as<int>();
            d.context_len = c.lens.as<int>(); d.out = dout.get(); d.partials = partials.get();
            d.batch = a.batch; d.q_heads = a.query_heads; d.kv_heads = a.kv_heads; d.head_dim = a.head_dim;
            d.head_dim_value = a.head_dim_value; d.block_tokens = c.page_tokens; d.max_blocks = c.pages();
            d.num_blocks = c.pages() * c.batch; d.max_context = c.length; d.splits = splits; d.scale = a.scale;
            d.dtype = c.dtype;
            timer.start(s);
            throw_on(sfb_k_attention_decode_paged(&d, s));
            const double ms = timer.stop(s);
            if (milliseconds) *milliseconds = ms;
        } else {
            // several query tokens: gather the live tokens and run the tiled prefill kernel on them
            const size_t rows = static_cast<size_t>(c.batch) * c.kv_heads * c.length;
            DeviceBuffer dk(rows * c.dim * dtype_size(c.dtype)), dv(rows * c.dim_v * dtype_size(c.dtype));
            timer.start(s);
            throw_on(sfb_k_paged_kv_gather(c.k_pool.get(), c.v_pool.get(), dk.get(), dv.get(), c.table.as<int>(),
                                           c.batch, c.kv_heads, c.length, c.dim, c.dim_v, c.page_tokens, c.pages(),
                                           static_cast<sfb_dtype>(c.dtype), s));
            sfb_attention_args p{};
            p.q = dq.get(); p.key = dk.get(); p.value = dv.get(); p.out = dout.get();
            p.batch = a.batch; p.q_heads = a.query_heads; p.kv_heads = a.kv_heads; p.seq_q = a.sequence_query;
            p.seq_kv = c.length; p.head_dim = a.head_dim; p.head_dim_value = a.head_dim_value; p.causal = a.causal;
            p.scale = a.scale; p.token_major = 0; p.dtype = c.dtype; p.backend = 1;
            throw_on(sfb_k_attention_prefill(&p, s));
            const double ms = timer.stop(s);
            if (milliseconds) *milliseconds = ms;
        }
        fetch(dout.get(), no, c.dtype, out, s);
    });
}

sfb_status sfb_moe_route_topk(const sfb_moe_config* config, const float* input, int tokens,
                              const float* router_weight, const float* router_bias, int dtype,
                              int* expert_ids, float* expert_weights, int* counts) {
    return guarded([&] {
        if (!config || !input || !router_weight || !expert_ids || !expert_weights || !counts)
            throw std::invalid_argument("MoE input does not match hidden dimension");
        validate_moe(*config);
        const auto& c = *config;
        if (tokens <= 0) throw std::invalid_argument("MoE input does not match hidden dimension");
        cudaStream_t s = nullptr;
        const size_t A = static_cast<size_t>(tokens) * c.top_k;
        Staged x(input, static_cast<size_t>(tokens) * c.hidden, dtype, s);
        Staged w(router_weight, static_cast<size_t>(c.hidden) * c.experts, SFB_F32, s);
        Staged bias(router_bias, c.experts, SFB_F32, s);
        DeviceBuffer ids(A * 4), wts(A * 4), cnt(static_cast<size_t>(c.experts) * 4);
        throw_on(sfb_k_moe_route(x.get(), static_cast<sfb_dtype>(dtype), static_cast<const float*>(w.get()),
                                 router_bias ? static_cast<const float*>(bias.get()) : nullptr, tokens, c.hidden,
                                 c.experts, c.top_k, ids.as<int>(), wts.as<float>(), cnt.as<int>(), s));
        cuda_check(cudaMemcpyAsync(expert_ids, ids.get(), A * 4, cudaMemcpyDeviceToHost, s), "download");
        cuda_check(cudaMemcpyAsync(expert_weights, wts.get(), A * 4, cudaMemcpyDeviceToHost, s), "download");
        cuda_check(cudaMemcpyAsync(counts, cnt.get(), static_cast<size_t>(c.experts) * 4, cudaMemcpyDeviceToHost, s), "download");
        cuda_check(cudaStreamSynchronize(s), "download sync");
    });
}

sfb_status sfb_moe_dispatch_tokens(const sfb_moe_config* config, const float* input, int tokens,
                                   const int* expert_ids, const float* expert_weights, const int* counts,
                                   int dtype, float* values, int* offsets, int* token_ids, int* route_slots,
                                   float* routing_weights) {
    return guarded([&] {
        if (!config || !expert_ids || !expert_weights || !counts || !offsets || !token_ids || !route_slots || !routing_weights)
            throw std::invalid_argument("routing trace does not match MoE configuration");
        validate_moe(*config);
        const auto& c = *config;
        if (tokens <= 0 || (values && !input)) throw std::invalid_argument("MoE input is smaller than routing trace");
        validate_routing_trace(tokens, c.top_k, c.experts, expert_ids, expert_weights, counts);
        cudaStream_t s = nullptr;
        const size_t A = static_cast<size_t>(tokens) * c.top_k;
        Staged x(values ? input : nullptr, values ? static_cast<size_t>(tokens) * c.hidden : 1, dtype, s);
        DeviceBuffer ids(A * 4), wts(A * 4), cnt(static_cast<size_t>(c.experts) * 4), off(static_cast<size_t>(c.experts + 1) * 4),
            tok(A * 4), slot(A * 4), rw(A * 4), dest(A * 4), scratch(sfb_moe_dispatch_scratch_bytes(tokens, c.experts, c.top_k)),
            vals(values ? A * c.hidden * dtype_size(dtype) : 0);
        cuda_check(cudaMemcpyAsync(ids.get(), expert_ids, A * 4, cudaMemcpyHostToDevice, s), "upload");
        cuda_check(cudaMemcpyAsync(wts.get(), expert_weights, A * 4, cudaMemcpyHostToDevice, s), "upload");
        cuda_check(cudaMemcpyAsync(cnt.get(), counts, static_cast<size_t>(c.experts) * 4, cudaMemcpyHostToDevice, s), "upload");
        throw_on(sfb_k_moe_dispatch(x.get(), static_cast<sfb_dtype>(dtype), ids.as<int>(), wts.as<float>(), cnt.as<int>(),
                                    tokens, c.hidden, c.experts, c.top_k, values ? vals.get() : nullptr, off.as<int>(),
                                    tok.as<int>(), slot.as<int>(), rw.as<float>(), dest.as<int>(), scratch.as<int>(), s));
        cuda_check(cudaMemcpyAsync(offsets, off.get(), static_cast<size_t>(c.experts + 1) * 4, cudaMemcpyDeviceToHost, s), "download");
        cuda_check(cudaMemcpyAsync(token_ids, tok.get(), A * 4, cudaMemcpyDeviceToHost, s), "download");
        cuda_check(cudaMemcpyAsync(route_slots, slot.get(), A * 4, cudaMemcpyDeviceToHost, s), "download");
        cuda_check(cudaMemcpyAsync(routing_weights, rw.get(), A * 4, cudaMemcpyDeviceToHost, s), "download");
        cuda_check(cudaStreamSynchronize(s), "download sync");
        if (values) fetch(vals.get(), A * c.hidden, dtype, values, s);
    });
}

namespace {
// Weight-only INT8 round trip of a packed [n, k] bf16 weight (rows = output channels), in place:
// quantize_matmul_weights per output channel, then q * scale (src/next_milestones.cpp:611-637).
void int8_round_trip(void* w, long long n, int k, cudaStream_t s) {
    constexpr long long kRowsPerPass = 1 << 16;  // bounds the int8 scratch
    for (long long first = 0; first < n; first += kRowsPerPass) {
        const int rows = static_cast<int>(std::min(kRowsPerPass, n - first));
        DeviceBuffer q(static_cast<size_t>(sfb_tiled_weight_elems(rows, k))),
            scales(static_cast<size_t>(ceil_div(rows, 128)) * 128 * sizeof(float));
        cuda_check(cudaMemsetAsync(scales.get(), 0, static_cast<size_t>(ceil_div(rows, 128)) * 128 * sizeof(float), s), "scale clear");
        char* slab = static_cast<char*>(w) + static_cast<size_t>(first) * k * 2;
        throw_on(sfb_k_quantize_weight_int8(slab, q.get(), scales.as<float>(), rows, k, s));
        throw_on(sfb_k_dequantize_weight_int8(q.get(), scales.as<float>(), slab, rows, k, s));
        cuda_check(cudaStreamSynchronize(s), "weight quantization");
    }
}

sfb_status moe_execute(const sfb_moe_config* config, const float* input, int tokens, const float* w1,
                       const float* w3, const float* w2, const int* expert_ids, const float* expert_weights,
                       const int* counts, int dtype, int gemm_backend, bool int8, float* out, double* milliseconds);
}  // namespace

sfb_status sfb_moe_execute(const sfb_moe_config* config, const float* input, int tokens, const float* w1,
                           const float* w3, const float* w2, const int* expert_ids, const float* expert_weights,
                           const int* counts, int dtype, int gemm_backend, float* out, double* milliseconds) {
    return moe_execute(config, input, tokens, w1, w3, w2, expert_ids, expert_weights, counts, dtype, gemm_backend, false,
                       out, milliseconds);
}

sfb_status sfb_moe_execute_quantized(const sfb_moe_config* config, const float* input, int tokens, const float* w1,
                                     const float* w3, const float* w2, const int* expert_ids,
                                     const float* expert_weights, const int* counts, int per_channel, int gemm_backend,
                                     float* out, double* milliseconds) {
    if (!per_channel) {
        return guarded([] { throw std::invalid_argument("quantized MoE: only per-output-channel scales are built"); });
    }
    return moe_execute(config, input, tokens, w1, w3, w2, expert_ids, expert_weights, counts, SFB_BF16, gemm_backend, true,
                       out, milliseconds);
}

// The compiled MoE block: expert weights packed once and kept on the device together with every buffer a pass needs
// (MoeExecutablePlan, include/schedforge/moe_compiler.h:205-212; the reference's plan holds kernels and reads the
// weights from MoeData at execute time, a device plan keeps them resident instead).
struct sfb_moe_plan {
    sfb_moe_config config{};
    int dtype = SFB_BF16, gemm_backend = SFB_GEMM_AUTO, block = 0;
    bool has_router = false, has_bias = false;
    DeviceBuffer w13, w2t;            // bf16: [E][2I][H] (W3 | W1 interleaved in blocks), [E][H][I]
    DeviceBuffer w1f, w3f, w2f;       // fp32: the reference's layouts
    DeviceBuffer router, bias;        // fp32 [H, E], [E]
    DeviceBuffer x, ids, wts, cnt, off, tok, slot, rw, dest, scratch, xs, act, gate, y, result, table, stage_f32;
};

namespace {

void moe_plan_build(sfb_moe_plan& p, const sfb_moe_config& c, const float* w1, const float* w3, const float* w2,
                    const float* router_weight, const float* router_bias, int dtype, int gemm_backend, bool int8) {
    validate_moe(c);
    if (!w1 || !w3 || !w2) throw std::invalid_argument("MoE plan has no expert kernels");
    if (dtype != SFB_F32 && dtype != SFB_BF16) throw std::invalid_argument("unknown MoE plan dtype");
    if (int8 && dtype != SFB_BF16) throw std::invalid_argument("quantized MoE needs a bf16 plan");
    p.config = c; p.dtype = dtype; p.gemm_backend = gemm_backend;
    cudaStream_t s = nullptr;
    const int H = c.hidden, I = c.intermediate, E = c.experts, K = c.top_k, T = c.tokens;
    const size_t A = static_cast<size_t>(T) * K, ee = static_cast<size_t>(H) * I, esz = dtype_size(dtype);
    if (dtype == SFB_BF16) {
        p.block = I % 128 == 0 && T * K > 128 ? 128 : (I % 64 == 0 ? 64 : I);
        p.w13.allocate(static_cast<size_t>(E) * 2 * ee * 2);
        p.w2t.allocate(static_cast<size_t>(E) * ee * 2);
        DeviceBuffer stage(ee * 4);
        for (int e = 0; e < E; ++e) {
            char* d13 = p.w13.as<char>() + static_cast<size_t>(e) * 2 * ee * 2;
            cuda_check(cudaMemcpyAsync(stage.get(), w3 + e * ee, ee * 4, cudaMemcpyHostToDevice, s), "upload");
            pack_weight_transposed(stage.as<float>(), I, 0, H, 0, I, d13, p.block, 2 * p.block, 0, s);
            cuda_check(cudaMemcpyAsync(stage.get(), w1 + e * ee, ee * 4, cudaMemcpyHostToDevice, s), "upload");
            pack_weight_transposed(stage.as<float>(), I, 0, H, 0, I, d13, p.block, 2 * p.block, p.block, s);
            cuda_check(cudaMemcpyAsync(stage.get(), w2 + e * ee, ee * 4, cudaMemcpyHostToDevice, s), "upload");
            pack_weight_transposed(stage.as<float>(), H, 0, I, 0, H, p.w2t.as<char>() + static_cast<size_t>(e) * ee * 2, 1 << 30, 0, 0, s);
        }
        if (int8) {  // every row of the packed slabs is one output channel of one expert matrix
            int8_round_trip(p.w13.get(), static_cast<long long>(E) * 2 * I, H, s);
            int8_round_trip(p.w2t.get(), static_cast<long long>(E) * H, I, s);
        }
        cuda_check(cudaStreamSynchronize(s), "weight pack");
        p.act.allocate(A * I * 2);
        p.table.allocate(sizeof(int) * 4 * (A / 128 + E + 2));
    } else {
        for (auto [dst, src] : {std::pair<DeviceBuffer*, const float*>{&p.w1f, w1}, {&p.w3f, w3}, {&p.w2f, w2}}) {
            dst->allocate(static_cast<size_t>(E) * ee * 4);
            cuda_check(cudaMemcpyAsync(dst->get(), src, static_cast<size_t>(E) * ee * 4, cudaMemcpyHostToDevice, s), "upload");
        }
        cuda_check(cudaStreamSynchronize(s), "weight upload");
        p.act.allocate(A * I * 4);
        p.gate.allocate(A * I * 4);
    }
    if (router_weight) {
        p.router.allocate(static_cast<size_t>(H) * E * 4);
        cuda_check(cudaMemcpy(p.router.get(), router_weight, static_cast<size_t>(H) * E * 4, cudaMemcpyHostToDevice), "upload");
        p.has_router = true;
        if (router_bias) {
            p.bias.allocate(static_cast<size_t>(E) * 4);
            cuda_check(cudaMemcpy(p.bias.get(), router_bias, static_cast<size_t>(E) * 4, cudaMemcpyHostToDevice), "upload");
            p.has_bias = true;
        }
    }
    p.stage_f32.allocate(static_cast<size_t>(T) * H * 4);
    p.x.allocate(static_cast<size_t>(T) * H * esz);
    p.ids.allocate(A * 4); p.wts.allocate(A * 4); p.cnt.allocate(static_cast<size_t>(E) * 4);
    p.off.allocate(static_cast<size_t>(E + 1) * 4); p.tok.allocate(A * 4); p.slot.allocate(A * 4); p.rw.allocate(A * 4);
    p.dest.allocate(A * 4); p.scratch.allocate(sfb_moe_dispatch_scratch_bytes(T, E, K));
    p.xs.allocate(A * H * esz); p.y.allocate(A * H * esz); p.result.allocate(static_cast<size_t>(T) * H * esz);
}

// One pass (execute_moe, src/moe_compiler.cpp:684-758): with a trace the router is skipped, without one route_topk
// runs first and its time is part of the result (:734-740).  Guard: tokens <= plan.config.tokens (:696-697).
void moe_plan_run(sfb_moe_plan& p, const float* input, int tokens, const int* expert_ids, const float* expert_weights,
                  const int* counts, float* out, double* milliseconds) {
    const auto& c = p.config;
    if (!input || !out) throw std::invalid_argument("MoE input is smaller than routing trace");
    if (tokens <= 0 || tokens > c.tokens) throw std::invalid_argument("runtime token count exceeds compiled MoE guard");
    const bool traced = expert_ids || expert_weights || counts;
    if (traced) validate_routing_trace(tokens, c.top_k, c.experts, expert_ids, expert_weights, counts);
    else if (!p.has_router) throw std::invalid_argument("MoE plan has no router weights and no routing trace was given");
    cudaStream_t s = nullptr;
    const int H = c.hidden, I = c.intermediate, E = c.experts, K = c.top_k;
    const size_t A = static_cast<size_t>(tokens) * K, ee = static_cast<size_t>(H) * I;
    const auto dt = static_cast<sfb_dtype>(p.dtype);
    if (p.dtype == SFB_F32) {
        cuda_check(cudaMemcpyAsync(p.x.get(), input, static_cast<size_t>(tokens) * H * 4, cudaMemcpyHostToDevice, s), "upload");
    } else {
        cuda_check(cudaMemcpyAsync(p.stage_f32.get(), input, static_cast<size_t>(tokens) * H * 4, cudaMemcpyHostToDevice, s), "upload");
        throw_on(sfb_k_convert(p.stage_f32.get(), SFB_F32, p.x.get(), SFB_BF16, static_cast<int64_t>(tokens) * H, s));
    }
    if (traced) {
        cuda_check(cudaMemcpyAsync(p.ids.get(), expert_ids, A * 4, cudaMemcpyHostToDevice, s), "upload");
        cuda_check(cudaMemcpyAsync(p.wts.get(), expert_weights, A * 4, cudaMemcpyHostToDevice, s), "upload");
        cuda_check(cudaMemcpyAsync(p.cnt.get(), counts, static_cast<size_t>(E) * 4, cudaMemcpyHostToDevice, s), "upload");
    }
    Timer timer;
    timer.start(s);
    if (!traced)
        throw_on(sfb_k_moe_route(p.x.get(), dt, p.router.as<float>(), p.has_bias ? p.bias.as<float>() : nullptr, tokens, H, E, K,
                                 p.ids.as<int>(), p.wts.as<float>(), p.cnt.as<int>(), s));
    throw_on(sfb_k_moe_dispatch(p.x.get(), dt, p.ids.as<int>(), p.wts.as<float>(), p.cnt.as<int>(), tokens, H, E, K, p.xs.get(),
                                p.off.as<int>(), p.tok.as<int>(), p.slot.as<int>(), p.rw.as<float>(), p.dest.as<int>(),
                                p.scratch.as<int>(), s));
    if (p.dtype == SFB_BF16) {
        sfb_gemm_args g{};
        g.a = p.xs.get(); g.bt = p.w13.get(); g.out = p.act.get(); g.m = static_cast<int>(A); g.n = 2 * I; g.k = H;
        g.epilogue = SFB_EPI_SWIGLU; g.backend = p.gemm_backend; g.swiglu_block = p.block;
        g.group_offsets = p.off.as<int>(); g.groups = E; g.tile_table = p.table.get();
        throw_on(sfb_k_gemm_bf16(&g, s));
        sfb_gemm_args g2{};
        g2.a = p.act.get(); g2.bt = p.w2t.get(); g2.out = p.y.get(); g2.m = static_cast<int>(A); g2.n = H; g2.k = I;
        g2.epilogue = SFB_EPI_STORE; g2.backend = p.gemm_backend;
        g2.group_offsets = p.off.as<int>(); g2.groups = E; g2.tile_table = p.table.get();
        throw_on(sfb_k_gemm_bf16(&g2, s));
    } else {
        std::vector<int> ho(E + 1);
        cuda_check(cudaMemcpyAsync(ho.data(), p.off.get(), sizeof(int) * (E + 1), cudaMemcpyDeviceToHost, s), "offsets");
        cuda_check(cudaStreamSynchronize(s), "offsets sync");
        float *xs = p.xs.as<float>(), *first = p.act.as<float>(), *gate = p.gate.as<float>();
        for (int e = 0; e < E; ++e) {
            const int lo = ho[e], rows = ho[e + 1] - lo;
            if (rows <= 0) continue;
            throw_on(sfb_k_gemm_f32(xs + static_cast<size_t>(lo) * H, p.w1f.as<float>() + e * ee, first + static_cast<size_t>(lo) * I, rows, I, H, s));
            throw_on(sfb_k_gemm_f32(xs + static_cast<size_t>(lo) * H, p.w3f.as<float>() + e * ee, gate + static_cast<size_t>(lo) * I, rows, I, H, s));
        }
        moe_silu_mul_f32(first, gate, static_cast<int64_t>(A) * I, s);
        for (int e = 0; e < E; ++e) {
            const int lo = ho[e], rows = ho[e + 1] - lo;
            if (rows <= 0) continue;
            throw_on(sfb_k_gemm_f32(first + static_cast<size_t>(lo) * I, p.w2f.as<float>() + e * ee,
                                    p.y.as<float>() + static_cast<size_t>(lo) * H, rows, H, I, s));
        }
    }
    throw_on(sfb_k_moe_combine(p.y.get(), p.dest.as<int>(), p.rw.as<float>(), nullptr, p.result.get(), tokens, H, K, dt, s));
    const double ms = timer.stop(s);
    if (milliseconds) *milliseconds = ms;
    fetch(p.result.get(), static_cast<size_t>(tokens) * H, p.dtype, out, s);
}

// The one-call forms: a plan for this call only (weights uploaded and packed every time: a parity harness).
sfb_status moe_execute(const sfb_moe_config* config, const float* input, int tokens, const float* w1,
                       const float* w3, const float* w2, const int* expert_ids, const float* expert_weights,
                       const int* counts, int dtype, int gemm_backend, bool int8, float* out, double* milliseconds) {
    return guarded([&] {
        if (!config || !input || !w1 || !w3 || !w2 || !expert_ids || !expert_weights || !counts || !out)
            throw std::invalid_argument("MoE plan has no expert kernels");
        validate_moe(*config);
        if (tokens <= 0 || tokens > config->tokens) throw std::invalid_argument("runtime token count exceeds compiled MoE guard");
        validate_routing_trace(tokens, config->top_k, config->experts, expert_ids, expert_weights, counts);
        sfb_moe_config sized = *config;
        sized.tokens = tokens;  // buffers for this call's rows
        sfb_moe_plan plan;
        moe_plan_build(plan, sized, w1, w3, w2, nullptr, nullptr, dtype, gemm_backend, int8);
        moe_plan_run(plan, input, tokens, expert_ids, expert_weights, counts, out, milliseconds);
    });
}
}  // namespace

sfb_status sfb_moe_compile(const sfb_moe_config* config, const float* w1, const float* w3, const float* w2,
                           const float* router_weight, const float* router_bias, int dtype, int gemm_backend,
                           int weight_int8, sfb_moe_plan** plan) {
    return guarded([&] {
        if (!config || !plan) throw std::invalid_argument("invalid MoE configuration");
        *plan = nullptr;
        auto owned = std::make_unique<sfb_moe_plan>();
        moe_plan_build(*owned, *config, w1, w3, w2, router_weight, router_bias, dtype, gemm_backend, weight_int8 != 0);
        *plan = owned.release();
    });
}

void sfb_moe_destroy(sfb_moe_plan* plan) { delete plan; }

sfb_status sfb_moe_plan_execute(sfb_moe_plan* plan, const float* input, int tokens, const int* expert_ids,
                                const float* expert_weights, const int* counts, float* out, double* milliseconds) {
    return guarded([&] {
        if (!plan) throw std::invalid_argument("MoE plan has no expert kernels");
        moe_plan_run(*plan, input, tokens, expert_ids, expert_weights, counts, out, milliseconds);
    });
}

sfb_status sfb_moe_plan_tasks(const sfb_moe_config* config, const int* counts, int split_threshold, int* tasks,
                              int capacity, int* task_count) {
    return guarded([&] {
        if (!config || !counts || !tasks || !task_count) throw std::invalid_argument("invalid MoE configuration");
        validate_moe(*config);
        const auto& c = *config;
        // Token buckets {4,16,64} plus the compiled token count; segments longer than the split
        // threshold are cut into chunks; longest tasks first (stable).
        std::vector<int> buckets = {4, 16, 64};
        if (buckets.back() < c.tokens) buckets.push_back(c.tokens);
        const int threshold = split_threshold > 0 ? split_threshold : 32;
        struct Task { int expert, begin, end, bucket; };
        std::vector<Task> planned;
        int begin = 0;
        for (int e = 0; e < c.experts; ++e) {
            const int end = begin + counts[e];
            const int chunk = counts[e] > threshold ? threshold : counts[e];
            for (int b = begin; b < end; b += chunk) {
                const int stop = std::min(b + chunk, end), rows = stop - b;
                int bucket = std::max(rows, buckets.back());
                for (const int candidate : buckets)
                    if (rows <= candidate) { bucket = candidate; break; }
                planned.push_back({e, b, stop, bucket});
            }
            begin = end;
        }
        std::stable_sort(planned.begin(), planned.end(),
                         [](const Task& l, const Task& r) { return l.end - l.begin > r.end - r.begin; });
        *task_count = static_cast<int>(planned.size());
        for (int i = 0; i < *task_count && i < capacity; ++i) {
            tasks[4 * i] = planned[i].expert; tasks[4 * i + 1] = planned[i].begin;
            tasks[4 * i + 2] = planned[i].end; tasks[4 * i + 3] = planned[i].bucket;
        }
    });
}

}  // extern "C"
