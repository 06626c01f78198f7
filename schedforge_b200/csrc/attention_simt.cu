// CUDA-core attention kernels (any head size, fp32 or bf16 storage, fp32 math):
//   * prefill: exact causal/non-causal GQA attention with an online softmax over KV tiles
//     (never materialises the score matrix, skips KV tiles above the causal frontier);
//   * paged decode: split-KV partials over a block table + log-sum-exp combine;
//   * paged KV append / gather.
// The bf16 prefill hot path is the tensor-core kernel in attention_tcgen05.cu and the
// head_dim-128 bf16 decode hot path is decode_paged_d128 below; the generic kernels here
// cover fp32 plans, odd head sizes and serve as their cross-check.
#include "attention_decode.cuh"
#include "common.cuh"
#include "ptx_sm100.cuh"

#include <cfloat>

namespace sfb {

sfb_status attention_prefill_tcgen05(const sfb_attention_args& args, cudaStream_t stream);  // attention_tcgen05.cu
bool attention_prefill_tcgen05_supported(const sfb_attention_args& args);

namespace {

constexpr int kRowsPerWarp = 4;
constexpr int kWarps = 4;
constexpr int kTileKeys = 32;
constexpr int kMaxChunks = 8;  // head_dim_value <= 256

struct PrefillParams {
    const void *q, *key, *value;
    void* out;
    int batch, q_heads, kv_heads, seq_q, seq_kv, dim, dim_v;
    int causal, token_major;
    float scale;
};

// Block = 4 warps x 4 query rows of one (batch, head).  Per KV tile of 32 keys: lane j
// scores key j for each of the warp's rows, the warp reduces max/sum, then every lane
// accumulates its slice of the output dimensions (d = lane, lane+32, ...).
template <class T>
__global__ void __launch_bounds__(kWarps * 32)
attention_prefill_kernel(PrefillParams p) {
    extern __shared__ float smem[];
    const int D = p.dim, Dv = p.dim_v;
    float* ks = smem;                                   // [32][D+1]
    float* vs = ks + kTileKeys * (D + 1);               // [32][Dv]
    float* qs = vs + kTileKeys * Dv;                    // [16][D]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows_per_block = kWarps * kRowsPerWarp;
    const int q_blocks = (p.seq_q + rows_per_block - 1) / rows_per_block;
    const int qb = blockIdx.x % q_blocks;
    const int head = (blockIdx.x / q_blocks) % p.q_heads;
    const int b = blockIdx.x / q_blocks / p.q_heads;
    const int kvh = head * p.kv_heads / p.q_heads;
    const int q0 = qb * rows_per_block;
    const T* qbase = static_cast<const T*>(p.q) + (static_cast<size_t>(b) * p.q_heads + head) * p.seq_q * D;
    const T* kbase = static_cast<const T*>(p.key) + (static_cast<size_t>(b) * p.kv_heads + kvh) * p.seq_kv * D;
    const T* vbase = static_cast<const T*>(p.value) + (static_cast<size_t>(b) * p.kv_heads + kvh) * p.seq_kv * Dv;

    for (int i = threadIdx.x; i < rows_per_block * D; i += blockDim.x) {
        const int r = i / D, d = i % D;
        qs[i] = (q0 + r < p.seq_q) ? to_float(qbase[static_cast<size_t>(q0 + r) * D + d]) : 0.0F;
    }
    float mx[kRowsPerWarp], den[kRowsPerWarp], acc[kRowsPerWarp][kMaxChunks];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        mx[r] = -INFINITY;
        den[r] = 0.0F;
#pragma unroll
        for (int c = 0; c < kMaxChunks; ++c) acc[r][c] = 0.0F;
    }
    const int offset = p.seq_kv - p.seq_q;  // key j visible to query i iff j <= offset + i
    const int last_row = min(q0 + rows_per_block, p.seq_q) - 1;
    const int key_limit = p.causal ? min(p.seq_kv, offset + last_row + 1) : p.seq_kv;

    for (int k0 = 0; k0 < key_limit; k0 += kTileKeys) {
        __syncthreads();
        for (int i = threadIdx.x; i < kTileKeys * D; i += blockDim.x) {
            const int j = i / D, d = i % D;
            ks[j * (D + 1) + d] = (k0 + j < p.seq_kv) ? to_float(kbase[static_cast<size_t>(k0 + j) * D + d]) : 0.0F;
        }
        for (int i = threadIdx.x; i < kTileKeys * Dv; i += blockDim.x) {
            const int j = i / Dv, d = i % Dv;
            vs[i] = (k0 + j < p.seq_kv) ? to_float(vbase[static_cast<size_t>(k0 + j) * Dv + d]) : 0.0F;
        }
        __syncthreads();
        const int key = k0 + lane;
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const int qi = q0 + warp * kRowsPerWarp + r;
            if (qi >= p.seq_q) continue;  // warp-uniform
            const bool visible = key < p.seq_kv && (!p.causal || key <= offset + qi);
            float score = -INFINITY;
            if (visible) {
                const float* qrow = qs + (warp * kRowsPerWarp + r) * D;
                const float* krow = ks + lane * (D + 1);
                float dot = 0.0F;
                for (int d = 0; d < D; ++d) dot = fmaf(qrow[d], krow[d], dot);
                score = dot * p.scale;
            }
            const float tile_max = warp_max(score);
            if (tile_max == -INFINITY) continue;  // every key of this tile is masked for this row
            const float new_max = fmaxf(mx[r], tile_max);
            const float alpha = mx[r] == -INFINITY ? 0.0F : expf(mx[r] - new_max);
            const float prob = visible ? expf(score - new_max) : 0.0F;
            den[r] = den[r] * alpha + warp_sum(prob);
            mx[r] = new_max;
#pragma unroll
            for (int c = 0; c < kMaxChunks; ++c) acc[r][c] *= alpha;
            for (int j = 0; j < kTileKeys; ++j) {
                const float pj = __shfl_sync(0xffffffffu, prob, j);
                if (pj == 0.0F) continue;  // warp-uniform
#pragma unroll
                for (int c = 0; c < kMaxChunks; ++c) {
                    const int d = lane + 32 * c;
                    if (d < Dv) acc[r][c] = fmaf(pj, vs[j * Dv + d], acc[r][c]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        const int qi = q0 + warp * kRowsPerWarp + r;
        if (qi >= p.seq_q) continue;
        T* orow;
        if (p.token_major)
            orow = static_cast<T*>(p.out) + (static_cast<size_t>(b) * p.seq_q + qi) * (p.q_heads * Dv) + head * Dv;
        else
            orow = static_cast<T*>(p.out) + ((static_cast<size_t>(b) * p.q_heads + head) * p.seq_q + qi) * Dv;
#pragma unroll
        for (int c = 0; c < kMaxChunks; ++c) {
            const int d = lane + 32 * c;
            if (d < Dv) orow[d] = from_float<T>(acc[r][c] / den[r]);
        }
    }
}

// ---- paged decode (parameters and split rule: attention_decode.cuh) ----------------------
// Generic: one block of 128 threads per (batch, q_head, split).  Chunks of 128 keys:
// thread j scores key j (reads the key row through the block table), block max/sum,
// then thread d accumulates output dimension d over the chunk.
template <class T>
__global__ void __launch_bounds__(128)
decode_paged_generic_kernel(DecodeParams p) {
    extern __shared__ float smem[];
    float* qs = smem;               // [D]
    float* probs = qs + p.dim;      // [128]
    __shared__ float red[4];
    __shared__ int phys[128];
    const int split = blockIdx.y;
    const int head = blockIdx.x % p.q_heads, b = blockIdx.x / p.q_heads;
    const int kvh = head * p.kv_heads / p.q_heads;
    const int D = p.dim, Dv = p.dim_v, P = p.block_tokens;
    const int ctx = guarded_context(p, b);
    int begin, end;
    split_range(ctx, p.chunk_tokens, split, begin, end);
    const T* qrow = static_cast<const T*>(p.q) + (static_cast<size_t>(b) * p.q_heads + head) * D;
    for (int d = threadIdx.x; d < D; d += 128) qs[d] = to_float(qrow[d]);
    const int* table = p.block_table + static_cast<size_t>(b) * p.max_blocks;
    const T* kpool = static_cast<const T*>(p.k_pool);
    const T* vpool = static_cast<const T*>(p.v_pool);
    float run_max = -INFINITY, run_sum = 0.0F;
    float acc[2] = {0.0F, 0.0F};  // output dims threadIdx.x and threadIdx.x + 128
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int k0 = begin; k0 < end; k0 += 128) {
        __syncthreads();
        const int key = k0 + threadIdx.x;
        float score = -INFINITY;
        if (key < end) {
            int page = table[key / P];
            if (p.num_blocks > 0 && (page < 0 || page >= p.num_blocks)) {  // outside the pool: read block 0 instead, flag it
                page = 0;
                atomicOr(p.status, kCodeDecodeBounds);
            }
            phys[threadIdx.x] = page;
            const T* krow = kpool + ((static_cast<size_t>(page) * p.kv_heads + kvh) * P + key % P) * D;
            float dot = 0.0F;
            for (int d = 0; d < D; ++d) dot = fmaf(qs[d], to_float(krow[d]), dot);
            score = dot * p.scale;
        }
        float m = warp_max(score);
        if (lane == 0) red[warp] = m;
        __syncthreads();
        m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
        const float new_max = fmaxf(run_max, m);
        const float alpha = run_max == -INFINITY ? 0.0F : expf(run_max - new_max);
        const float prob = key < end ? expf(score - new_max) : 0.0F;
        probs[threadIdx.x] = prob;
        float s = warp_sum(prob);
        __syncthreads();
        if (lane == 0) red[warp] = s;
        __syncthreads();
        s = red[0] + red[1] + red[2] + red[3];
        run_sum = run_sum * alpha + s;
        run_max = new_max;
        const int live = min(128, end - k0);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int d = threadIdx.x + 128 * c;
            if (d >= Dv) continue;
            float a = acc[c] * alpha;
            for (int j = 0; j < live; ++j) {
                const int kj = k0 + j;
                const T* vrow = vpool + ((static_cast<size_t>(phys[j]) * p.kv_heads + kvh) * P + kj % P) * Dv;
                a = fmaf(probs[j], to_float(vrow[d]), a);
            }
            acc[c] = a;
        }
    }
    float* rec = p.partials + (static_cast<size_t>(blockIdx.x) * p.splits + split) * (Dv + 2);
    if (threadIdx.x == 0) { rec[0] = run_max; rec[1] = run_sum; }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int d = threadIdx.x + 128 * c;
        if (d < Dv) rec[2 + d] = acc[c];
    }
}

// One warp per (batch, q_head): merges the split partials in split order, skipping empty
// splits, and writes numerator / denominator.
template <class T>
__global__ void decode_combine_kernel(const float* __restrict__ partials, T* __restrict__ out, int rows,
                                      int splits, int dim_v) {
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* rec = partials + static_cast<size_t>(row) * splits * (dim_v + 2);
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, rec[static_cast<size_t>(s) * (dim_v + 2)]);
    float den = 0.0F;
    for (int s = 0; s < splits; ++s) {
        const float ms = rec[static_cast<size_t>(s) * (dim_v + 2)];
        if (ms != -INFINITY) den += rec[static_cast<size_t>(s) * (dim_v + 2) + 1] * expf(ms - m);
    }
    for (int d = lane; d < dim_v; d += 32) {
        float a = 0.0F;
        for (int s = 0; s < splits; ++s) {
            const float ms = rec[static_cast<size_t>(s) * (dim_v + 2)];
            if (ms != -INFINITY) a += rec[static_cast<size_t>(s) * (dim_v + 2) + 2 + d] * expf(ms - m);
        }
        out[static_cast<size_t>(row) * dim_v + d] = from_float<T>(a / den);
    }
}

// The same merge for at most 32 splits: lane s holds the record header of split s, the weights
// exp(max_s - max) / denominator are computed once per row and broadcast by shuffles, and the
// loads of all splits are independent.
template <class T>
__global__ void decode_combine_warp_kernel(const float* __restrict__ partials, T* __restrict__ out, int rows,
                                           int splits, int dim_v) {
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    grid_dependents_may_launch();
    grid_dependency_wait();  // the partials come from the kernel before
    if (row >= rows) return;
    const size_t record = static_cast<size_t>(dim_v) + 2;
    const float* rec = partials + static_cast<size_t>(row) * splits * record;
    float ms = -INFINITY, ls = 0.0F;
    if (lane < splits) {
        ms = rec[lane * record];
        ls = rec[lane * record + 1];
    }
    const float m = warp_max(ms);
    float w = ms == -INFINITY ? 0.0F : expf(ms - m);
    float den = 0.0F;
    for (int s = 0; s < splits; ++s) den += __shfl_sync(0xffffffffu, ls * w, s);  // split order, as the serial merge
    for (int d = lane; d < dim_v; d += 32) {
        float a = 0.0F;
        for (int s = 0; s < splits; ++s) {
            const float ws = __shfl_sync(0xffffffffu, w, s);
            if (ws != 0.0F) a += rec[s * record + 2 + d] * ws;
        }
        out[static_cast<size_t>(row) * dim_v + d] = from_float<T>(a / den);
    }
}

template <class T>
__global__ void paged_append_kernel(const T* __restrict__ new_k, const T* __restrict__ new_v, T* __restrict__ k_pool,
                                    T* __restrict__ v_pool, const int* __restrict__ table,
                                    const int* __restrict__ start_len, int batch, int kv_heads, int tokens, int dim,
                                    int dim_v, int P, int max_blocks, int num_blocks, uint32_t* status) {
    const int width = dim + dim_v;
    const int64_t total = static_cast<int64_t>(batch) * kv_heads * tokens * width;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int c = static_cast<int>(i % width);
        const int64_t r = i / width;
        const int t = static_cast<int>(r % tokens);
        const int h = static_cast<int>((r / tokens) % kv_heads);
        const int b = static_cast<int>(r / tokens / kv_heads);
        const int pos = start_len[b] + t;
        // a position past the table or a block id outside the pool (num_blocks > 0) is skipped and flagged
        if (pos < 0 || pos / P >= max_blocks) { atomicOr(status, kCodeDecodeBounds); continue; }
        const int page = table[static_cast<size_t>(b) * max_blocks + pos / P];
        if (page < 0 || (num_blocks > 0 && page >= num_blocks)) { atomicOr(status, kCodeDecodeBounds); continue; }
        const size_t row = (static_cast<size_t>(page) * kv_heads + h) * P + pos % P;
        const size_t src = (static_cast<size_t>(b) * kv_heads + h) * tokens + t;
        if (c < dim) k_pool[row * dim + c] = new_k[src * dim + c];
        else v_pool[row * dim_v + (c - dim)] = new_v[src * dim_v + (c - dim)];
    }
}

template <class T>
__global__ void paged_gather_kernel(const T* __restrict__ k_pool, const T* __restrict__ v_pool, T* __restrict__ keys,
                                    T* __restrict__ values, const int* __restrict__ table, int batch, int kv_heads,
                                    int length, int dim, int dim_v, int P, int max_blocks) {
    const int width = dim + dim_v;
    const int64_t total = static_cast<int64_t>(batch) * kv_heads * length * width;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int c = static_cast<int>(i % width);
        const int64_t r = i / width;
        const int t = static_cast<int>(r % length);
        const int h = static_cast<int>((r / length) % kv_heads);
        const int b = static_cast<int>(r / length / kv_heads);
        const int page = table[static_cast<size_t>(b) * max_blocks + t / P];
        const size_t row = (static_cast<size_t>(page) * kv_heads + h) * P + t % P;
        const size_t dst = (static_cast<size_t>(b) * kv_heads + h) * length + t;
        if (c < dim) keys[dst * dim + c] = k_pool[row * dim + c];
        else values[dst * dim_v + (c - dim)] = v_pool[row * dim_v + (c - dim)];
    }
}

int stream_grid(int64_t work) {
    const int64_t blocks = ceil_div64(work, 256);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace
}  // namespace sfb

using namespace sfb;

extern "C" {

sfb_status sfb_k_attention_prefill(const sfb_attention_args* a, sfb_stream stream) {
    SFB_REQUIRE(a && a->q && a->key && a->value && a->out, "attention: null tensor");
    SFB_REQUIRE(a->batch > 0 && a->q_heads > 0 && a->kv_heads > 0 && a->seq_q > 0 && a->seq_kv > 0 &&
                a->head_dim > 0 && a->head_dim_value > 0 && a->q_heads % a->kv_heads == 0,
                "invalid attention configuration");
    SFB_REQUIRE(!a->causal || a->seq_q <= a->seq_kv, "causal attention requires sequence_query <= sequence_kv");
    SFB_REQUIRE((a->q_head_rows == 0 || a->q_head_rows >= a->seq_q) && (a->kv_head_rows == 0 || a->kv_head_rows >= a->seq_kv),
                "attention: head strides shorter than the sequences");
    sfb_attention_args args = *a;
    if (args.scale <= 0.0F) args.scale = 1.0F / sqrtf(static_cast<float>(args.head_dim));
    int backend = args.backend;
    if (backend == 0) backend = attention_prefill_tcgen05_supported(args) ? 2 : 1;
    if (backend == 2) {
        if (!attention_prefill_tcgen05_supported(args))
            return fail(SFB_UNSUPPORTED, "attention: shape not supported by the tcgen05 kernel");
        return attention_prefill_tcgen05(args, as_stream(stream));
    }
    if ((args.q_head_rows > 0 && args.q_head_rows != args.seq_q) || (args.kv_head_rows > 0 && args.kv_head_rows != args.seq_kv))
        return fail(SFB_UNSUPPORTED, "attention: slices of longer sequences need the tcgen05 kernel");
    if (args.head_dim_value > 32 * kMaxChunks || args.head_dim > 512)
        return fail(SFB_UNSUPPORTED, "attention: head_dim_value > 256 is not supported");
    PrefillParams p{args.q, args.key, args.value, args.out, args.batch, args.q_heads, args.kv_heads,
                    args.seq_q, args.seq_kv, args.head_dim, args.head_dim_value, args.causal,
                    args.token_major, args.scale};
    const int rows_per_block = kWarps * kRowsPerWarp;
    const int grid = args.batch * args.q_heads * ceil_div(args.seq_q, rows_per_block);
    const size_t smem = sizeof(float) * (static_cast<size_t>(kTileKeys) * (args.head_dim + 1) +
                                         static_cast<size_t>(kTileKeys) * args.head_dim_value +
                                         static_cast<size_t>(rows_per_block) * args.head_dim);
    if (args.dtype == SFB_F32) {
        if (smem > 48 * 1024)
            SFB_CUDA(cudaFuncSetAttribute(attention_prefill_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attention_prefill_kernel<float><<<grid, kWarps * 32, smem, as_stream(stream)>>>(p);
    } else {
        if (smem > 48 * 1024)
            SFB_CUDA(cudaFuncSetAttribute(attention_prefill_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attention_prefill_kernel<bf16><<<grid, kWarps * 32, smem, as_stream(stream)>>>(p);
    }
    return check_launch("attention_prefill");
}

size_t sfb_attention_decode_workspace(int batch, int q_heads, int head_dim_value, int splits) {
    return sizeof(float) * static_cast<size_t>(batch) * q_heads * (splits < 1 ? 1 : splits) * (head_dim_value + 2);
}

int sfb_attention_decode_default_splits(int batch, int kv_heads, int max_context) {
    // Long splits stream best (a CTA's pipeline fill is paid once per split: 2048-token splits reach
    // 0.85 of the copy bandwidth, 512-token splits 0.75); shorter ones, down to 128 tokens, only while
    // there are too few (sequence, kv head, split) blocks for eight per SM.
    const int base = batch * kv_heads > 0 ? batch * kv_heads : 1;
    int chunk = 2048;
    int splits = (max_context + chunk - 1) / chunk;
    while (static_cast<long long>(base) * splits < 8LL * sm_count() && chunk > 128) {
        chunk /= 2;
        splits = (max_context + chunk - 1) / chunk;
    }
    if (splits > 128) splits = 128;
    return splits < 1 ? 1 : splits;
}

sfb_status sfb_k_attention_decode_paged(const sfb_decode_args* a, sfb_stream stream) {
    SFB_REQUIRE(a && a->q && a->k_pool && a->v_pool && a->block_table && (a->context_len || a->uniform_context > 0) &&
                    a->out && a->partials,
                "paged decode: null tensor");
    SFB_REQUIRE(a->batch > 0 && a->q_heads > 0 && a->kv_heads > 0 && a->head_dim > 0 && a->head_dim_value > 0 &&
                a->block_tokens > 0 && a->max_blocks > 0 && a->q_heads % a->kv_heads == 0,
                "invalid grouped-query attention configuration");
    const int splits = a->splits > 0 ? a->splits
                                     : sfb_attention_decode_default_splits(a->batch, a->kv_heads, a->max_context);
    DecodeParams p{a->q, a->k_pool, a->v_pool, a->block_table, a->context_len, a->out,
                   static_cast<float*>(a->partials), a->batch, a->q_heads, a->kv_heads, a->head_dim,
                   a->head_dim_value, a->block_tokens, a->max_blocks, splits,
                   a->scale > 0.0F ? a->scale : 1.0F / sqrtf(static_cast<float>(a->head_dim)), 0, 0, 0, nullptr, a->uniform_context};
    {
        const int bound = a->max_context > 0 ? a->max_context : a->max_blocks * a->block_tokens;
        const int granule = 4 * a->block_tokens;
        p.chunk_tokens = ceil_div(ceil_div(bound, splits), granule) * granule;
        const long long covered = static_cast<long long>(splits) * p.chunk_tokens;
        const long long table_tokens = static_cast<long long>(a->max_blocks) * a->block_tokens;
        p.context_limit = static_cast<int>(covered < table_tokens ? covered : table_tokens);
        p.num_blocks = a->num_blocks;
        p.status = device_status_word();
    }
    cudaStream_t s = as_stream(stream);
    const int group = a->q_heads / a->kv_heads;
    const int pages_bound = ceil_div(ceil_div(a->max_context > 0 ? a->max_context : a->max_blocks * a->block_tokens,
                                              a->block_tokens), splits) + 2;
    const bool fast = a->dtype == SFB_BF16 && a->head_dim == 128 && a->head_dim_value == 128 &&
                      a->block_tokens == 16 && a->num_blocks > 0 && pages_bound <= kDecodeMaxPages && group <= 8 &&
                      (reinterpret_cast<uintptr_t>(a->k_pool) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->v_pool) & 15) == 0;
    if (fast) {
        SFB_TRY(decode_paged_d128_launch(p, *a, group, s));
    } else {
        if (a->head_dim_value > 256) return fail(SFB_UNSUPPORTED, "paged decode: head_dim_value > 256");
        dim3 grid(a->batch * a->q_heads, splits);
        const size_t smem = sizeof(float) * (a->head_dim + 128);
        if (a->dtype == SFB_F32) decode_paged_generic_kernel<float><<<grid, 128, smem, s>>>(p);
        else decode_paged_generic_kernel<bf16><<<grid, 128, smem, s>>>(p);
    }
    SFB_TRY(check_launch("attention_decode_paged"));
    const int rows = a->batch * a->q_heads;
    if (splits <= 32 && a->head_dim_value % 32 == 0) {
        if (a->dtype == SFB_F32)
            SFB_CUDA(launch_dependent(decode_combine_warp_kernel<float>, dim3(ceil_div(rows, 4)), dim3(128), 0, s,
                                      static_cast<const float*>(p.partials), static_cast<float*>(a->out), rows, splits, a->head_dim_value));
        else
            SFB_CUDA(launch_dependent(decode_combine_warp_kernel<bf16>, dim3(ceil_div(rows, 4)), dim3(128), 0, s,
                                      static_cast<const float*>(p.partials), static_cast<bf16*>(a->out), rows, splits, a->head_dim_value));
    } else if (a->dtype == SFB_F32)
        decode_combine_kernel<float><<<ceil_div(rows, 4), 128, 0, s>>>(p.partials, static_cast<float*>(a->out), rows, splits, a->head_dim_value);
    else
        decode_combine_kernel<bf16><<<ceil_div(rows, 4), 128, 0, s>>>(p.partials, static_cast<bf16*>(a->out), rows, splits, a->head_dim_value);
    return check_launch("attention_decode_combine");
}

sfb_status sfb_k_paged_kv_append(const void* new_k, const void* new_v, void* k_pool, void* v_pool,
                                 const int* block_table, const int* start_len, int batch,
                                 int kv_heads, int tokens, int head_dim, int head_dim_value,
                                 int block_tokens, int max_blocks, int num_blocks, sfb_dtype dtype, sfb_stream stream) {
    SFB_REQUIRE(new_k && new_v && k_pool && v_pool && block_table && start_len, "paged append: null tensor");
    SFB_REQUIRE(batch > 0 && kv_heads > 0 && tokens > 0 && head_dim > 0 && head_dim_value > 0 && block_tokens > 0 &&
                    max_blocks > 0,
                "paged KV append shape mismatch");
    uint32_t* status = device_status_word();
    const int64_t work = static_cast<int64_t>(batch) * kv_heads * tokens * (head_dim + head_dim_value);
    const int grid = stream_grid(work);
    if (dtype == SFB_F32)
        paged_append_kernel<float><<<grid, 256, 0, as_stream(stream)>>>(
            static_cast<const float*>(new_k), static_cast<const float*>(new_v), static_cast<float*>(k_pool),
            static_cast<float*>(v_pool), block_table, start_len, batch, kv_heads, tokens, head_dim, head_dim_value,
            block_tokens, max_blocks, num_blocks, status);
    else
        paged_append_kernel<bf16><<<grid, 256, 0, as_stream(stream)>>>(
            static_cast<const bf16*>(new_k), static_cast<const bf16*>(new_v), static_cast<bf16*>(k_pool),
            static_cast<bf16*>(v_pool), block_table, start_len, batch, kv_heads, tokens, head_dim, head_dim_value,
            block_tokens, max_blocks, num_blocks, status);
    return check_launch("paged_kv_append");
}

sfb_status sfb_k_paged_kv_gather(const void* k_pool, const void* v_pool, void* keys, void* values,
                                 const int* block_table, int batch, int kv_heads, int length,
                                 int head_dim, int head_dim_value, int block_tokens,
                                 int max_blocks, sfb_dtype dtype, sfb_stream stream) {
    SFB_REQUIRE(k_pool && v_pool && keys && values && block_table, "paged gather: null tensor");
    SFB_REQUIRE(length > 0, "cannot gather empty paged KV cache");
    const int64_t work = static_cast<int64_t>(batch) * kv_heads * length * (head_dim + head_dim_value);
    const int grid = stream_grid(work);
    if (dtype == SFB_F32)
        paged_gather_kernel<float><<<grid, 256, 0, as_stream(stream)>>>(
            static_cast<const float*>(k_pool), static_cast<const float*>(v_pool), static_cast<float*>(keys),
            static_cast<float*>(values), block_table, batch, kv_heads, length, head_dim, head_dim_value,
            block_tokens, max_blocks);
    else
        paged_gather_kernel<bf16><<<grid, 256, 0, as_stream(stream)>>>(
            static_cast<const bf16*>(k_pool), static_cast<const bf16*>(v_pool), static_cast<bf16*>(keys),
            static_cast<bf16*>(values), block_table, batch, kv_heads, length, head_dim, head_dim_value,
            block_tokens, max_blocks);
    return check_launch("paged_kv_gather");
}

}  // extern "C"
