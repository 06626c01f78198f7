// MoE routing chain: router + softmax + top-k + histogram, prefix sum + stable dispatch,
// weighted combine.  All integer outputs (expert ids, counts, offsets, the dispatch
// permutation) are deterministic and equal to the sequential reference's: the router
// accumulates each logit as a sequential float sum (multiply rounded, add rounded,
// features ascending), and the dispatch ranks every assignment by counting earlier
// assignments to the same expert instead of racing on atomics.
#include <algorithm>

#include "common.cuh"

#include <mutex>

namespace sfb {
namespace {

constexpr int kMaxExperts = 64;
constexpr int kMaxTopK = 8;
constexpr int kFeatureChunk = 128;
constexpr int kChunk = 1024;  // assignments per dispatch block

// Second half of the router for thread (tl, e) that holds logit `acc`: bias, softmax over the experts,
// top-k (descending logit, ties to the lower id), renormalised weights, histogram.
template <class Dummy = void>
__device__ __forceinline__ void route_finish(float acc, float* logits, const float* __restrict__ bias, int tokens,
                                             int experts, int top_k, int token0, int tl, int e,
                                             int* __restrict__ expert_ids, float* __restrict__ expert_weights,
                                             int* __restrict__ counts) {
    if (bias) acc = __fadd_rn(acc, bias[e]);
    logits[tl * experts + e] = acc;
    __syncthreads();
    const int token = token0 + tl;
    if (e != 0 || token >= tokens) return;
    const float* l = logits + tl * experts;
    float mx = -INFINITY;
    for (int i = 0; i < experts; ++i) mx = fmaxf(mx, l[i]);
    float den = 0.0F;
    for (int i = 0; i < experts; ++i) den = __fadd_rn(den, expf(l[i] - mx));
    // top-k by descending logit (= descending softmax numerator), ties to the lower id
    int chosen[kMaxTopK];
    unsigned long long taken = 0ULL;
    for (int s = 0; s < top_k; ++s) {
        int best = -1;
        float best_value = -INFINITY;
        for (int i = 0; i < experts; ++i) {
            if ((taken >> i) & 1ULL) continue;
            if (best < 0 || l[i] > best_value) { best = i; best_value = l[i]; }
        }
        taken |= 1ULL << best;
        chosen[s] = best;
    }
    float selected = 0.0F;
    for (int s = 0; s < top_k; ++s) selected = __fadd_rn(selected, __fdiv_rn(expf(l[chosen[s]] - mx), den));
    for (int s = 0; s < top_k; ++s) {
        const int id = chosen[s];
        expert_ids[static_cast<size_t>(token) * top_k + s] = id;
        expert_weights[static_cast<size_t>(token) * top_k + s] = __fdiv_rn(__fdiv_rn(expf(l[id] - mx), den), selected);
        atomicAdd(&counts[id], 1);  // integer histogram: order-independent
    }
}

// blockDim = tokens_per_block * experts.  Thread (t, e) owns logit[t][e].
// The features are walked in chunks of 128 through shared memory.  A logit is a serial chain of
// 4096 rounded additions by definition (the oracle's order), so everything else must stay off that
// path: the next chunk's activations and router columns are fetched into registers (16-byte
// loads) before the current chunk is summed and parked in shared memory afterwards.
template <class T>
__global__ void moe_route_kernel(const T* __restrict__ x, const float* __restrict__ router,
                                 const float* __restrict__ bias, int tokens, int hidden, int experts,
                                 int top_k, int tokens_per_block, int* __restrict__ expert_ids,
                                 float* __restrict__ expert_weights, int* __restrict__ counts) {
    extern __shared__ float smem[];
    float* xs = smem;                                              // [tpb][chunk+1]
    float* ws = xs + tokens_per_block * (kFeatureChunk + 1);       // [chunk][E]
    float* logits = ws + kFeatureChunk * experts;                  // [tpb][E]
    const int e = threadIdx.x % experts, tl = threadIdx.x / experts;
    const int token0 = blockIdx.x * tokens_per_block;
    constexpr int kGroupsMax = 4;  // groups of 8 features per thread and chunk (host picks the block size accordingly)
    const int x_groups = tokens_per_block * (kFeatureChunk / 8);   // 8 features each
    const int w_groups = kFeatureChunk * experts / 4;              // 4 floats each
    const bool vector_x = (hidden % 8 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0);
    const bool vector_w = (experts % 4 == 0) && (reinterpret_cast<uintptr_t>(router) % 16 == 0);
    float xr[kGroupsMax][8];
    float4 wr[kGroupsMax];
    auto fetch = [&](int f0) {
        const int fn = min(kFeatureChunk, hidden - f0);
#pragma unroll
        for (int k = 0; k < kGroupsMax; ++k) {
            const int g = threadIdx.x + k * blockDim.x;
            if (g < x_groups) {
                const int t = g / (kFeatureChunk / 8), f = (g % (kFeatureChunk / 8)) * 8;
                const bool row_ok = token0 + t < tokens;
                const T* src = x + static_cast<size_t>(token0 + t) * hidden + f0 + f;
                if (row_ok && vector_x && f + 8 <= fn) {
                    if constexpr (sizeof(T) == 2) {
                        const uint4 packed = *reinterpret_cast<const uint4*>(src);
                        const bf16* v = reinterpret_cast<const bf16*>(&packed);
#pragma unroll
                        for (int j = 0; j < 8; ++j) xr[k][j] = to_float(v[j]);
                    } else {
                        const float4 lo = reinterpret_cast<const float4*>(src)[0], hi = reinterpret_cast<const float4*>(src)[1];
                        xr[k][0] = lo.x; xr[k][1] = lo.y; xr[k][2] = lo.z; xr[k][3] = lo.w;
                        xr[k][4] = hi.x; xr[k][5] = hi.y; xr[k][6] = hi.z; xr[k][7] = hi.w;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) xr[k][j] = (row_ok && f + j < fn) ? to_float(src[j]) : 0.0F;
                }
            }
            if (g < w_groups) {
                const int i = g * 4;
                const float* src = router + static_cast<size_t>(f0) * experts + i;
                if (vector_w && i + 4 <= fn * experts) {
                    wr[k] = *reinterpret_cast<const float4*>(src);
                } else {
                    wr[k].x = i < fn * experts ? src[0] : 0.0F;
                    wr[k].y = i + 1 < fn * experts ? src[1] : 0.0F;
                    wr[k].z = i + 2 < fn * experts ? src[2] : 0.0F;
                    wr[k].w = i + 3 < fn * experts ? src[3] : 0.0F;
                }
            }
        }
    };
    auto park = [&]() {
#pragma unroll
        for (int k = 0; k < kGroupsMax; ++k) {
            const int g = threadIdx.x + k * blockDim.x;
            if (g < x_groups) {
                const int t = g / (kFeatureChunk / 8), f = (g % (kFeatureChunk / 8)) * 8;
#pragma unroll
                for (int j = 0; j < 8; ++j) xs[t * (kFeatureChunk + 1) + f + j] = xr[k][j];
            }
            if (g < w_groups) {
                float* dst = ws + g * 4;
                dst[0] = wr[k].x; dst[1] = wr[k].y; dst[2] = wr[k].z; dst[3] = wr[k].w;
            }
        }
    };
    float acc = 0.0F;
    fetch(0);
    for (int f0 = 0; f0 < hidden; f0 += kFeatureChunk) {
        const int fn = min(kFeatureChunk, hidden - f0);
        __syncthreads();  // the previous chunk has been consumed
        park();
        __syncthreads();
        if (f0 + kFeatureChunk < hidden) fetch(f0 + kFeatureChunk);  // in flight while this chunk is summed
        const float* xrow = xs + tl * (kFeatureChunk + 1);
        int f = 0;
        for (; f + 8 <= fn; f += 8) {
            float product[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) product[j] = __fmul_rn(xrow[f + j], ws[(f + j) * experts + e]);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = __fadd_rn(acc, product[j]);
        }
        for (; f < fn; ++f) acc = __fadd_rn(acc, __fmul_rn(xrow[f], ws[f * experts + e]));
    }
    route_finish(acc, logits, bias, tokens, experts, top_k, token0, tl, e, expert_ids, expert_weights, counts);
}

// Plain form of the router (any number of experts): the chunk is staged with scalar loads.
template <class T>
__global__ void moe_route_simple_kernel(const T* __restrict__ x, const float* __restrict__ router,
                                 const float* __restrict__ bias, int tokens, int hidden, int experts,
                                 int top_k, int tokens_per_block, int* __restrict__ expert_ids,
                                 float* __restrict__ expert_weights, int* __restrict__ counts) {
    extern __shared__ float smem[];
    float* xs = smem;                                              // [tpb][chunk+1]
    float* ws = xs + tokens_per_block * (kFeatureChunk + 1);       // [chunk][E]
    float* logits = ws + kFeatureChunk * experts;                  // [tpb][E]
    const int e = threadIdx.x % experts, tl = threadIdx.x / experts;
    const int token0 = blockIdx.x * tokens_per_block;
    float acc = 0.0F;
    for (int f0 = 0; f0 < hidden; f0 += kFeatureChunk) {
        const int fn = min(kFeatureChunk, hidden - f0);
        __syncthreads();
        for (int i = threadIdx.x; i < tokens_per_block * kFeatureChunk; i += blockDim.x) {
            const int t = i / kFeatureChunk, f = i % kFeatureChunk;
            xs[t * (kFeatureChunk + 1) + f] = (token0 + t < tokens && f < fn)
                ? to_float(x[static_cast<size_t>(token0 + t) * hidden + f0 + f]) : 0.0F;
        }
        for (int i = threadIdx.x; i < fn * experts; i += blockDim.x)
            ws[i] = router[static_cast<size_t>(f0) * experts + i];
        __syncthreads();
        const float* xrow = xs + tl * (kFeatureChunk + 1);
        for (int f = 0; f < fn; ++f) acc = __fadd_rn(acc, __fmul_rn(xrow[f], ws[f * experts + e]));
    }
    route_finish(acc, logits, bias, tokens, experts, top_k, token0, tl, e, expert_ids, expert_weights, counts);
}

__global__ void dispatch_histogram_kernel(const int* __restrict__ expert_ids, int assignments, int experts,
                                          int* __restrict__ chunk_counts) {
    __shared__ int hist[kMaxExperts];
    if (threadIdx.x < experts) hist[threadIdx.x] = 0;
    __syncthreads();
    const int i = blockIdx.x * kChunk + threadIdx.x;
    if (i < assignments) atomicAdd(&hist[expert_ids[i]], 1);
    __syncthreads();
    if (threadIdx.x < experts) chunk_counts[blockIdx.x * experts + threadIdx.x] = hist[threadIdx.x];
}

// One block.  offsets = exclusive scan of counts; chunk_counts[c][e] becomes the first
// destination row of expert e's assignments inside chunk c.
__global__ void dispatch_scan_kernel(const int* __restrict__ counts, int experts, int chunks,
                                     int* __restrict__ offsets, int* __restrict__ chunk_counts) {
    __shared__ int base[kMaxExperts + 1];
    if (threadIdx.x == 0) {
        int running = 0;
        for (int e = 0; e < experts; ++e) { base[e] = running; offsets[e] = running; running += counts[e]; }
        base[experts] = running;
        offsets[experts] = running;
    }
    __syncthreads();
    if (threadIdx.x < experts) {
        int running = base[threadIdx.x];
        for (int c = 0; c < chunks; ++c) {
            const int n = chunk_counts[c * experts + threadIdx.x];
            chunk_counts[c * experts + threadIdx.x] = running;
            running += n;
        }
    }
}

// Stable rank inside the chunk: earlier lanes of the same warp via ballot, earlier warps
// via a shared per-warp histogram.
__global__ void __launch_bounds__(kChunk)
dispatch_rank_kernel(const int* __restrict__ expert_ids, const float* __restrict__ expert_weights,
                     const int* __restrict__ chunk_base, int assignments, int experts, int top_k,
                     int* __restrict__ token_ids, int* __restrict__ route_slots,
                     float* __restrict__ routing_weights, int* __restrict__ dest_of) {
    __shared__ int warp_hist[kChunk / 32][kMaxExperts];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i = blockIdx.x * kChunk + threadIdx.x;
    const int mine = i < assignments ? expert_ids[i] : -1;
    int lane_rank = 0;
    for (int e = 0; e < experts; ++e) {
        const unsigned votes = __ballot_sync(0xffffffffu, mine == e);
        if (mine == e) lane_rank = __popc(votes & ((1u << lane) - 1u));
        if (lane == 0) warp_hist[warp][e] = __popc(votes);
    }
    __syncthreads();
    if (mine < 0) return;
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_hist[w][mine];
    const int dest = chunk_base[blockIdx.x * experts + mine] + before + lane_rank;
    token_ids[dest] = i / top_k;
    route_slots[dest] = i % top_k;
    routing_weights[dest] = expert_weights[i];
    dest_of[i] = dest;
}

// values[dest_of[a], :] = x[a / top_k, :], 16-byte vectors when the row allows it.
template <class T>
__global__ void dispatch_gather_kernel(const T* __restrict__ x, const int* __restrict__ dest_of,
                                       T* __restrict__ values, int assignments, int hidden, int top_k) {
    constexpr int kVec = 16 / sizeof(T);
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    if (hidden % kVec == 0) {
        const int vec_per_row = hidden / kVec;
        const int64_t total = static_cast<int64_t>(assignments) * vec_per_row;
        for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
            const int a = static_cast<int>(i / vec_per_row), v = static_cast<int>(i % vec_per_row);
            const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(a / top_k) * hidden);
            uint4* dst = reinterpret_cast<uint4*>(values + static_cast<size_t>(dest_of[a]) * hidden);
            dst[v] = src[v];
        }
    } else {
        const int64_t total = static_cast<int64_t>(assignments) * hidden;
        for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
            const int a = static_cast<int>(i / hidden), f = static_cast<int>(i % hidden);
            values[static_cast<size_t>(dest_of[a]) * hidden + f] = x[static_cast<size_t>(a / top_k) * hidden + f];
        }
    }
}

// One thread per (token, feature): contributions in ascending dispatched position, each
// `acc = acc + w*y` as a rounded multiply then a rounded add; then residual + acc.
// bf16, hidden % 8 == 0: one warp per token, a lane owns 8 adjacent features at a time (16-byte loads
// and stores); the slots are sorted once per token.  Same arithmetic per element as the kernel below.
__global__ void __launch_bounds__(256)
moe_combine_rows_kernel(const bf16* __restrict__ y, const int* __restrict__ dest_of,
                        const float* __restrict__ routing_weights, const bf16* __restrict__ residual,
                        bf16* __restrict__ out, int tokens, int hidden, int top_k) {
    const int warps = (gridDim.x * blockDim.x) >> 5, lane = threadIdx.x & 31;
    for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < tokens; t += warps) {
        int dest[kMaxTopK];
        float weight[kMaxTopK];
        for (int s = 0; s < top_k; ++s) dest[s] = dest_of[static_cast<size_t>(t) * top_k + s];
        for (int a = 1; a < top_k; ++a) {  // insertion sort, top_k <= 8
            const int v = dest[a];
            int b = a - 1;
            while (b >= 0 && dest[b] > v) { dest[b + 1] = dest[b]; --b; }
            dest[b + 1] = v;
        }
        for (int s = 0; s < top_k; ++s) weight[s] = routing_weights[dest[s]];
        for (int f = lane * 8; f < hidden; f += 256) {
            float acc[8] = {0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F};
            for (int s = 0; s < top_k; ++s) {
                const uint4 packed = *reinterpret_cast<const uint4*>(y + static_cast<size_t>(dest[s]) * hidden + f);
                const bf16* v = reinterpret_cast<const bf16*>(&packed);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], __fmul_rn(weight[s], to_float(v[j])));
            }
            uint4 result;
            bf16* r = reinterpret_cast<bf16*>(&result);
            if (residual) {
                const uint4 packed = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * hidden + f);
                const bf16* v = reinterpret_cast<const bf16*>(&packed);
#pragma unroll
                for (int j = 0; j < 8; ++j) r[j] = from_float<bf16>(__fadd_rn(to_float(v[j]), acc[j]));
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) r[j] = from_float<bf16>(acc[j]);
            }
            *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * hidden + f) = result;
        }
    }
}

template <class T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ dest_of,
                                   const float* __restrict__ routing_weights, const T* __restrict__ residual,
                                   T* __restrict__ out, int tokens, int hidden, int top_k) {
    const int64_t total = static_cast<int64_t>(tokens) * hidden;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int t = static_cast<int>(i / hidden), f = static_cast<int>(i % hidden);
        int dest[kMaxTopK];
        for (int s = 0; s < top_k; ++s) dest[s] = dest_of[static_cast<size_t>(t) * top_k + s];
        for (int a = 1; a < top_k; ++a) {  // insertion sort, top_k <= 8
            const int v = dest[a];
            int b = a - 1;
            while (b >= 0 && dest[b] > v) { dest[b + 1] = dest[b]; --b; }
            dest[b + 1] = v;
        }
        float acc = 0.0F;
        for (int s = 0; s < top_k; ++s)
            acc = __fadd_rn(acc, __fmul_rn(routing_weights[dest[s]], to_float(y[static_cast<size_t>(dest[s]) * hidden + f])));
        out[i] = from_float<T>(residual ? __fadd_rn(to_float(residual[i]), acc) : acc);
    }
}

__global__ void silu_mul_kernel(float* __restrict__ first, const float* __restrict__ gate, int64_t count) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        const float g = gate[i];
        first[i] = __fmul_rn(first[i], g / (1.0F + expf(-g)));
    }
}

int stream_grid(int64_t work) {
    const int64_t blocks = ceil_div64(work, 256);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace

void moe_silu_mul_f32(float* first, const float* gate, int64_t count, cudaStream_t stream) {
    silu_mul_kernel<<<stream_grid(count), 256, 0, stream>>>(first, gate, count);
    count_launch();
}

}  // namespace sfb

using namespace sfb;

// ---- scratch for the allocation-free dispatch entry point -------------------------------
// sfb_k_moe_dispatch_static serves callers that are not allowed to allocate device memory:
// code running inside a memory-budgeted serving process whose allocator owns every byte, a
// plugin loaded under a "no cudaMalloc after start-up" rule, or a real-time loop where an
// allocation could stall.  They still need the per-chunk histogram the dispatch kernels use
// as scratch, so the library carries one copy per GPU in its own image: the array below.
// It costs kStaticScratchInts * 4 bytes = 66 816 bytes on every GPU that loads the library,
// until the process exits.
constexpr int kStaticMaxAssignments = 262144;  // tokens * top_k the static variant accepts
constexpr int kStaticScratchInts = (kStaticMaxAssignments / kChunk + 1 + 4) * kMaxExperts;
static __device__ __align__(256) int g_dispatch_scratch[kStaticScratchInts];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
int* g_scratch_address[kMaxDevices] = {};

// Device address of g_dispatch_scratch on the CURRENT device.  In host code the array's name is
// only a handle for the runtime, not an address a kernel could use, so the address is asked
// for once per device with cudaGetSymbolAddress and remembered.
sfb_status static_scratch(int** address) {
    int device = 0;
    SFB_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return fail(SFB_UNSUPPORTED, "moe_dispatch_static: device index out of range");
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_address[device]) {
        void* symbol = nullptr;
        SFB_CUDA(cudaGetSymbolAddress(&symbol, g_dispatch_scratch));
        if (!symbol) return fail(SFB_CUDA_ERROR, "moe_dispatch_static: scratch symbol has no device address");
        g_scratch_address[device] = static_cast<int*>(symbol);
    }
    *address = g_scratch_address[device];
    return SFB_OK;
}
}  // namespace

extern "C" {

sfb_status sfb_k_moe_route(const void* x, sfb_dtype x_dtype, const float* router, const float* bias,
                           int tokens, int hidden, int experts, int top_k, int* expert_ids,
                           float* expert_weights, int* counts, sfb_stream stream) {
    SFB_REQUIRE(x && router && expert_ids && expert_weights && counts, "moe_route: null tensor");
    SFB_REQUIRE(tokens > 0 && hidden > 0 && experts > 0 && top_k > 0 && top_k <= experts, "invalid MoE configuration");
    if (experts > kMaxExperts || top_k > kMaxTopK)
        return fail(SFB_UNSUPPORTED, "moe_route: experts > 64 or top_k > 8");
    cudaStream_t s = as_stream(stream);
    SFB_CUDA(cudaMemsetAsync(counts, 0, sizeof(int) * experts, s));
    // The prefetching kernel gives every thread at most four 16-byte groups of activations and four of
    // router weights per chunk, which needs at least 4 experts and 8 tokens per block.
    const bool fast = experts >= 4;
    int tpb = fast ? 16 : 256 / experts;
    while (tpb * experts > 1024 && tpb > 8) tpb /= 2;
    if (tpb < 1) tpb = 1;
    if (!fast && tpb > 32) tpb = 32;
    const int block = tpb * experts;
    const int grid = ceil_div(tokens, tpb);
    const size_t smem = sizeof(float) * (static_cast<size_t>(tpb) * (kFeatureChunk + 1) +
                                         static_cast<size_t>(kFeatureChunk) * experts + static_cast<size_t>(tpb) * experts);
    auto launch = [&](auto kernel, auto* typed_x) -> sfb_status {
        if (smem > 48 * 1024)
            SFB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        kernel<<<grid, block, smem, s>>>(typed_x, router, bias, tokens, hidden, experts, top_k, tpb, expert_ids,
                                         expert_weights, counts);
        return SFB_OK;
    };
    if (x_dtype == SFB_F32)
        SFB_TRY(fast ? launch(moe_route_kernel<float>, static_cast<const float*>(x))
                     : launch(moe_route_simple_kernel<float>, static_cast<const float*>(x)));
    else
        SFB_TRY(fast ? launch(moe_route_kernel<bf16>, static_cast<const bf16*>(x))
                     : launch(moe_route_simple_kernel<bf16>, static_cast<const bf16*>(x)));
    return check_launch("moe_route");
}

size_t sfb_moe_dispatch_scratch_bytes(int tokens, int experts, int top_k) {
    const int64_t assignments = static_cast<int64_t>(tokens) * top_k;
    return sizeof(int) * static_cast<size_t>((assignments + kChunk - 1) / kChunk + 1) * experts;
}

sfb_status sfb_k_moe_dispatch(const void* x, sfb_dtype dtype, const int* expert_ids,
                              const float* expert_weights, const int* counts, int tokens, int hidden,
                              int experts, int top_k, void* values, int* offsets, int* token_ids,
                              int* route_slots, float* routing_weights, int* dest_of, int* scratch,
                              sfb_stream stream) {
    SFB_REQUIRE(expert_ids && expert_weights && counts && offsets && token_ids && route_slots && routing_weights &&
                dest_of && scratch, "moe_dispatch: null tensor");
    SFB_REQUIRE(tokens > 0 && hidden > 0 && experts > 0 && top_k > 0 && top_k <= experts,
                "routing trace does not match MoE configuration");
    if (experts > kMaxExperts || top_k > kMaxTopK)
        return fail(SFB_UNSUPPORTED, "moe_dispatch: experts > 64 or top_k > 8");
    cudaStream_t s = as_stream(stream);
    const int assignments = tokens * top_k;
    const int chunks = ceil_div(assignments, kChunk);
    dispatch_histogram_kernel<<<chunks, kChunk, 0, s>>>(expert_ids, assignments, experts, scratch);
    SFB_TRY(check_launch("moe_dispatch_histogram"));
    dispatch_scan_kernel<<<1, kMaxExperts, 0, s>>>(counts, experts, chunks, offsets, scratch);
    SFB_TRY(check_launch("moe_dispatch_scan"));
    dispatch_rank_kernel<<<chunks, kChunk, 0, s>>>(expert_ids, expert_weights, scratch, assignments, experts, top_k,
                                                    token_ids, route_slots, routing_weights, dest_of);
    SFB_TRY(check_launch("moe_dispatch_rank"));
    if (values) {
        SFB_REQUIRE(x, "moe_dispatch: null input");
        const int vec = dtype == SFB_F32 ? 4 : 8;
        const int64_t work = static_cast<int64_t>(assignments) * (hidden % vec == 0 ? hidden / vec : hidden);
        const int grid = stream_grid(work);
        if (dtype == SFB_F32)
            dispatch_gather_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), dest_of,
                                                               static_cast<float*>(values), assignments, hidden, top_k);
        else
            dispatch_gather_kernel<bf16><<<grid, 256, 0, s>>>(static_cast<const bf16*>(x), dest_of,
                                                              static_cast<bf16*>(values), assignments, hidden, top_k);
        SFB_TRY(check_launch("moe_dispatch_gather"));
    }
    return SFB_OK;
}

sfb_status sfb_k_moe_dispatch_static(const void* x, sfb_dtype dtype, const int* expert_ids,
                                     const float* expert_weights, const int* counts, int tokens, int hidden,
                                     int experts, int top_k, void* values, int* offsets, int* token_ids,
                                     int* route_slots, float* routing_weights, int* dest_of,
                                     sfb_stream stream) {
    SFB_REQUIRE(tokens > 0 && top_k > 0 && experts > 0, "routing trace does not match MoE configuration");
    if (static_cast<int64_t>(tokens) * top_k > kStaticMaxAssignments || experts > kMaxExperts)
        return fail(SFB_UNSUPPORTED,
                    "moe_dispatch_static: tokens * top_k exceeds 262144 (or experts > 64), the size of the built-in "
                    "scratch; use sfb_k_moe_dispatch with caller-provided scratch");
    int* scratch = nullptr;
    SFB_TRY(static_scratch(&scratch));
    // Nothing in the scratch has to start at zero: the histogram kernel overwrites every entry the
    // later kernels read, so whatever the previous call left behind is never observed.
    return sfb_k_moe_dispatch(x, dtype, expert_ids, expert_weights, counts, tokens, hidden, experts, top_k, values,
                              offsets, token_ids, route_slots, routing_weights, dest_of, scratch, stream);
}

sfb_status sfb_k_moe_combine(const void* y, const int* dest_of, const float* routing_weights,
                             const void* residual, void* out, int tokens, int hidden, int top_k,
                             sfb_dtype dtype, sfb_stream stream) {
    SFB_REQUIRE(y && dest_of && routing_weights && out, "moe_combine: null tensor");
    SFB_REQUIRE(tokens > 0 && hidden > 0 && top_k > 0, "invalid MoE configuration");
    if (top_k > kMaxTopK) return fail(SFB_UNSUPPORTED, "moe_combine: top_k > 8");
    const int grid = stream_grid(static_cast<int64_t>(tokens) * hidden);
    if (dtype == SFB_F32)
        moe_combine_kernel<float><<<grid, 256, 0, as_stream(stream)>>>(
            static_cast<const float*>(y), dest_of, routing_weights, static_cast<const float*>(residual),
            static_cast<float*>(out), tokens, hidden, top_k);
    else if (hidden % 8 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(residual) & 15) == 0)
        moe_combine_rows_kernel<<<std::min(ceil_div(tokens, 8), sm_count() * 16), 256, 0, as_stream(stream)>>>(
            static_cast<const bf16*>(y), dest_of, routing_weights, static_cast<const bf16*>(residual),
            static_cast<bf16*>(out), tokens, hidden, top_k);
    else
        moe_combine_kernel<bf16><<<grid, 256, 0, as_stream(stream)>>>(
            static_cast<const bf16*>(y), dest_of, routing_weights, static_cast<const bf16*>(residual),
            static_cast<bf16*>(out), tokens, hidden, top_k);
    return check_launch("moe_combine");
}

}  // extern "C"
