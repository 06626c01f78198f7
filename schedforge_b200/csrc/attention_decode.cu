// Split-KV decode over a paged KV cache, bf16, head_dim = head_dim_value = 128, 16-token blocks.
//
// The kernel is HBM-bound: every K/V byte of a (sequence, kv head) must be read once.  One CTA
// (4 warps) handles one (sequence, kv head, split).  A KV block is moved from the pool into shared
// memory by TMA as two 16-row x 128-byte boxes with the 128-byte swizzle (plain tiled loads, no
// multicast), four blocks per pipeline stage, three stages in flight (~96 KiB per CTA), so the
// amount of data in flight does not depend on how many warps are resident.  Each warp takes one
// block per stage and does the arithmetic on the legacy warp-level tensor path (mma.sync
// m16n8k16, ldmatrix from the swizzled tile without bank conflicts): the group's query heads are
// the (zero-padded) 16 rows of the A operand, so all heads of the group share each K/V byte, and
// the instruction count per token is ~20x below a CUDA-core formulation, which keeps the issue
// slots from becoming the limiter.  Base-2 online softmax per warp with a lazily moved maximum;
// warps and splits are merged with the log-sum-exp rule (partials + combine kernel).
// The arithmetic here is deliberately NOT reshaped for tcgen05: with one query token per sequence
// the tensor work is negligible and the byte stream is what has to be kept full.
#include "attention_decode.cuh"
#include "ptx_sm100.cuh"

namespace sfb {
namespace {

constexpr int D = 128;
constexpr int P = 16;                       // tokens per KV block
constexpr int kStages = 3;
constexpr int kPagesPerStage = 4;           // one per warp
constexpr int kPageBytes = P * D * 2;       // 4 KiB: two 2 KiB halves (dims 0-63, 64-127)
constexpr int kStageBytes = 2 * kPagesPerStage * kPageBytes;  // K pages then V pages
constexpr int kThreads = 128;

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Address of 16-byte chunk `chunk` (0..15 over the 128 dims) of token row `row` inside a swizzled page.
__device__ __forceinline__ uint32_t page_chunk(uint32_t page, int row, int chunk) {
    return page + (chunk >> 3) * (kPageBytes / 2) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

template <int GROUP>
__global__ void __launch_bounds__(kThreads, 2)
decode_paged_mma_kernel(const __grid_constant__ CUtensorMap tma_k, const __grid_constant__ CUtensorMap tma_v,
                        const __grid_constant__ DecodeParams p, uint32_t* status) {
    constexpr float kLog2e = 1.4426950408889634F;
    extern __shared__ uint8_t decode_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(decode_smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
    uint64_t* empty_bar = full_bar + kStages;
    volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(empty_bar + kStages);
    int* page_ids = reinterpret_cast<int*>(empty_bar + kStages) + 2;

    const int split = blockIdx.z, kvh = blockIdx.y, b = blockIdx.x;
    grid_dependents_may_launch();
    grid_dependency_wait();  // the queries (and an appended page) come from the kernels before
    const int ctx = guarded_context(p, b);
    int begin, end;
    split_range(ctx, p.chunk_tokens, split, begin, end);
    if (begin >= end) {  // nothing of this sequence falls into this split: neutral partial
        for (int idx = threadIdx.x; idx < GROUP * D; idx += kThreads) {
            const int h = idx / D, d = idx % D;
            float* rec = p.partials + ((static_cast<size_t>(b) * p.q_heads + kvh * GROUP + h) * p.splits + split) * (D + 2);
            if (d == 0) { rec[0] = -INFINITY; rec[1] = 0.0F; }
            rec[2 + d] = 0.0F;
        }
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = lane >> 2, quad = lane & 3;   // fragment row (= query head of the group) and column pair

    // Q as A fragments for the 8 k-slices of 16 dims; rows >= GROUP and rows 8-15 are zero padding
    uint32_t qa[8][4];
    {
        const bf16* qrow = static_cast<const bf16*>(p.q) + (static_cast<size_t>(b) * p.q_heads + kvh * GROUP + row) * D;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            qa[s][0] = row < GROUP ? *reinterpret_cast<const uint32_t*>(qrow + 16 * s + quad * 2) : 0u;
            qa[s][2] = row < GROUP ? *reinterpret_cast<const uint32_t*>(qrow + 16 * s + 8 + quad * 2) : 0u;
            qa[s][1] = 0u;
            qa[s][3] = 0u;
        }
    }
    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0F; }
    float m_used = -INFINITY, l_part = 0.0F;   // l_part: this lane's share of the row sum
    const float scale = p.scale * kLog2e;

    const int first_block = begin / P, last_block = (end + P - 1) / P;
    const int n_pages = last_block - first_block;
    const int n_stages = (n_pages + kPagesPerStage - 1) / kPagesPerStage;
    const int* table = p.block_table + static_cast<size_t>(b) * p.max_blocks;
    for (int i = threadIdx.x; i < n_pages; i += kThreads) {
        int page = table[first_block + i];
        if (page < 0 || page >= p.num_blocks) {  // outside the pool: the copy then lies outside the tensor map and reads zeros
            page = p.num_blocks;
            atomicOr(status, kCodeDecodeBounds);
        }
        page_ids[i] = page;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 4);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
        ptx::prefetch_tensormap(&tma_k);
        ptx::prefetch_tensormap(&tma_v);
    }
    __syncthreads();
    auto issue_stage = [&](int it) -> bool {  // thread 0 only
        const int s = it % kStages;
        if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[s]), ((it / kStages) & 1) ^ 1, abort_flag, status, 0x20)) return false;
        const int np = min(kPagesPerStage, n_pages - it * kPagesPerStage);
        const uint32_t bar = ptx::smem_u32(&full_bar[s]);
        ptx::mbar_expect_tx(bar, static_cast<uint32_t>(np) * 2 * kPageBytes);
        const uint32_t stage = ptx::smem_u32(smem + s * kStageBytes);
        for (int w = 0; w < np; ++w) {
            const int pool_row = (page_ids[it * kPagesPerStage + w] * p.kv_heads + kvh) * P;
            const uint32_t kd = stage + w * kPageBytes, vd = stage + (kPagesPerStage + w) * kPageBytes;
            ptx::tma_load_2d(kd, &tma_k, bar, 0, pool_row);
            ptx::tma_load_2d(kd + kPageBytes / 2, &tma_k, bar, 64, pool_row);
            ptx::tma_load_2d(vd, &tma_v, bar, 0, pool_row);
            ptx::tma_load_2d(vd + kPageBytes / 2, &tma_v, bar, 64, pool_row);
        }
        return true;
    };
    if (threadIdx.x == 0)
        for (int it = 0; it < min(kStages, n_stages); ++it) issue_stage(it);

    for (int it = 0; it < n_stages; ++it) {
        const int s = it % kStages;
        if (!ptx::mbar_wait(ptx::smem_u32(&full_bar[s]), (it / kStages) & 1, abort_flag, status, 0x40)) break;
        const int local = it * kPagesPerStage + warp;
        if (local < n_pages) {
            const uint32_t kpage = ptx::smem_u32(smem + s * kStageBytes + warp * kPageBytes);
            const uint32_t vpage = kpage + kPagesPerStage * kPageBytes;
            const int token0 = (first_block + local) * P;
            // S[16 x 16] = Q . K^T: two n-tiles of 8 tokens, 8 k-slices
            float sc[2][4];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                sc[t][0] = sc[t][1] = sc[t][2] = sc[t][3] = 0.0F;
#pragma unroll
                for (int sp = 0; sp < 4; ++sp) {  // pairs of k-slices (32 dims)
                    uint32_t kb[4];
                    ldmatrix_x4(page_chunk(kpage, 8 * t + (lane & 7), 4 * sp + (lane >> 3)), kb);
                    mma_bf16(sc[t], qa[2 * sp], kb[0], kb[1]);
                    mma_bf16(sc[t], qa[2 * sp + 1], kb[2], kb[3]);
                }
            }
            // scores of row `row`: tokens 8t + 2*quad + {0,1}
            float x[4];
            float tile_max = -INFINITY;
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int token = token0 + 8 * t + 2 * quad + e;
                    x[2 * t + e] = token < end ? sc[t][e] * scale : -INFINITY;
                    tile_max = fmaxf(tile_max, x[2 * t + e]);
                }
            tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
            tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
            if (tile_max > m_used + 8.0F) {  // lazily moved maximum (also the first block: m_used = -inf)
                const float alpha = fast_exp2(m_used - tile_max);
                l_part *= alpha;
#pragma unroll
                for (int j = 0; j < 16; ++j) { o[j][0] *= alpha; o[j][1] *= alpha; }
                m_used = tile_max;
            }
            uint32_t pa[4];
            {
                float pr[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    pr[i] = x[i] == -INFINITY ? 0.0F : fast_exp2(x[i] - m_used);
                    l_part += pr[i];
                }
                pa[0] = pack_bf16(pr[0], pr[1]);   // tokens 0-7 of the block  (k 0..7)
                pa[2] = pack_bf16(pr[2], pr[3]);   // tokens 8-15               (k 8..15)
                pa[1] = 0u;
                pa[3] = 0u;
            }
            // O[16 x 128] += P[16 x 16] . V[16 x 128]: 16 n-tiles of 8 dims
#pragma unroll
            for (int jp = 0; jp < 8; ++jp) {
                uint32_t vb[4];
                ldmatrix_x4_trans(page_chunk(vpage, ((lane >> 3) & 1) * 8 + (lane & 7), 2 * jp + (lane >> 4)), vb);
                mma_bf16(o[2 * jp], pa, vb[0], vb[1]);
                mma_bf16(o[2 * jp + 1], pa, vb[2], vb[3]);
            }
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&empty_bar[s]));
        if (threadIdx.x == 0 && it + kStages < n_stages)
            if (!issue_stage(it + kStages)) break;
    }
    __syncthreads();
    if (*abort_flag)
        for (int i = 0; i < 200; ++i) __nanosleep(1000);  // let copies in flight land before the CTA exits

    // row sums: add the four column-pair lanes of each row
    l_part += __shfl_xor_sync(0xffffffffu, l_part, 1);
    l_part += __shfl_xor_sync(0xffffffffu, l_part, 2);
    // merge the four warps through shared memory (the pipeline buffers are free now)
    float* wm = reinterpret_cast<float*>(smem);            // [4][GROUP]
    float* wd = wm + 4 * GROUP;                            // [4][GROUP]
    float* wacc = wd + 4 * GROUP;                          // [4][GROUP][D]
    if (row < GROUP) {
        if (quad == 0) { wm[warp * GROUP + row] = m_used; wd[warp * GROUP + row] = l_part; }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float* dst = wacc + (static_cast<size_t>(warp) * GROUP + row) * D + 8 * j + 2 * quad;
            dst[0] = o[j][0];
            dst[1] = o[j][1];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < GROUP * D; idx += kThreads) {
        const int h = idx / D, d = idx % D;
        const float m = fmaxf(fmaxf(wm[h], wm[GROUP + h]), fmaxf(wm[2 * GROUP + h], wm[3 * GROUP + h]));
        float sum = 0.0F, a = 0.0F;
        if (m != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float mw = wm[w * GROUP + h];
                const float f = mw == -INFINITY ? 0.0F : fast_exp2(mw - m);
                sum += wd[w * GROUP + h] * f;
                a += wacc[(static_cast<size_t>(w) * GROUP + h) * D + d] * f;
            }
        }
        float* rec = p.partials + ((static_cast<size_t>(b) * p.q_heads + kvh * GROUP + h) * p.splits + split) * (D + 2);
        if (d == 0) { rec[0] = m * 0.6931471805599453F; rec[1] = sum; }  // maximum back in natural-log units
        rec[2 + d] = a;
    }
}

template <int GROUP>
sfb_status launch_group(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeParams& p, size_t smem, dim3 grid,
                        cudaStream_t stream) {
    SFB_CUDA(cudaFuncSetAttribute(decode_paged_mma_kernel<GROUP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(smem)));
    SFB_CUDA(launch_dependent(decode_paged_mma_kernel<GROUP>, grid, dim3(kThreads), smem, stream, mk, mv, p,
                              device_status_word()));
    return check_launch("attention_decode_paged_mma");
}

}  // namespace

sfb_status decode_paged_d128_launch(const DecodeParams& p, const sfb_decode_args& a, int group, cudaStream_t stream) {
    CUtensorMap mk, mv;
    const uint64_t rows = static_cast<uint64_t>(a.num_blocks > 0 ? a.num_blocks : 1) * a.kv_heads * P;
    if (!encode_tensor_map_bf16_2d(&mk, a.k_pool, rows, D, P, 64) || !encode_tensor_map_bf16_2d(&mv, a.v_pool, rows, D, P, 64))
        return SFB_CUDA_ERROR;
    const int pages_per_split = p.chunk_tokens / P + 2;
    const size_t smem = static_cast<size_t>(kStages) * kStageBytes + 64 + sizeof(int) * (pages_per_split + 2) + 1024;
    dim3 grid(a.batch, a.kv_heads, p.splits);
    switch (group) {
        case 1: return launch_group<1>(mk, mv, p, smem, grid, stream);
        case 2: return launch_group<2>(mk, mv, p, smem, grid, stream);
        case 3: return launch_group<3>(mk, mv, p, smem, grid, stream);
        case 4: return launch_group<4>(mk, mv, p, smem, grid, stream);
        case 5: return launch_group<5>(mk, mv, p, smem, grid, stream);
        case 6: return launch_group<6>(mk, mv, p, smem, grid, stream);
        case 7: return launch_group<7>(mk, mv, p, smem, grid, stream);
        case 8: return launch_group<8>(mk, mv, p, smem, grid, stream);
        default: return fail(SFB_UNSUPPORTED, "paged decode: more than 8 query heads per kv head");
    }
}

}  // namespace sfb
