// bf16 GEMM on the 5th-generation tensor cores: out = epilogue(A[m,k] . Bt[n,k]^T).
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0      TMA producer: streams 128x64 A tiles and BNx64 B tiles (128-byte swizzle)
//               through a ring of shared-memory stages guarded by full/empty mbarriers;
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) four times per
//               stage into one of TWO accumulator buffers in tensor memory and commits the
//               stage back to the producer and the finished tile to the epilogue;
//   warps 2-5   epilogue: tcgen05.ld the accumulator (one row per thread, 32 columns at a
//               time), apply the fused epilogue and store straight to global memory, while
//               the MMA warp already works on the next tile in the other buffer.
// Epilogues: plain store, + residual, SwiGLU over [gate | up] halves of the tile, and
// RoPE + scatter into head-major Q/K/V for the fused QKV projection.
// Grouped mode (MoE experts): a device-built tile table maps every M-tile to a row range
// of one expert; the weight slab of that expert is addressed through the row coordinate
// of the B tensor map, rows outside the range are masked in the epilogue.
//
// Tiles are visited in bands of 16 M-tiles so that one band's A rows stay in L2 while
// the CTAs sweep the N direction.
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace sfb {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GROUP_M = 16;
constexpr int kThreads = 192;
constexpr uint32_t kCodeProducer = 0x1, kCodeMma = 0x2, kCodeEpilogue = 0x4;

template <int BN>
struct Tile {
    static constexpr int kStages = BN == 256 ? 4 : 6;
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kBarrierBytes = 256;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;
};

struct TcParams {
    void* out;
    int m, n, k;
    int epilogue, out_f32;
    const bf16* residual;
    bf16 *q, *key, *value;
    const float *rope_cos, *rope_sin;
    int seq, q_heads, kv_heads, head_dim;
    const int* tile_table;  // grouped: [0] = number of M-tiles, entries from [4]
    int dense_m_tiles;
    int n_tiles;
    uint32_t* status;
};

struct TileCoord {
    int row_start, row_end, group, n_index;
};

__device__ __forceinline__ int load_m_tiles(const TcParams& p) {
    return p.tile_table ? p.tile_table[0] : p.dense_m_tiles;
}

__device__ __forceinline__ TileCoord tile_coord(const TcParams& p, int tile, int m_tiles) {
    const int band_tiles = GROUP_M * p.n_tiles;
    const int band = tile / band_tiles;
    const int first_m = band * GROUP_M;
    const int band_m = min(GROUP_M, m_tiles - first_m);
    const int local = tile - band * band_tiles;
    const int m_index = first_m + local % band_m;
    TileCoord c;
    c.n_index = local / band_m;
    if (p.tile_table) {
        const int* e = p.tile_table + 4 + 4 * m_index;
        c.row_start = e[0];
        c.row_end = e[1];
        c.group = e[2];
    } else {
        c.row_start = m_index * BM;
        c.row_end = min(p.m, c.row_start + BM);
        c.group = 0;
    }
    return c;
}

// 32 consecutive outputs of one row: vector stores when the destination is 16-byte
// aligned and the chunk is complete, scalar stores otherwise.
__device__ __forceinline__ void store_chunk(void* out, int out_f32, size_t index, const float (&v)[32],
                                            int valid) {
    if (out_f32) {
        float* dst = static_cast<float*>(out) + index;
        if (valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
            for (int i = 0; i < valid; ++i) dst[i] = v[i];
        }
    } else {
        bf16* dst = static_cast<bf16*>(out) + index;
        if (valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 packed;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
                reinterpret_cast<uint4*>(dst)[i] = packed;
            }
        } else {
            for (int i = 0; i < valid; ++i) dst[i] = from_float<bf16>(v[i]);
        }
    }
}

__device__ __forceinline__ void load_bf16_chunk(const bf16* src, float (&v)[32], int valid) {
    if (valid == 32 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 packed = reinterpret_cast<const uint4*>(src)[i];
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&packed);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h[j]);
                v[8 * i + 2 * j] = f.x;
                v[8 * i + 2 * j + 1] = f.y;
            }
        }
    } else {
        for (int i = 0; i < 32; ++i) v[i] = i < valid ? to_float(src[i]) : 0.0F;
    }
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const __grid_constant__ TcParams p) {
    using T = Tile<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + T::kStages * T::kStageBytes);
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + T::kStages;
    uint64_t* tmem_full = bars + 2 * T::kStages;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < T::kStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&tmem_full[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&tmem_empty[b]), 128);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
        ptx::prefetch_tensormap(&tma_a);
        ptx::prefetch_tensormap(&tma_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), T::kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int m_tiles = load_m_tiles(p);
    const int total_tiles = m_tiles * p.n_tiles;
    const int k_blocks = (p.k + BK - 1) / BK;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const TileCoord c = tile_coord(p, tile, m_tiles);
                const int b_row = c.group * p.n + c.n_index * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % T::kStages, ph = (it / T::kStages) & 1;
                    if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[s]), ph ^ 1, abort_flag, p.status, kCodeProducer)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full = ptx::smem_u32(&full_bar[s]);
                    ptx::mbar_expect_tx(full, T::kStageBytes);
                    uint8_t* stage = smem + s * T::kStageBytes;
                    ptx::tma_load_2d(ptx::smem_u32(stage), &tma_a, full, kb * BK, c.row_start);
                    ptx::tma_load_2d(ptx::smem_u32(stage + T::kABytes), &tma_b, full, kb * BK, b_row);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16(BM, BN);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++tcount) {
                const uint32_t buf = tcount & 1, tph = (tcount >> 1) & 1;
                if (!ptx::mbar_wait(ptx::smem_u32(&tmem_empty[buf]), tph ^ 1, abort_flag, p.status, kCodeMma)) break;
                ptx::tc_fence_after();
                const uint32_t acc = tmem_base + buf * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % T::kStages, ph = (it / T::kStages) & 1;
                    if (!ptx::mbar_wait(ptx::smem_u32(&full_bar[s]), ph, abort_flag, p.status, kCodeMma)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    uint8_t* stage = smem + s * T::kStageBytes;
                    const uint64_t da = ptx::umma_desc_k_sw128(ptx::smem_u32(stage));
                    const uint64_t db = ptx::umma_desc_k_sw128(ptx::smem_u32(stage + T::kABytes));
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk)
                        ptx::umma_bf16(acc, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0);
                    ptx::umma_commit(ptx::smem_u32(&empty_bar[s]));
                }
                if (ok) ptx::umma_commit(ptx::smem_u32(&tmem_full[buf]));
            }
        }
    } else {
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        uint32_t tcount = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++tcount) {
            const TileCoord c = tile_coord(p, tile, m_tiles);
            const uint32_t buf = tcount & 1, tph = (tcount >> 1) & 1;
            if (!ptx::mbar_wait(ptx::smem_u32(&tmem_full[buf]), tph, abort_flag, p.status, kCodeEpilogue)) break;
            ptx::tc_fence_after();
            const uint32_t acc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            const int row = c.row_start + row_in_tile;
            const bool row_ok = row < c.row_end;
            const int n0 = c.n_index * BN;
            uint32_t r0[32];
            float v[32];
            if (p.epilogue == SFB_EPI_SWIGLU) {
                const int half_n = p.n / 2;
                uint32_t r1[32];
                for (int ch = 0; ch < BN / 64; ++ch) {
                    const int out_col = c.n_index * (BN / 2) + ch * 32;
                    if (out_col >= half_n) break;
                    ptx::tmem_ld_32x32(acc + ch * 32, r0);
                    ptx::tmem_ld_32x32(acc + BN / 2 + ch * 32, r1);
                    ptx::tmem_ld_wait();
                    if (row_ok) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float g = __uint_as_float(r0[i]), u = __uint_as_float(r1[i]);
                            v[i] = g / (1.0F + __expf(-g)) * u;
                        }
                        store_chunk(p.out, p.out_f32, static_cast<size_t>(row) * half_n + out_col, v,
                                    min(32, half_n - out_col));
                    }
                }
            } else {
                for (int ch = 0; ch < BN / 32; ++ch) {
                    const int col = n0 + ch * 32;
                    if (col >= p.n) break;
                    ptx::tmem_ld_32x32(acc + ch * 32, r0);
                    ptx::tmem_ld_wait();
                    if (!row_ok) continue;
                    const int valid = min(32, p.n - col);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r0[i]);
                    if (p.epilogue == SFB_EPI_ROPE_SPLIT) {
                        const int hidden = p.q_heads * p.head_dim, kvw = p.kv_heads * p.head_dim;
                        const int b = row / p.seq, t = row - b * p.seq;
                        bf16* dst;
                        int heads, local;
                        bool rotate = true;
                        if (col < hidden) { dst = p.q; heads = p.q_heads; local = col; }
                        else if (col < hidden + kvw) { dst = p.key; heads = p.kv_heads; local = col - hidden; }
                        else { dst = p.value; heads = p.kv_heads; local = col - hidden - kvw; rotate = false; }
                        const int head = local / p.head_dim, d0 = local - head * p.head_dim;
                        if (rotate) {
                            const float* cs = p.rope_cos + static_cast<size_t>(t) * (p.head_dim / 2) + d0 / 2;
                            const float* sn = p.rope_sin + static_cast<size_t>(t) * (p.head_dim / 2) + d0 / 2;
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float4 c4 = reinterpret_cast<const float4*>(cs)[i];
                                const float4 s4 = reinterpret_cast<const float4*>(sn)[i];
                                const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const float e = v[8 * i + 2 * j], o = v[8 * i + 2 * j + 1];
                                    v[8 * i + 2 * j] = e * cc[j] - o * ss[j];
                                    v[8 * i + 2 * j + 1] = e * ss[j] + o * cc[j];
                                }
                            }
                        }
                        const size_t o = ((static_cast<size_t>(b) * heads + head) * p.seq + t) * p.head_dim + d0;
                        store_chunk(dst, 0, o, v, 32);
                    } else {
                        const size_t index = static_cast<size_t>(row) * p.n + col;
                        if (p.epilogue == SFB_EPI_RESIDUAL) {
                            float res[32];
                            load_bf16_chunk(p.residual + index, res, valid);
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] += res[i];
                        }
                        store_chunk(p.out, p.out_f32, index, v, valid);
                    }
                }
            }
            ptx::tc_fence_before();
            ptx::mbar_arrive(ptx::smem_u32(&tmem_empty[buf]));
        }
    }

    __syncwarp();
    ptx::tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // A wait gave up: let copies that may still be in flight land before the shared
        // memory and tensor memory of this CTA are released.
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, T::kTmemCols);
    }
}

__global__ void build_tile_table_kernel(const int* __restrict__ offsets, int groups, int* __restrict__ table,
                                        int capacity) {
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    int count = 0;
    for (int g = 0; g < groups; ++g) {
        const int begin = offsets[g], end = offsets[g + 1];
        for (int r = begin; r < end; r += BM) {
            if (count < capacity) {
                int* e = table + 4 + 4 * count;
                e[0] = r;
                e[1] = min(r + BM, end);
                e[2] = g;
                e[3] = 0;
                ++count;
            }
        }
    }
    table[0] = count;
}

template <int BN>
sfb_status launch(const sfb_gemm_args& g, cudaStream_t stream) {
    using T = Tile<BN>;
    static bool configured = false;
    if (!configured) {
        SFB_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      T::kSmemBytes));
        configured = true;
    }
    const int groups = g.group_offsets ? g.groups : 1;
    CUtensorMap map_a, map_b;
    if (!encode_tensor_map_bf16_2d(&map_a, g.a, static_cast<uint64_t>(g.m), static_cast<uint64_t>(g.k), BM, BK))
        return SFB_CUDA_ERROR;
    if (!encode_tensor_map_bf16_2d(&map_b, g.bt, static_cast<uint64_t>(groups) * g.n, static_cast<uint64_t>(g.k),
                                   BN, BK))
        return SFB_CUDA_ERROR;
    TcParams p{};
    p.out = g.out;
    p.m = g.m; p.n = g.n; p.k = g.k;
    p.epilogue = g.epilogue;
    p.out_f32 = g.out_f32;
    p.residual = static_cast<const bf16*>(g.residual);
    p.q = static_cast<bf16*>(g.q);
    p.key = static_cast<bf16*>(g.key);
    p.value = static_cast<bf16*>(g.value);
    p.rope_cos = g.rope_cos;
    p.rope_sin = g.rope_sin;
    p.seq = g.seq; p.q_heads = g.q_heads; p.kv_heads = g.kv_heads; p.head_dim = g.head_dim;
    p.n_tiles = ceil_div(g.n, BN);
    p.status = device_status_word();
    int max_m_tiles;
    if (g.group_offsets) {
        SFB_REQUIRE(g.tile_table, "gemm: grouped tcgen05 mode needs tile_table scratch");
        max_m_tiles = g.m / BM + groups + 1;
        build_tile_table_kernel<<<1, 32, 0, stream>>>(g.group_offsets, groups, static_cast<int*>(g.tile_table),
                                                       max_m_tiles);
        SFB_TRY(check_launch("build_tile_table"));
        p.tile_table = static_cast<const int*>(g.tile_table);
        p.dense_m_tiles = 0;
    } else {
        max_m_tiles = ceil_div(g.m, BM);
        p.tile_table = nullptr;
        p.dense_m_tiles = max_m_tiles;
    }
    const long long tiles = static_cast<long long>(max_m_tiles) * p.n_tiles;
    const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
    gemm_tcgen05_kernel<BN><<<grid, kThreads, T::kSmemBytes, stream>>>(map_a, map_b, p);
    return check_launch("gemm_tcgen05");
}

int pick_bn(const sfb_gemm_args& g) {
    if (g.epilogue == SFB_EPI_SWIGLU) return 2 * g.swiglu_block;
    // Few rows (decode) or a narrow output: more, smaller tiles keep more SMs streaming weights.
    const long long wide_tiles = static_cast<long long>(ceil_div(g.m, BM)) * ceil_div(g.n, 256);
    return (g.n < 256 || wide_tiles < sm_count()) ? 128 : 256;
}

}  // namespace

bool gemm_bf16_tcgen05_supported(const sfb_gemm_args& g) {
    if (g.k % 8 != 0) return false;  // TMA row pitch must be a multiple of 16 bytes
    if ((reinterpret_cast<uintptr_t>(g.a) & 15) || (reinterpret_cast<uintptr_t>(g.bt) & 15)) return false;
    if (g.epilogue == SFB_EPI_SWIGLU && g.swiglu_block != 64 && g.swiglu_block != 128) return false;
    if (g.epilogue == SFB_EPI_ROPE_SPLIT && g.head_dim % 32 != 0) return false;
    return true;
}

sfb_status gemm_bf16_tcgen05(const sfb_gemm_args& g, cudaStream_t stream) {
    return pick_bn(g) == 256 ? launch<256>(g, stream) : launch<128>(g, stream);
}

}  // namespace sfb
