// bf16 GEMM on the 5th-generation tensor cores: out = epilogue(A[m,k] . Bt[n,k]^T).
//
// One persistent CTA per SM, 320 threads in three roles:
//   warp 0      TMA producer: streams 128x64 A tiles and BNx64 B tiles (128-byte swizzle)
//               through rings of shared-memory stages guarded by full/empty mbarriers;
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) four times per
//               K block into one of TWO accumulator buffers in tensor memory and commits the
//               stages back to the producer and the finished work item to the epilogue;
//   warps 2-9   epilogue: tcgen05.ld the accumulator (one row per thread, 32 columns at a
//               time; two warps share each 32-row quarter and alternate over the column
//               chunks), apply the fused epilogue and store to global memory, while the MMA
//               warp already works on the next item in the other buffer.
// Epilogues: plain store, + residual, SwiGLU over [gate | up] halves of the tile, and
// RoPE + scatter into head-major Q/K/V for the fused QKV projection.
// Grouped mode (MoE experts): a device-built tile table maps every M-tile to a row range
// of one expert; the weight slab of that expert is addressed through the row coordinate
// of the B tensor map, rows outside the range are masked in the epilogue.
//
// Many rows (prefill): a work item is one output tile; tiles are visited in bands of 16
// M-tiles so that one band's A rows stay in L2 while the CTAs sweep the N direction.
//
// One M-tile (decode): every weight byte is read once, the kernel is HBM-bound, and one SM
// can only keep a bounded number of HBM bytes in flight, so ALL SMs must stream for the whole
// kernel.  The (tile, K block) pairs are laid end to end and cut into one equal contiguous
// range per CTA.  A range that covers a whole tile runs the fused epilogue from tensor
// memory.  Ranges that cover part of a tile add their fp32 partial sums into a zeroed
// accumulator in global memory (reductions performed at L2) and count the K blocks they
// contributed; the CTA whose contribution completes the tile reads the sums back, runs the
// epilogue and restores the zeros.  No CTA ever waits for another.  In this mode the
// activation tiles (L2 hits) and the weight tiles (HBM) use separate rings, a shallow and a
// deep one, so that nearly all of shared memory holds HBM bytes in flight.
#include <algorithm>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace sfb {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GROUP_M = 16;
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr uint32_t kCodeProducer = 0x1, kCodeMma = 0x2, kCodeEpilogue = 0x4;

template <int BN, bool STREAM>
struct Tile {
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kStagesA = STREAM ? 6 : (BN == 256 ? 4 : 6);
    static constexpr int kStagesB = STREAM ? (192 * 1024 - kStagesA * kABytes) / kBBytes : kStagesA;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kBarrierBytes = 512;
    // per warp 32 rows x 32 fp32 columns, then per warp 32 row sums of squares
    static constexpr int kEpilogueStagingBytes = kEpilogueWarps * 32 * 32 * 4 + kEpilogueWarps * 32 * 4;
    static constexpr int kSmemBytes =
        kStagesA * kABytes + kStagesB * kBBytes + kEpilogueStagingBytes + kBarrierBytes + 1024;
    static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
    static_assert(8 * (2 * kStagesA + 2 * kStagesB + 4) + 16 <= kBarrierBytes, "barrier block too small");
};

struct TcParams {
    void* out;
    int m, n, k;
    int epilogue, out_f32;
    const bf16* residual;
    bf16 *q, *key, *value;
    const float *rope_cos, *rope_sin;
    int seq, q_heads, kv_heads, head_dim, rope_row_offset;
    const int* tile_table;  // grouped: [0] = number of M-tiles, entries from [4]
    int dense_m_tiles;
    int n_tiles;
    int b_tiled;            // weight stored as 64x64 blocks, 8 KB contiguous each
    // equal K-block ranges per CTA (one M-tile only): fp32 [n_tiles][BM][BN] sums + one counter per tile
    const float* col_scale;             // weight-only INT8: one factor per output column, applied before the epilogue
    bf16* peer_out[SFB_MAX_PEERS - 1];  // copies of the output in other GPUs' memory (fused all-reduce)
    int peer_count;
    bf16* scatter_out[SFB_MAX_PEERS];   // two-shot form: this rank's slot in the receive buffer of every row owner
    int scatter_rows;                   // rows per owner (0 = off)
    float* accum;
    int* tile_counters;
    int shared_tiles;       // trailing tiles whose K blocks are cut into equal ranges (0 = none)
    uint32_t* status;
    // RMSNorm folded into this GEMM: accumulator row r is multiplied by 1/sqrt(ss[r] / k + eps); ss[r] is a float, or
    // (row_ss_fixed) an unsigned 64-bit fixed-point sum with 24 fraction bits as ss_out leaves it
    const void* row_ss;
    int row_ss_fixed;
    float rms_eps;
    // per-row sums of squares of the stored bf16 outputs: every (warp, 128-column group) adds its share to the row's
    // 64-bit fixed-point sum with an integer atomic, so the total does not depend on the order of arrival
    unsigned long long* ss_out;
    // A arrives from other ranks while the kernel runs (all-gather by copy engines): rows [o * owner_rows, ...) are
    // complete once owner_flags[o] has reached owner_epoch; this rank's own rows (owner_self) are there from the start
    // and the tiles are visited starting with them (m_rotate M-tiles further on)
    const uint32_t* owner_flags;
    uint32_t owner_epoch;
    int owner_rows, owner_self, m_rotate;
    // zero-filled by this kernel after its dependency wait (the sums the NEXT kernels will add to)
    unsigned long long* clear;
    unsigned clear_pieces;  // 8-byte words
    // RoPE epilogue of a decode step: the paged cache that receives K and V
    bf16 *kv_k_pool, *kv_v_pool;
    const int* kv_table;
    int kv_position, kv_block_tokens, kv_max_blocks, kv_num_blocks;
};

struct TileCoord {
    int row_start, row_end, group, n_index;
};

// One work item: K blocks [kb0, kb1) of one output tile.
struct Segment {
    int tile, kb0, kb1;
};

// The sequence of work items of one CTA.  Every role walks its own copy.
// Whole tiles go round-robin.  With sum scratch (one M-tile), the tiles left over after the
// last full round are not handed to a few CTAs: their (tile, K block) pairs are laid end to
// end and cut into one equal range per CTA.  A CTA works through its range first (the piece
// at its head, the piece at its tail, then any whole tiles inside it) and through its
// round-robin tiles afterwards, so that summing and completing shared tiles overlaps streaming.
struct Walk {
    long long unit, unit_end;  // this CTA's range of the left-over tiles' K blocks
    int first_shared;          // tiles [first_shared, total_tiles) are cut into ranges
    int tile, stride, k_blocks;
    int phase;                 // 0 = head piece, 1 = tail piece, 2 = whole tiles of the range, 3 = round-robin
    __device__ bool next(Segment& sg) {
        if (phase == 0) {
            phase = 1;
            const int first = static_cast<int>(unit % k_blocks);
            if (first != 0 && unit < unit_end) {
                sg.tile = first_shared + static_cast<int>(unit / k_blocks);
                sg.kb0 = first;
                sg.kb1 = static_cast<int>(min(static_cast<long long>(k_blocks), first + (unit_end - unit)));
                unit += sg.kb1 - sg.kb0;
                return true;
            }
        }
        if (phase == 1) {  // `unit` is on a tile boundary or the range is used up
            phase = 2;
            const int last = static_cast<int>(unit_end % k_blocks);
            if (last != 0 && unit < unit_end) {
                sg.tile = first_shared + static_cast<int>(unit_end / k_blocks);
                sg.kb0 = 0;
                sg.kb1 = last;
                unit_end -= last;
                return true;
            }
        }
        sg.kb0 = 0;
        sg.kb1 = k_blocks;
        if (phase == 2) {
            if (unit < unit_end) {
                sg.tile = first_shared + static_cast<int>(unit / k_blocks);
                unit += k_blocks;
                return true;
            }
            phase = 3;
        }
        if (tile >= first_shared) return false;
        sg.tile = tile;
        tile += stride;
        return true;
    }
};

__device__ __forceinline__ int load_m_tiles(const TcParams& p) {
    return p.tile_table ? p.tile_table[0] : p.dense_m_tiles;
}

__device__ __forceinline__ Walk make_walk(const TcParams& p, int m_tiles, int k_blocks) {
    Walk w;
    const int total_tiles = m_tiles * p.n_tiles;
    w.k_blocks = k_blocks;
    w.tile = blockIdx.x;
    w.stride = gridDim.x;
    w.first_shared = total_tiles - p.shared_tiles;
    const long long units = static_cast<long long>(p.shared_tiles) * k_blocks;
    w.unit = units * blockIdx.x / gridDim.x;
    w.unit_end = units * (blockIdx.x + 1) / gridDim.x;
    w.phase = p.shared_tiles > 0 ? 0 : 3;
    return w;
}

template <bool ROTATE = false>
__device__ __forceinline__ TileCoord tile_coord(const TcParams& p, int tile, int m_tiles) {
    const int band_tiles = GROUP_M * p.n_tiles;
    const int band = tile / band_tiles;
    const int first_m = band * GROUP_M;
    const int band_m = min(GROUP_M, m_tiles - first_m);
    const int local = tile - band * band_tiles;
    int m_index = first_m + local % band_m;
    if constexpr (ROTATE) {
        if (p.m_rotate > 0) m_index = (m_index + p.m_rotate) % m_tiles;
    }
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

// ---- epilogue --------------------------------------------------------------------------
// A thread of an epilogue warp reads one accumulator ROW from tensor memory.  Storing rows
// straight from there would make every store instruction touch 32 different lines, which
// takes microseconds per tile.  So each warp first parks 32 columns of its 32 rows in shared
// memory (fp32, 16-byte pieces XOR-swizzled by row so that both phases are conflict-free) and
// then walks them with 4 adjacent lanes per row: every lane owns 8 adjacent columns, applies
// the rest of the epilogue and issues 16-byte loads and stores that coalesce per row.
// SiLU(gate) * up is computed before staging, where a thread has 32 independent values.
constexpr int kStageFloatsPerWarp = 32 * 32;

// phase 1: lane = row, 32 values = staged columns [0, 32)
__device__ __forceinline__ void stage_write(float* stage, int lane, const uint32_t (&r)[32]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int piece = j ^ (lane & 7);
        *reinterpret_cast<uint4*>(stage + lane * 32 + piece * 4) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    }
}
// phase 2: 8 staged values of row `r` starting at staged column `first` (a multiple of 8)
__device__ __forceinline__ void stage_read8(const float* stage, int r, int first, float (&f)[8]) {
    const int p0 = (first >> 2) ^ (r & 7), p1 = ((first >> 2) + 1) ^ (r & 7);
    const float4 lo = *reinterpret_cast<const float4*>(stage + r * 32 + p0 * 4);
    const float4 hi = *reinterpret_cast<const float4*>(stage + r * 32 + p1 * 4);
    f[0] = lo.x; f[1] = lo.y; f[2] = lo.z; f[3] = lo.w;
    f[4] = hi.x; f[5] = hi.y; f[6] = hi.z; f[7] = hi.w;
}

// 8 adjacent outputs: one 16-byte (bf16) or two 16-byte (fp32) stores when complete and aligned
__device__ __forceinline__ void store8(void* out, int out_f32, size_t index, const float (&f)[8], int valid) {
    if (out_f32) {
        float* dst = static_cast<float*>(out) + index;
        if (valid >= 8 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
            reinterpret_cast<float4*>(dst)[0] = make_float4(f[0], f[1], f[2], f[3]);
            reinterpret_cast<float4*>(dst)[1] = make_float4(f[4], f[5], f[6], f[7]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i < valid) dst[i] = f[i];
        }
    } else {
        bf16* dst = static_cast<bf16*>(out) + index;
        if (valid >= 8 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
            uint4 packed;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
            *reinterpret_cast<uint4*>(dst) = packed;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i < valid) dst[i] = from_float<bf16>(f[i]);
        }
    }
}

__device__ __forceinline__ void add_bf16x8(const bf16* src, float (&f)[8], int valid) {
    if (valid >= 8 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        const uint4 packed = *reinterpret_cast<const uint4*>(src);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 x = __bfloat1622float2(h[j]);
            f[2 * j] += x.x;
            f[2 * j + 1] += x.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < valid) f[i] += to_float(src[i]);
    }
}

// Sum of squares of up to 8 values as they read back after rounding to bf16.
__device__ __forceinline__ float sumsq_bf16x8(const float (&f)[8], int valid) {
    float ss = 0.0F;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float v = __bfloat162float(__float2bfloat16_rn(f[i]));
        if (i < valid) ss = fmaf(v, v, ss);
    }
    return ss;
}

// Decode step: the new token's key / value (8 elements of one head) also goes to slot kv_position + t of sequence b
// in the paged cache.  A position past the table or a block outside the pool is skipped and flagged, never written.
// Kept out of line: it runs for a handful of rows per step and must not cost the common epilogue its registers.
__device__ __noinline__ void kv_append8(const TcParams& p, bf16* pool, int b, int t, int head, int d0, const float (&f)[8]) {
    const int pos = p.kv_position + t, block = pos / p.kv_block_tokens;
    int page = -1;
    if (block < p.kv_max_blocks) page = p.kv_table[static_cast<size_t>(b) * p.kv_max_blocks + block];
    if (page >= 0 && page < p.kv_num_blocks)
        store8(pool, 0, ((static_cast<size_t>(page) * p.kv_heads + head) * p.kv_block_tokens + pos % p.kv_block_tokens) *
                                p.head_dim + d0, f, 8);
    else
        atomicOr(p.status, 0x200u);
}

// Epilogue of output columns [col, col + 8) of `row` (not SwiGLU); col is a multiple of 8.  Returns the sum of
// squares of the stored values when the kernel collects them for the RMSNorm of the next GEMM (else 0).
// EXTRA = the launch uses one of the rarer epilogue features (paged K/V append, scatter to row owners, sums of squares):
// kernels without them are compiled without that code, which the hot prefill epilogue would otherwise pay for.
template <bool EXTRA>
__device__ __forceinline__ float emit8(const TcParams& p, int row, int col, float (&f)[8], bool residual_added = false) {
    if (col >= p.n) return 0.0F;
    if (p.epilogue == SFB_EPI_ROPE_SPLIT) {  // head_dim % 32 == 0: the 8 columns lie in one head
        const int hidden = p.q_heads * p.head_dim, kvw = p.kv_heads * p.head_dim;
        const int token = row + p.rope_row_offset;
        const int b = token / p.seq, t = token - b * p.seq;
        bf16* dst;
        bf16* pool = nullptr;
        int heads, local;
        bool rotate = true;
        if (col < hidden) { dst = p.q; heads = p.q_heads; local = col; }
        else if (col < hidden + kvw) { dst = p.key; heads = p.kv_heads; local = col - hidden; pool = p.kv_k_pool; }
        else { dst = p.value; heads = p.kv_heads; local = col - hidden - kvw; rotate = false; pool = p.kv_v_pool; }
        const int head = local / p.head_dim, d0 = local - head * p.head_dim;
        if (rotate) {
            const size_t at = static_cast<size_t>(t) * (p.head_dim / 2) + d0 / 2;
            const float4 c4 = *reinterpret_cast<const float4*>(p.rope_cos + at);
            const float4 s4 = *reinterpret_cast<const float4*>(p.rope_sin + at);
            const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float e = f[2 * j], o = f[2 * j + 1];
                f[2 * j] = e * cc[j] - o * ss[j];
                f[2 * j + 1] = e * ss[j] + o * cc[j];
            }
        }
        store8(dst, 0, ((static_cast<size_t>(b) * heads + head) * p.seq + t) * p.head_dim + d0, f, 8);
        if constexpr (EXTRA) {
            if (pool) kv_append8(p, pool, b, t, head, d0, f);
        }
        return 0.0F;
    }
    const size_t index = static_cast<size_t>(row) * p.n + col;
    const int valid = p.n - col;
    if (p.epilogue == SFB_EPI_RESIDUAL && !residual_added) add_bf16x8(p.residual + index, f, valid);
    if constexpr (EXTRA) {
        if (p.scatter_rows > 0) {  // reduce-scatter: the piece goes to the owner of its row only (a peer store unless that is this rank)
            const int owner = row / p.scatter_rows;
            store8(p.scatter_out[owner], 0, static_cast<size_t>(row - owner * p.scatter_rows) * p.n + col, f, valid);
            return 0.0F;
        }
    }
    store8(p.out, p.out_f32, index, f, valid);
    for (int i = 0; i < p.peer_count; ++i) store8(p.peer_out[i], 0, index, f, valid);  // peer stores over NVLink
    if constexpr (EXTRA) return p.ss_out ? sumsq_bf16x8(f, valid) : 0.0F;
    return 0.0F;
}

// phase 2 for one warp: the staged values are output columns [col0, col0 + 32) of rows
// [row0, row0 + 32); `plain` = they are final (SwiGLU) and only need storing into [m, width].
template <bool EXTRA>
__device__ __forceinline__ void emit_staged(const TcParams& p, const float* stage, int lane, int row0, int row_end,
                                            int col0, bool plain, int width, float* row_sums) {
    // The residual rows come from DRAM: all four loads of this lane go out before the first is used
    // (one at a time, they made the epilogue of a tile as long as its main loop).
    const bool prefetch = !plain && p.epilogue == SFB_EPI_RESIDUAL && (p.n & 7) == 0 &&
                          (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0;
    uint4 residual[4];
    if (prefetch) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = row0 + i * 8 + (lane >> 2), col = col0 + (lane & 3) * 8;
            residual[i] = (row < row_end && col < width)
                ? __ldg(reinterpret_cast<const uint4*>(p.residual + static_cast<size_t>(row) * p.n + col))
                : make_uint4(0u, 0u, 0u, 0u);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = i * 8 + (lane >> 2), first = (lane & 3) * 8;
        const int row = row0 + r, col = col0 + first;
        const bool live = row < row_end && col < width;
        if (!live && (!EXTRA || !row_sums)) continue;
        float f[8];
        stage_read8(stage, r, first, f);
        if (prefetch) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&residual[i]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 x = __bfloat1622float2(h[j]);
                f[2 * j] += x.x;
                f[2 * j + 1] += x.y;
            }
        }
        if (plain) {
            store8(p.out, p.out_f32, static_cast<size_t>(row) * width + col, f, width - col);
        } else {
            float v = live ? emit8<EXTRA>(p, row, col, f, prefetch) : 0.0F;
            if constexpr (EXTRA) {
                if (row_sums) {  // the four lanes of a row add up; one of them keeps the row's running sum in shared memory
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    if ((lane & 3) == 0) row_sums[r] += v;
                }
            }
        }
    }
}

constexpr float kSumFixedScale = 16777216.0F;  // 2^24

// Sums of squares collected by one warp over the chunks of one 128-column group: lane r holds row r's sum in
// shared memory; it is added to the row's fixed-point total and cleared.
__device__ __forceinline__ void flush_row_ss(const TcParams& p, float* row_sums, int lane, int row0, int row_end) {
    __syncwarp();
    const float v = row_sums[lane];
    row_sums[lane] = 0.0F;
    if (row0 + lane < row_end) atomicAdd(p.ss_out + row0 + lane, __float2ull_rn(v * kSumFixedScale));
    __syncwarp();
}

// Epilogue of one work item for an epilogue thread: `acc` is the tensor-memory address of the
// accumulator (lane quarter and buffer included), `tmem_empty_bar` the barrier that hands it back.
template <int BN, bool SCALED, bool EXTRA>
__device__ __forceinline__ void epilogue_segment(const TcParams& p, const Segment& sg, const TileCoord& c, int k_blocks,
                                                 uint32_t acc, uint32_t tmem_empty_bar, float* stage,
                                                 volatile uint32_t* last_flag, int quarter, int pass, int lane,
                                                 bool leader, float row_inv, float* row_sums_area) {
    constexpr uint32_t kEpilogueThreads = 32 * kEpilogueWarps;
    const int row_in_tile = quarter * 32 + lane;
    const int row0 = c.row_start + quarter * 32;
    const bool row_ok = row0 + lane < c.row_end;
    const bool swiglu = p.epilogue == SFB_EPI_SWIGLU;
    // An output chunk is 32 columns: one 32-column group of the accumulator, or for SwiGLU
    // a gate group and its up group from the other half of the tile.
    const int chunks = swiglu ? BN / 64 : BN / 32;
    const int width = swiglu ? p.n / 2 : p.n;
    const int out0 = swiglu ? c.n_index * (BN / 2) : c.n_index * BN;
    const bool whole = sg.kb0 == 0 && sg.kb1 == k_blocks;
    uint32_t r0[32], r1[32];
    // Sums of a tile: [BN / 4 column groups][BM rows][4], so that a warp touches 512 contiguous bytes.
    float* sums = p.accum + static_cast<size_t>(sg.tile) * BM * BN + row_in_tile * 4;
    if (!whole) {
        // Part of a tile: add the partial sums, then find out whether they completed the tile.
#pragma unroll 1
        for (int g = pass; g < BN / 32; g += 2) {
            if (c.n_index * BN + g * 32 >= p.n) break;
            ptx::tmem_ld_32x32(acc + g * 32, r0);
            ptx::tmem_ld_wait();
            if (!row_ok) continue;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                ptx::red_add_f32x4(sums + (g * 8 + i) * (BM * 4), __uint_as_float(r0[4 * i]),
                                   __uint_as_float(r0[4 * i + 1]), __uint_as_float(r0[4 * i + 2]),
                                   __uint_as_float(r0[4 * i + 3]));
        }
        ptx::tc_fence_before();
        ptx::mbar_arrive(tmem_empty_bar);
        __threadfence();
        ptx::named_barrier(1, kEpilogueThreads);
        if (leader) {
            const int mine = sg.kb1 - sg.kb0;
            *last_flag = (atomicAdd(p.tile_counters + sg.tile, mine) + mine == k_blocks) ? 1u : 0u;
        }
        ptx::named_barrier(1, kEpilogueThreads);
        if (*last_flag == 0) return;
        // this CTA completed the tile: it reads the sums back (past L1), restores the zeros
        // and runs the epilogue
        __threadfence();
        if (leader) p.tile_counters[sg.tile] = 0;
    }
    // 32 accumulator columns starting at `group_col`, from tensor memory or from the sums
    auto fetch = [&](int group_col, uint32_t (&dst)[32]) {
        if (whole) {
            ptx::tmem_ld_32x32(acc + group_col, dst);
            return;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float4* src = reinterpret_cast<float4*>(sums + (group_col / 4 + i) * (BM * 4));
            float4 f = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
            if (row_ok) {
                f = __ldcg(src);
                __stcg(src, make_float4(0.0F, 0.0F, 0.0F, 0.0F));
            }
            dst[4 * i] = __float_as_uint(f.x); dst[4 * i + 1] = __float_as_uint(f.y);
            dst[4 * i + 2] = __float_as_uint(f.z); dst[4 * i + 3] = __float_as_uint(f.w);
        }
    };
    // A completed cut-up tile: the sums of this warp's second chunk are requested together with the first
    // (one L2 round trip on the kernel's critical path instead of two); r1 is free when there is no SwiGLU.
    const bool ahead = !whole && !swiglu && pass + 2 < chunks && out0 + (pass + 2) * 32 < width;
    if (ahead) {
        if (out0 + pass * 32 < width) fetch(pass * 32, r0);
        fetch((pass + 2) * 32, r1);
    }
    const bool collect = EXTRA && p.ss_out != nullptr && !swiglu;
    float* row_sums = collect ? row_sums_area : nullptr;
#pragma unroll 1
    for (int ch = pass; ch < chunks; ch += 2) {
        const int col0 = out0 + ch * 32;
        const bool live = col0 < width;
        if (live) {
            if (ahead && ch == pass + 2) {
#pragma unroll
                for (int i = 0; i < 32; ++i) r0[i] = r1[i];
            } else if (!(ahead && ch == pass)) {
                fetch(ch * 32, r0);
            }
            if (swiglu) fetch(BN / 2 + ch * 32, r1);
            if (whole) ptx::tmem_ld_wait();
        }
        if (whole && ch + 2 >= chunks) {  // this thread has read all it needs: hand the accumulator back
            ptx::tc_fence_before();
            ptx::mbar_arrive(tmem_empty_bar);
        }
        if (!live) continue;
        if constexpr (SCALED) {  // weight-only INT8: the sums are over integer weights, one factor per output column
            const float* scale0 = p.col_scale + c.n_index * BN + ch * 32;
            const float* scale1 = scale0 + BN / 2;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                r0[i] = __float_as_uint(__uint_as_float(r0[i]) * __ldg(scale0 + i));
                if (swiglu) r1[i] = __float_as_uint(__uint_as_float(r1[i]) * __ldg(scale1 + i));
            }
        }
        if (EXTRA && p.row_ss) {  // folded RMSNorm: the whole accumulator row carries the factor 1/rms(row of A)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                r0[i] = __float_as_uint(__uint_as_float(r0[i]) * row_inv);
                if (swiglu) r1[i] = __float_as_uint(__uint_as_float(r1[i]) * row_inv);
            }
        }
        if (swiglu) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float gate = __uint_as_float(r0[i]);
                r0[i] = __float_as_uint(__fdividef(gate, 1.0F + __expf(-gate)) * __uint_as_float(r1[i]));
            }
        }
        stage_write(stage, lane, r0);
        __syncwarp();
        emit_staged<EXTRA>(p, stage, lane, row0, c.row_end, col0, swiglu, width, row_sums);
        __syncwarp();
        // the chunks of this warp advance by 64 columns: the last one inside a 128-column group closes its slot
        if (collect && ((col0 + 64) / 128 != col0 / 128 || ch + 2 >= chunks || col0 + 64 >= width))
            flush_row_ss(p, row_sums, lane, row0, c.row_end);
    }
}

// 1 / rms of row `row` of A from the sum of squares its producer left (see TcParams::row_ss).
__device__ __forceinline__ float folded_row_inv(const TcParams& p, int row, bool row_ok) {
    if (!p.row_ss || !row_ok) return 1.0F;
    const float ss = p.row_ss_fixed
        ? static_cast<float>(__ldcg(static_cast<const unsigned long long*>(p.row_ss) + row)) * (1.0F / kSumFixedScale)
        : __ldcg(static_cast<const float*>(p.row_ss) + row);
    return 1.0F / sqrtf(ss / static_cast<float>(p.k) + p.rms_eps);
}

template <int BN, bool STREAM, bool EXTRA>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const __grid_constant__ TcParams p) {
    using T = Tile<BN, STREAM>;
    constexpr int SA = T::kStagesA, SB = T::kStagesB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + SA * T::kABytes;
    float* staging = reinterpret_cast<float*>(smem_b + SB * T::kBBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_b + SB * T::kBBytes + T::kEpilogueStagingBytes);
    // shared rings (STREAM = false): full_a/empty_a are unused, full_b/empty_b guard whole stages
    uint64_t* full_b = bars;
    uint64_t* empty_b = full_b + SB;
    uint64_t* full_a = empty_b + SB;
    uint64_t* empty_a = full_a + SA;
    uint64_t* tmem_full = empty_a + SA;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* last_flag = tmem_slot + 2;  // epilogue warps: this CTA completed the tile

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SB; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_b[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_b[s]), 1);
        }
        for (int s = 0; s < SA; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_a[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_a[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&tmem_full[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&tmem_empty[b]), 32 * kEpilogueWarps);
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
    grid_dependents_may_launch();
    // Weights do not depend on the kernel before this one: in a dense GEMM the producer fetches them
    // first and only then waits for that kernel; every other role waits right away.
    const bool early_weights = p.tile_table == nullptr;
    if (!(warp == 0 && lane == 0 && early_weights)) grid_dependency_wait();

    const int m_tiles = load_m_tiles(p);
    const int k_blocks = (p.k + BK - 1) / BK;
    Walk walk = make_walk(p, m_tiles, k_blocks);

    // weight tile of K block `kb` for output columns [n_index * BN, +BN) of slab `group`
    auto load_b = [&](uint8_t* dst, uint32_t bar, int kb, const TileCoord& c) {
        if (p.b_tiled) {
            // rows of the map are the 64-row blocks laid end to end, 128 bytes each; a block past
            // the last weight row lies outside the map and reads as zeros
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) {
                const int block = (c.n_index * (BN / 64) + j) * k_blocks + kb;
                ptx::tma_load_2d(ptx::smem_u32(dst + j * 8192), &tma_b, bar, 0, block * 64);
            }
        } else {
            ptx::tma_load_2d(ptx::smem_u32(dst), &tma_b, bar, kb * BK, c.group * p.n + c.n_index * BN);
        }
    };

    if (warp == 0) {
        if (lane == 0) {
            if constexpr (!STREAM) {
                Segment sg;
                uint32_t it = 0;
                bool ok = true;
                // the first ring-full of weight tiles goes out before the wait for the previous kernel
                uint32_t early = 0;
                if (early_weights) {
                    Walk ahead = walk;
                    Segment first;
                    if (ahead.next(first)) {
                        const TileCoord c = tile_coord<EXTRA>(p, first.tile, m_tiles);
                        for (int kb = first.kb0; kb < first.kb1 && early < static_cast<uint32_t>(SB); ++kb, ++early) {
                            const uint32_t full = ptx::smem_u32(&full_b[early]);
                            ptx::mbar_expect_tx(full, T::kStageBytes);
                            load_b(smem_b + early * T::kBBytes, full, kb, c);
                        }
                    }
                    grid_dependency_wait();
                }
                uint32_t arrived = 0;  // owners whose rows this CTA has seen complete
                while (ok && walk.next(sg)) {
                    const TileCoord c = tile_coord<EXTRA>(p, sg.tile, m_tiles);
                    if constexpr (EXTRA) {
                        if (p.owner_flags) {
                            const int owner = c.row_start / p.owner_rows;
                            if (owner != p.owner_self && !((arrived >> owner) & 1u)) {
                                const long long start = clock64();
                                uint32_t spins = 0;
                                while (static_cast<int>(ptx::load_acquire_sys_u32(p.owner_flags + owner) - p.owner_epoch) < 0) {
                                    if ((++spins & 0xFFu) == 0 && (*abort_flag || clock64() - start > 2 * ptx::kWaitCycles)) {
                                        *abort_flag = 1;
                                        atomicOr(p.status, 0x100u);
                                        ok = false;
                                        break;
                                    }
                                }
                                if (!ok) break;
                                arrived |= 1u << owner;
                            }
                        }
                    }
                    for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
                        const uint32_t s = it % SB, ph = (it / SB) & 1;
                        const uint32_t full = ptx::smem_u32(&full_b[s]);
                        if (it >= early) {
                            if (!ptx::mbar_wait(ptx::smem_u32(&empty_b[s]), ph ^ 1, abort_flag, p.status, kCodeProducer)) {
                                ok = false;
                                break;
                            }
                            ptx::mbar_expect_tx(full, T::kStageBytes);
                            load_b(smem_b + s * T::kBBytes, full, kb, c);
                        }
                        ptx::tma_load_2d(ptx::smem_u32(smem_a + s * T::kABytes), &tma_a, full, kb * BK, c.row_start);
                    }
                }
            } else {
                // Two cursors over the same sequence; whichever ring has a free stage gets its next load.
                struct Cursor {
                    Walk walk;
                    Segment sg;
                    TileCoord c;
                    int kb;
                    uint32_t it;
                    bool live;
                };
                auto open = [&](Cursor& cu) {
                    cu.live = cu.walk.next(cu.sg);
                    if (cu.live) {
                        cu.c = tile_coord<EXTRA>(p, cu.sg.tile, m_tiles);
                        cu.kb = cu.sg.kb0;
                    }
                };
                auto advance = [&](Cursor& cu) {
                    ++cu.it;
                    if (++cu.kb == cu.sg.kb1) open(cu);
                };
                Cursor ca{walk, {}, {}, 0, 0, false}, cb{walk, {}, {}, 0, 0, false};
                open(ca);
                open(cb);
                // fill the weight ring before waiting for the previous kernel (the ring is empty: no waits)
                while (cb.live && cb.it < static_cast<uint32_t>(SB)) {
                    const uint32_t full = ptx::smem_u32(&full_b[cb.it]);
                    ptx::mbar_expect_tx(full, T::kBBytes);
                    load_b(smem_b + cb.it * T::kBBytes, full, cb.kb, cb.c);
                    advance(cb);
                }
                grid_dependency_wait();
                long long stall_start = 0;
                uint32_t idle = 0;
                while (ca.live || cb.live) {
                    bool progressed = false;
                    if (cb.live) {
                        const uint32_t s = cb.it % SB, ph = (cb.it / SB) & 1;
                        if (ptx::mbar_try_wait(ptx::smem_u32(&empty_b[s]), ph ^ 1)) {
                            const uint32_t full = ptx::smem_u32(&full_b[s]);
                            ptx::mbar_expect_tx(full, T::kBBytes);
                            load_b(smem_b + s * T::kBBytes, full, cb.kb, cb.c);
                            advance(cb);
                            progressed = true;
                        }
                    }
                    if (ca.live) {
                        const uint32_t s = ca.it % SA, ph = (ca.it / SA) & 1;
                        if (ptx::mbar_try_wait(ptx::smem_u32(&empty_a[s]), ph ^ 1)) {
                            const uint32_t full = ptx::smem_u32(&full_a[s]);
                            ptx::mbar_expect_tx(full, T::kABytes);
                            ptx::tma_load_2d(ptx::smem_u32(smem_a + s * T::kABytes), &tma_a, full, ca.kb * BK,
                                             ca.c.row_start);
                            advance(ca);
                            progressed = true;
                        }
                    }
                    if (progressed) {
                        idle = 0;
                    } else if (idle++ == 0) {
                        stall_start = clock64();
                    } else if ((idle & 0x3FFu) == 0) {  // bounded like every other wait
                        if (*abort_flag) break;
                        if (clock64() - stall_start > ptx::kWaitCycles) {
                            *abort_flag = 1;
                            atomicOr(p.status, kCodeProducer);
                            break;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16(BM, BN);
            uint32_t it = 0, count = 0;
            bool ok = true;
            Segment sg;
            for (; ok && walk.next(sg); ++count) {
                const uint32_t buf = count & 1, tph = (count >> 1) & 1;
                if (!ptx::mbar_wait(ptx::smem_u32(&tmem_empty[buf]), tph ^ 1, abort_flag, p.status, kCodeMma)) break;
                ptx::tc_fence_after();
                const uint32_t acc = tmem_base + buf * BN;
                for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
                    const uint32_t sb = it % SB, phb = (it / SB) & 1;
                    const uint32_t sa = STREAM ? it % SA : sb, pha = (it / SA) & 1;
                    if (!ptx::mbar_wait(ptx::smem_u32(&full_b[sb]), phb, abort_flag, p.status, kCodeMma)) {
                        ok = false;
                        break;
                    }
                    if constexpr (STREAM) {
                        if (!ptx::mbar_wait(ptx::smem_u32(&full_a[sa]), pha, abort_flag, p.status, kCodeMma)) {
                            ok = false;
                            break;
                        }
                    }
                    ptx::tc_fence_after();
                    const uint64_t da = ptx::umma_desc_k_sw128(ptx::smem_u32(smem_a + sa * T::kABytes));
                    const uint64_t db = ptx::umma_desc_k_sw128(ptx::smem_u32(smem_b + sb * T::kBBytes));
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk)
                        ptx::umma_bf16(acc, da + 2 * kk, db + 2 * kk, idesc, (kb > sg.kb0) || kk != 0);
                    ptx::umma_commit(ptx::smem_u32(&empty_b[sb]));
                    if constexpr (STREAM) ptx::umma_commit(ptx::smem_u32(&empty_a[sa]));
                }
                if (ok) ptx::umma_commit(ptx::smem_u32(&tmem_full[buf]));
            }
        }
    } else {
        const int quarter = warp & 3;            // tensor-memory lanes this warp may read
        const int pass = (warp - 2) >> 2;        // the two warps of a quarter alternate over the chunks
        const bool leader = threadIdx.x == 64;  // first epilogue thread
        float* stage = staging + (warp - 2) * kStageFloatsPerWarp;
        staging[kEpilogueWarps * kStageFloatsPerWarp + (warp - 2) * 32 + lane] = 0.0F;  // this warp's row sums of squares
        __syncwarp();
        if constexpr (EXTRA) {
            // nothing that ran before this kernel still reads `clear`, nothing before the next kernel writes it
            for (unsigned i = blockIdx.x * (32 * kEpilogueWarps) + (threadIdx.x - 64); i < p.clear_pieces;
                 i += gridDim.x * (32 * kEpilogueWarps))
                p.clear[i] = 0ull;
        }
        uint32_t count = 0;
        Segment sg;
        for (; walk.next(sg); ++count) {
            const TileCoord c = tile_coord<EXTRA>(p, sg.tile, m_tiles);
            const uint32_t buf = count & 1, tph = (count >> 1) & 1;
            // read while the tile's main loop is still running
            float row_inv = EXTRA && !p.owner_flags
                ? folded_row_inv(p, c.row_start + quarter * 32 + lane, c.row_start + quarter * 32 + lane < c.row_end) : 1.0F;
            bool go = ptx::mbar_wait(ptx::smem_u32(&tmem_full[buf]), tph, abort_flag, p.status, kCodeEpilogue);
            if constexpr (EXTRA) {  // rows (and their sums of squares) that arrive during the kernel are complete once the tile's
                                    // products exist: the producer saw the owner's flag before it loaded them
                if (p.owner_flags) row_inv = folded_row_inv(p, c.row_start + quarter * 32 + lane, c.row_start + quarter * 32 + lane < c.row_end);
            }
            // With cut-up tiles the epilogue threads meet at barriers that have no time limit, so they must all
            // take the same decision here: one thread that saw the abort flag takes the whole group out.
            if (p.shared_tiles > 0) go = ptx::named_barrier_all(2, 32 * kEpilogueWarps, go);
            if (!go) break;
            ptx::tc_fence_after();
            const uint32_t acc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            epilogue_segment<BN, false, EXTRA>(p, sg, c, k_blocks, acc, ptx::smem_u32(&tmem_empty[buf]), stage, last_flag, quarter, pass,
                                 lane, leader, row_inv, staging + kEpilogueWarps * kStageFloatsPerWarp + (warp - 2) * 32);
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

// ---- weight-only INT8, one M-tile (decode) -----------------------------------------------------------
// The same work split and epilogue as the streaming bf16 kernel above, with half the weight bytes:
// the weight arrives as int8 in 64x64 blocks (4 KB each) through a ring of TMA stages; the eight
// epilogue warps turn each 128 x 64 int8 tile into the bf16, 128-byte-swizzled tile the MMA reads
// (exact: |q| <= 127) while the copies of the following tiles are in flight, and run the epilogue
// of a work item after its last tile; the per-column scale is applied to the fp32 sums first.
struct W8 {
    static constexpr int BN = 128;
    static constexpr int kABytes = BM * BK * 2;   // activations, bf16
    static constexpr int kQBytes = BN * BK;       // weights, int8
    static constexpr int kCBytes = BN * BK * 2;   // converted weights, bf16
    static constexpr int SA = 4, SQ = 10, SC = 3;
    static constexpr int kStagingBytes = kEpilogueWarps * 32 * 32 * 4 + kEpilogueWarps * 32 * 4;
    static constexpr int kBarrierBytes = 512;
    static constexpr int kSmemBytes = SA * kABytes + SQ * kQBytes + SC * kCBytes + kStagingBytes + kBarrierBytes + 1024;
    static constexpr int kTmemCols = 2 * BN;
    static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
    static_assert(8 * (2 * SA + 2 * SQ + 2 * SC + 4) + 16 <= kBarrierBytes, "barrier block too small");
};

__global__ void __launch_bounds__(kThreads, 1)
gemm_w8_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_q,
                       const __grid_constant__ TcParams p) {
    constexpr int BN = W8::BN, SA = W8::SA, SQ = W8::SQ, SC = W8::SC;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_c = smem_a + SA * W8::kABytes;
    uint8_t* smem_q = smem_c + SC * W8::kCBytes;
    float* staging = reinterpret_cast<float*>(smem_q + SQ * W8::kQBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(staging) + W8::kStagingBytes);
    uint64_t* full_a = bars;
    uint64_t* empty_a = full_a + SA;
    uint64_t* full_q = empty_a + SA;    // int8 tile landed (TMA bytes)
    uint64_t* empty_q = full_q + SQ;    // all 256 converting threads have read it
    uint64_t* full_c = empty_q + SQ;    // all 256 converting threads have written the bf16 tile
    uint64_t* empty_c = full_c + SC;    // the MMAs that read it have completed
    uint64_t* tmem_full = empty_c + SC;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* last_flag = tmem_slot + 2;
    constexpr uint32_t kConverters = kEpilogueWarps / 2;  // arrivals per tile: one per warp of the group of four that converts it

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < SA; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_a[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_a[s]), 1);
        }
        for (int s = 0; s < SQ; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_q[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_q[s]), kConverters);
        }
        for (int s = 0; s < SC; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_c[s]), kConverters);
            ptx::mbar_init(ptx::smem_u32(&empty_c[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&tmem_full[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&tmem_empty[b]), 32 * kEpilogueWarps);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
        ptx::prefetch_tensormap(&tma_a);
        ptx::prefetch_tensormap(&tma_q);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), W8::kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    grid_dependents_may_launch();
    if (!(warp == 0 && lane == 0)) grid_dependency_wait();

    const int m_tiles = 1;
    const int k_blocks = (p.k + BK - 1) / BK;
    Walk walk = make_walk(p, m_tiles, k_blocks);

    // int8 tile of K block `kb` for output columns [n_index * 128, +128): two 64-row blocks of 4 KB
    auto load_q = [&](uint8_t* dst, uint32_t bar, int kb, int n_index) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int block = (n_index * 2 + j) * k_blocks + kb;
            ptx::tma_load_2d(ptx::smem_u32(dst + j * 4096), &tma_q, bar, 0, block * 64);
        }
    };

    if (warp == 0) {
        if (lane == 0) {
            struct Cursor {
                Walk walk;
                Segment sg;
                TileCoord c;
                int kb;
                uint32_t it;
                bool live;
            };
            auto open = [&](Cursor& cu) {
                cu.live = cu.walk.next(cu.sg);
                if (cu.live) {
                    cu.c = tile_coord(p, cu.sg.tile, m_tiles);
                    cu.kb = cu.sg.kb0;
                }
            };
            auto advance = [&](Cursor& cu) {
                ++cu.it;
                if (++cu.kb == cu.sg.kb1) open(cu);
            };
            Cursor ca{walk, {}, {}, 0, 0, false}, cq{walk, {}, {}, 0, 0, false};
            open(ca);
            open(cq);
            while (cq.live && cq.it < static_cast<uint32_t>(SQ)) {  // weights do not depend on the kernel before
                const uint32_t full = ptx::smem_u32(&full_q[cq.it]);
                ptx::mbar_expect_tx(full, W8::kQBytes);
                load_q(smem_q + cq.it * W8::kQBytes, full, cq.kb, cq.c.n_index);
                advance(cq);
            }
            grid_dependency_wait();
            long long stall_start = 0;
            uint32_t idle = 0;
            while (ca.live || cq.live) {
                bool progressed = false;
                if (cq.live) {
                    const uint32_t s = cq.it % SQ, ph = (cq.it / SQ) & 1;
                    if (ptx::mbar_try_wait(ptx::smem_u32(&empty_q[s]), ph ^ 1)) {
                        const uint32_t full = ptx::smem_u32(&full_q[s]);
                        ptx::mbar_expect_tx(full, W8::kQBytes);
                        load_q(smem_q + s * W8::kQBytes, full, cq.kb, cq.c.n_index);
                        advance(cq);
                        progressed = true;
                    }
                }
                if (ca.live) {
                    const uint32_t s = ca.it % SA, ph = (ca.it / SA) & 1;
                    if (ptx::mbar_try_wait(ptx::smem_u32(&empty_a[s]), ph ^ 1)) {
                        const uint32_t full = ptx::smem_u32(&full_a[s]);
                        ptx::mbar_expect_tx(full, W8::kABytes);
                        ptx::tma_load_2d(ptx::smem_u32(smem_a + s * W8::kABytes), &tma_a, full, ca.kb * BK, ca.c.row_start);
                        advance(ca);
                        progressed = true;
                    }
                }
                if (progressed) {
                    idle = 0;
                } else if (idle++ == 0) {
                    stall_start = clock64();
                } else if ((idle & 0x3FFu) == 0) {  // bounded like every other wait
                    if (*abort_flag) break;
                    if (clock64() - stall_start > ptx::kWaitCycles) {
                        *abort_flag = 1;
                        atomicOr(p.status, kCodeProducer);
                        break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16(BM, BN);
            uint32_t it = 0, count = 0;
            bool ok = true;
            Segment sg;
            for (; ok && walk.next(sg); ++count) {
                const uint32_t buf = count & 1, tph = (count >> 1) & 1;
                if (!ptx::mbar_wait(ptx::smem_u32(&tmem_empty[buf]), tph ^ 1, abort_flag, p.status, kCodeMma)) break;
                ptx::tc_fence_after();
                const uint32_t acc = tmem_base + buf * BN;
                for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
                    const uint32_t sa = it % SA, pha = (it / SA) & 1;
                    const uint32_t sc = it % SC, phc = (it / SC) & 1;
                    if (!ptx::mbar_wait(ptx::smem_u32(&full_c[sc]), phc, abort_flag, p.status, kCodeMma) ||
                        !ptx::mbar_wait(ptx::smem_u32(&full_a[sa]), pha, abort_flag, p.status, kCodeMma)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint64_t da = ptx::umma_desc_k_sw128(ptx::smem_u32(smem_a + sa * W8::kABytes));
                    const uint64_t db = ptx::umma_desc_k_sw128(ptx::smem_u32(smem_c + sc * W8::kCBytes));
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk)
                        ptx::umma_bf16(acc, da + 2 * kk, db + 2 * kk, idesc, (kb > sg.kb0) || kk != 0);
                    ptx::umma_commit(ptx::smem_u32(&empty_c[sc]));
                    ptx::umma_commit(ptx::smem_u32(&empty_a[sa]));
                }
                if (ok) ptx::umma_commit(ptx::smem_u32(&tmem_full[buf]));
            }
        }
    } else {
        const int quarter = warp & 3;
        const int pass = (warp - 2) >> 2;
        const bool leader = threadIdx.x == 64;
        float* stage = staging + (warp - 2) * kStageFloatsPerWarp;
        staging[kEpilogueWarps * kStageFloatsPerWarp + (warp - 2) * 32 + lane] = 0.0F;  // this warp's row sums of squares
        __syncwarp();
        // converting thread: the 64 K values of one of the 128 weight rows, in every second tile
        // (the other group of four warps converts the tiles in between, so two conversions overlap)
        const int row = (threadIdx.x - 64) & 127;
        const uint32_t src_offset = (row >> 6) * 4096 + (row & 63) * 64;
        uint32_t it = 0, count = 0;
        bool ok = true;
        Segment sg;
        for (; ok && walk.next(sg); ++count) {
            const TileCoord c = tile_coord(p, sg.tile, m_tiles);
            for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
                if ((it & 1u) != static_cast<uint32_t>(pass)) continue;
                const uint32_t sq = it % SQ, phq = (it / SQ) & 1;
                const uint32_t sc = it % SC, phc = (it / SC) & 1;
                if (!ptx::mbar_wait(ptx::smem_u32(&full_q[sq]), phq, abort_flag, p.status, kCodeEpilogue) ||
                    !ptx::mbar_wait(ptx::smem_u32(&empty_c[sc]), phc ^ 1, abort_flag, p.status, kCodeEpilogue)) {
                    ok = false;
                    break;
                }
                const uint4* src = reinterpret_cast<const uint4*>(smem_q + sq * W8::kQBytes + src_offset);
                uint8_t* dst_row = smem_c + sc * W8::kCBytes + row * 128;
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const uint4 packed = src[v];
                    const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
                    uint32_t out[8];
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        // bytes as q + 128 in the low mantissa bits of 2^23, minus (2^23 + 128): exactly q
                        const uint32_t biased = words[w] ^ 0x80808080u;
                        const float f0 = __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7540)) - 8388736.0F;
                        const float f1 = __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7541)) - 8388736.0F;
                        const float f2 = __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7542)) - 8388736.0F;
                        const float f3 = __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7543)) - 8388736.0F;
                        const __nv_bfloat162 lo = __floats2bfloat162_rn(f0, f1), hi = __floats2bfloat162_rn(f2, f3);
                        out[2 * w] = *reinterpret_cast<const uint32_t*>(&lo);
                        out[2 * w + 1] = *reinterpret_cast<const uint32_t*>(&hi);
                    }
                    // 16 K values = two 16-byte pieces of the row, placed as the 128-byte swizzle wants them
                    const int piece = v * 2;
                    *reinterpret_cast<uint4*>(dst_row + ((piece ^ (row & 7)) * 16)) = make_uint4(out[0], out[1], out[2], out[3]);
                    *reinterpret_cast<uint4*>(dst_row + (((piece + 1) ^ (row & 7)) * 16)) = make_uint4(out[4], out[5], out[6], out[7]);
                }
                ptx::fence_proxy_async();  // the MMA reads these bytes through the async proxy
                __syncwarp();
                if (lane == 0) {  // one arrival per warp: 128 threads on one barrier would serialise
                    ptx::mbar_arrive(ptx::smem_u32(&full_c[sc]));
                    ptx::mbar_arrive(ptx::smem_u32(&empty_q[sq]));
                }
            }
            const uint32_t buf = count & 1, tph = (count >> 1) & 1;
            bool go = ok && ptx::mbar_wait(ptx::smem_u32(&tmem_full[buf]), tph, abort_flag, p.status, kCodeEpilogue);
            if (p.shared_tiles > 0) go = ptx::named_barrier_all(2, 32 * kEpilogueWarps, go);  // one decision for the group
            if (!go) break;
            ptx::tc_fence_after();
            const uint32_t acc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            epilogue_segment<BN, true, true>(p, sg, c, k_blocks, acc, ptx::smem_u32(&tmem_empty[buf]), stage, last_flag, quarter,
                                       pass, lane, leader,
                                       folded_row_inv(p, c.row_start + quarter * 32 + lane, c.row_start + quarter * 32 + lane < c.row_end),
                                       staging + kEpilogueWarps * kStageFloatsPerWarp + (warp - 2) * 32);
        }
    }

    __syncwarp();
    ptx::tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, W8::kTmemCols);
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

bool stream_shape(const sfb_gemm_args& g) { return g.m <= BM && !g.group_offsets; }

// folded RMSNorm, sums of squares of the output, decode-step RoPE position and paged K/V append
void fill_fold_params(TcParams& p, const sfb_gemm_args& g) {
    p.row_ss = g.row_ss;
    p.row_ss_fixed = g.row_ss_fixed;
    p.rms_eps = g.rms_epsilon;
    p.owner_flags = g.owner_flags;
    p.owner_epoch = g.owner_epoch;
    p.owner_rows = g.owner_rows;
    p.owner_self = g.owner_self;
    p.m_rotate = g.owner_flags && g.owner_rows > 0 ? (g.owner_self * g.owner_rows / BM) % std::max(1, ceil_div(g.m, BM)) : 0;
    p.clear = static_cast<unsigned long long*>(g.clear);
    p.clear_pieces = static_cast<unsigned>(g.clear_bytes / 8);
    p.scatter_rows = g.scatter_rows;
    for (int i = 0; i < SFB_MAX_PEERS; ++i) p.scatter_out[i] = static_cast<bf16*>(g.scatter_out[i]);
    p.ss_out = g.out_f32 || g.scatter_rows > 0 ? nullptr : static_cast<unsigned long long*>(g.ss_out);
    p.kv_k_pool = static_cast<bf16*>(g.kv_k_pool);
    p.kv_v_pool = static_cast<bf16*>(g.kv_v_pool);
    p.kv_table = g.kv_table;
    p.kv_position = g.kv_position;
    p.kv_block_tokens = g.kv_block_tokens;
    p.kv_max_blocks = g.kv_max_blocks;
    p.kv_num_blocks = g.kv_num_blocks;
}

template <int BN, bool STREAM, bool EXTRA>
sfb_status launch(const sfb_gemm_args& g, cudaStream_t stream) {
    using T = Tile<BN, STREAM>;
    static bool configured = false;
    if (!configured) {
        SFB_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STREAM, EXTRA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      T::kSmemBytes));
        configured = true;
    }
    const int groups = g.group_offsets ? g.groups : 1;
    CUtensorMap map_a, map_b;
    if (!encode_tensor_map_bf16_2d(&map_a, g.a, static_cast<uint64_t>(g.m), static_cast<uint64_t>(g.k), BM, BK))
        return SFB_CUDA_ERROR;
    if (g.bt_tiled) {
        const uint64_t blocks = static_cast<uint64_t>(ceil_div(g.n, 64)) * ceil_div(g.k, 64);
        if (!encode_tensor_map_bf16_2d(&map_b, g.bt, blocks * 64, 64, 64, 64)) return SFB_CUDA_ERROR;
    } else if (!encode_tensor_map_bf16_2d(&map_b, g.bt, static_cast<uint64_t>(groups) * g.n,
                                          static_cast<uint64_t>(g.k), BN, BK)) {
        return SFB_CUDA_ERROR;
    }
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
    p.rope_row_offset = g.rope_row_offset;
    p.n_tiles = ceil_div(g.n, BN);
    p.b_tiled = g.bt_tiled;
    p.peer_count = g.peer_count;
    for (int i = 0; i < g.peer_count; ++i) p.peer_out[i] = static_cast<bf16*>(g.peer_out[i]);
    p.status = device_status_word();
    fill_fold_params(p, g);
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
    int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
    if (STREAM && stream_shape(g) && g.split_workspace && (reinterpret_cast<uintptr_t>(g.split_workspace) & 15) == 0 &&
        g.split_workspace_bytes >= sfb_gemm_stream_workspace_bytes(g.n)) {
        // tiles left over after the last full round; cutting them up pays unless they nearly fill a round
        const int left = static_cast<int>(tiles % sm_count());
        if (left != 0 && left <= sm_count() * 7 / 8) {
            p.shared_tiles = left;
            p.accum = static_cast<float*>(g.split_workspace);
            p.tile_counters = reinterpret_cast<int*>(p.accum + static_cast<size_t>(p.n_tiles) * BM * BN);
            const long long units = static_cast<long long>(left) * ceil_div(g.k, BK);
            grid = static_cast<int>(tiles >= sm_count() || units >= sm_count() ? sm_count() : units);
        }
    }
    SFB_CUDA(launch_dependent(gemm_tcgen05_kernel<BN, STREAM, EXTRA>, dim3(grid), dim3(kThreads), T::kSmemBytes, stream, map_a,
                              map_b, p));
    return check_launch("gemm_tcgen05");
}

sfb_status launch_w8(const sfb_gemm_args& g, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        SFB_CUDA(cudaFuncSetAttribute(gemm_w8_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, W8::kSmemBytes));
        configured = true;
    }
    CUtensorMap map_a, map_q;
    if (!encode_tensor_map_bf16_2d(&map_a, g.a, static_cast<uint64_t>(g.m), static_cast<uint64_t>(g.k), BM, BK))
        return SFB_CUDA_ERROR;
    const uint64_t blocks = static_cast<uint64_t>(ceil_div(g.n, 64)) * ceil_div(g.k, 64);
    if (!encode_tensor_map_u8_2d(&map_q, g.bt, blocks * 64, 64, 64, 64)) return SFB_CUDA_ERROR;
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
    p.rope_row_offset = g.rope_row_offset;
    p.n_tiles = ceil_div(g.n, W8::BN);
    p.b_tiled = 1;
    p.col_scale = g.bt_scales;
    p.peer_count = g.peer_count;
    for (int i = 0; i < g.peer_count; ++i) p.peer_out[i] = static_cast<bf16*>(g.peer_out[i]);
    p.status = device_status_word();
    fill_fold_params(p, g);
    p.tile_table = nullptr;
    p.dense_m_tiles = 1;
    const long long tiles = p.n_tiles;
    int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
    if (g.split_workspace && (reinterpret_cast<uintptr_t>(g.split_workspace) & 15) == 0 &&
        g.split_workspace_bytes >= sfb_gemm_stream_workspace_bytes(g.n)) {
        const int left = static_cast<int>(tiles % sm_count());
        if (left != 0 && left <= sm_count() * 7 / 8) {
            p.shared_tiles = left;
            p.accum = static_cast<float*>(g.split_workspace);
            p.tile_counters = reinterpret_cast<int*>(p.accum + static_cast<size_t>(p.n_tiles) * BM * W8::BN);
            const long long units = static_cast<long long>(left) * ceil_div(g.k, BK);
            grid = static_cast<int>(tiles >= sm_count() || units >= sm_count() ? sm_count() : units);
        }
    }
    SFB_CUDA(launch_dependent(gemm_w8_tcgen05_kernel, dim3(grid), dim3(kThreads), W8::kSmemBytes, stream, map_a, map_q, p));
    return check_launch("gemm_w8_tcgen05");
}

int pick_bn(const sfb_gemm_args& g) {
    if (g.epilogue == SFB_EPI_SWIGLU) return 2 * g.swiglu_block;
    if (g.bt_tiled || stream_shape(g)) return 128;
    if (g.n < 256) return 128;
    // Wave quantisation: the tiles run in rounds of one per SM, so the time is about rounds x tile cost.  A round of
    // 128-column tiles measured 0.8 of a round of 256-column tiles (8192 rows; N 768..6144, K 2048..4096: the A tile
    // is re-read for half the work and the epilogue does not shrink), so the narrow tile only pays where it does not
    // add rounds: a short or narrow output whose wide tiles leave most SMs idle.
    const long long m_tiles = ceil_div(g.m, BM);
    const long long rounds_wide = ceil_div64(m_tiles * ceil_div(g.n, 256), sm_count());
    const long long rounds_narrow = ceil_div64(m_tiles * ceil_div(g.n, 128), sm_count());
    return rounds_narrow * 160 < rounds_wide * 200 ? 128 : 256;
}

}  // namespace

bool gemm_bf16_tcgen05_supported(const sfb_gemm_args& g) {
    if (g.k % 8 != 0) return false;  // TMA row pitch must be a multiple of 16 bytes
    if ((reinterpret_cast<uintptr_t>(g.a) & 15) || (reinterpret_cast<uintptr_t>(g.bt) & 15)) return false;
    if (g.epilogue == SFB_EPI_SWIGLU && g.swiglu_block != 64 && g.swiglu_block != 128) return false;
    if (g.bt_tiled && (g.group_offsets || (g.epilogue == SFB_EPI_SWIGLU && g.swiglu_block != 64))) return false;
    if (g.epilogue == SFB_EPI_ROPE_SPLIT && g.head_dim % 32 != 0) return false;
    if (g.bt_scales && (!stream_shape(g) || (g.epilogue == SFB_EPI_SWIGLU && g.swiglu_block != 64) ||
                        (reinterpret_cast<uintptr_t>(g.bt_scales) & 15)))
        return false;  // int8 weights: one M-tile, dense, 128-column tiles
    if (g.peer_count != 0 && (g.peer_count < 0 || g.peer_count >= SFB_MAX_PEERS || g.out_f32 || g.group_offsets ||
                              (g.epilogue != SFB_EPI_STORE && g.epilogue != SFB_EPI_RESIDUAL)))
        return false;
    if (g.scatter_rows != 0) {
        if (g.scatter_rows < 0 || g.out_f32 || g.group_offsets || g.peer_count != 0 ||
            (g.epilogue != SFB_EPI_STORE && g.epilogue != SFB_EPI_RESIDUAL) || ceil_div(g.m, g.scatter_rows) > SFB_MAX_PEERS)
            return false;
        for (int i = 0; i < ceil_div(g.m, g.scatter_rows); ++i)
            if (!g.scatter_out[i]) return false;
    }
    if (g.row_ss && g.group_offsets) return false;
    if (g.ss_out && (g.group_offsets || (reinterpret_cast<uintptr_t>(g.ss_out) & 7) ||
                     (g.epilogue != SFB_EPI_STORE && g.epilogue != SFB_EPI_RESIDUAL)))
        return false;
    if (g.clear && ((reinterpret_cast<uintptr_t>(g.clear) & 7) || g.clear_bytes % 8 != 0)) return false;
    if (g.owner_flags && (g.group_offsets || stream_shape(g) || g.owner_rows <= 0 || g.owner_rows % BM != 0 ||
                          g.m % g.owner_rows != 0 || g.m / g.owner_rows > SFB_MAX_PEERS || g.owner_self < 0 ||
                          g.owner_self >= g.m / g.owner_rows))
        return false;
    if (g.kv_k_pool && (g.epilogue != SFB_EPI_ROPE_SPLIT || !g.kv_v_pool || !g.kv_table || g.kv_block_tokens <= 0 ||
                        g.kv_max_blocks <= 0 || g.kv_position < 0))
        return false;
    return true;
}

sfb_status gemm_bf16_tcgen05(const sfb_gemm_args& g, cudaStream_t stream) {
    if (g.bt_scales) return launch_w8(g, stream);
    const bool extra = g.row_ss || g.ss_out || g.scatter_rows > 0 || g.kv_k_pool || g.clear || g.owner_flags;
    if (pick_bn(g) == 256) return extra ? launch<256, false, true>(g, stream) : launch<256, false, false>(g, stream);
    if (stream_shape(g)) return extra ? launch<128, true, true>(g, stream) : launch<128, true, false>(g, stream);
    return extra ? launch<128, false, true>(g, stream) : launch<128, false, false>(g, stream);
}

}  // namespace sfb

extern "C" size_t sfb_gemm_stream_workspace_bytes(int n) {
    if (n <= 0) return 0;
    const size_t tiles = static_cast<size_t>(sfb::ceil_div(n, 128));
    return tiles * (128 * 128 * sizeof(float)) + (tiles * sizeof(int) + 15) / 16 * 16;
}
