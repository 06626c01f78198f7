// Flash-attention prefill on the 5th-generation tensor cores (bf16, head_dim = 128).
//
// One CTA owns 256 consecutive query rows of one (batch, head) as two 128-row Q tiles and walks
// the keys in tiles of 64.  320 threads in four roles:
//   warps 0-3   softmax group of Q tile 0: thread r owns query row r.  Per KV tile it reads
//   warps 4-7   (tile 1)  its 64 scores from tensor memory, masks, takes the row max, and writes
//               p = 2^(s*c - m) as bf16 into a 128-byte-swizzled shared-memory tile that the next
//               MMA reads as its A operand.  No cross-thread reduction is ever needed.
//   warp 8      TMA producer: Q tiles once, then K tiles (4-deep ring) and V tiles (3-deep ring).
//   warp 9      MMA issuer (one thread): S_t = Q_t.K^T (M128 N64 K128) into tensor memory, then
//               O_t += P_t.V (M128 N128 K64, V as an MN-major operand) accumulated in tensor
//               memory.  S is double-buffered per Q tile: Q.K^T of KV tile j+2 is issued as soon
//               as the softmax group has consumed tile j, so a group never waits for the tensor
//               pipe, and the two Q tiles alternate on it.
// Running maxima are updated lazily: the accumulator in tensor memory is rescaled (by the
// owning softmax group, with tcgen05.ld/st) only when a row maximum grows by more than 2^8;
// the final division by the row sum makes the result exact regardless.
// Causal masking follows the reference: key j is visible to query i iff j <= Sk - Sq + i; KV
// tiles above the frontier of a Q tile are never loaded or multiplied for it.
// Every wait is bounded (see ptx_sm100.cuh).
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace sfb {
namespace {

constexpr int D = 128;          // head_dim == head_dim_value
constexpr int QT = 128;         // rows per Q tile
constexpr int KT = 64;          // keys per KV tile
constexpr int KSTAGES = 4;       // K ring (Q.K^T runs two tiles ahead of P.V)
constexpr int VSTAGES = 3;       // V ring
constexpr int kThreads = 320;
constexpr int kQBytes = QT * D * 2;        // 32 KiB per Q tile (two 16 KiB halves of 64 dims)
constexpr int kKBytes = KT * D * 2;        // 16 KiB
constexpr int kVBytes = KT * D * 2;        // 16 KiB
constexpr int kPBytes = QT * KT * 2;       // 16 KiB per Q tile
constexpr int kSmemBytes = 2 * kQBytes + KSTAGES * kKBytes + VSTAGES * kVBytes + 2 * kPBytes + 512 + 1024;
constexpr uint32_t kTmemCols = 512;        // S[t][buf] at (2t+buf)*64 in [0,256); O0 [256,384) O1 [384,512)
constexpr uint32_t kOCol = 256;
constexpr uint32_t kCodeAttn = 0x10;
constexpr float kRescaleThreshold = 8.0F;  // log2 units

struct FaParams {
    bf16* out;
    int batch, q_heads, kv_heads, seq_q, seq_kv;
    int causal, token_major;
    float scale_log2;  // scale * log2(e)
    uint32_t* status;
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(kThreads, 1)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                                 const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ FaParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_smem = smem;                                  // [2][2 halves][128][64]
    uint8_t* k_smem = q_smem + 2 * kQBytes;                  // [KSTAGES][2 halves][64][64]
    uint8_t* v_smem = k_smem + KSTAGES * kKBytes;            // [VSTAGES][2 halves][64 keys][64 dv]
    uint8_t* p_smem = v_smem + VSTAGES * kVBytes;            // [2][128][64]
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_smem + 2 * kPBytes);
    uint64_t* q_full = bars;                 // [2]
    uint64_t* k_full = bars + 2;             // [KSTAGES]
    uint64_t* k_empty = k_full + KSTAGES;    // [KSTAGES]
    uint64_t* v_full = k_empty + KSTAGES;    // [VSTAGES]
    uint64_t* v_empty = v_full + VSTAGES;    // [VSTAGES]
    uint64_t* s_full = v_empty + VSTAGES;    // [2 tiles][2 buffers]
    uint64_t* p_full = s_full + 4;           // [2]
    uint64_t* pv_done = p_full + 2;          // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_blocks = (p.seq_q + 2 * QT - 1) / (2 * QT);
    // heaviest (latest) query blocks first: they see the most keys under a causal mask
    const int qb = q_blocks - 1 - static_cast<int>(blockIdx.x % q_blocks);
    const int head = (blockIdx.x / q_blocks) % p.q_heads;
    const int b = blockIdx.x / q_blocks / p.q_heads;
    const int kvh = head * p.kv_heads / p.q_heads;
    const int q0 = qb * 2 * QT;
    const int offset = p.seq_kv - p.seq_q;
    int n_tiles[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int start = q0 + t * QT;
        if (start >= p.seq_q) { n_tiles[t] = 0; continue; }
        const int last = min(start + QT, p.seq_q) - 1;
        const int limit = p.causal ? min(p.seq_kv, offset + last + 1) : p.seq_kv;
        n_tiles[t] = (limit + KT - 1) / KT;
    }
    const int n_max = max(n_tiles[0], n_tiles[1]);
    const int q_row0 = (b * p.q_heads + head) * p.seq_q + q0;   // row in the [B*Hq*Sq, D] view
    const int kv_row0 = (b * p.kv_heads + kvh) * p.seq_kv;      // row in the [B*Hkv*Sk, D] view

    if (threadIdx.x == 0) {
        for (int t = 0; t < 2; ++t) {
            ptx::mbar_init(ptx::smem_u32(&q_full[t]), 1);
            ptx::mbar_init(ptx::smem_u32(&s_full[2 * t]), 1);
            ptx::mbar_init(ptx::smem_u32(&s_full[2 * t + 1]), 1);
            ptx::mbar_init(ptx::smem_u32(&p_full[t]), QT);
            ptx::mbar_init(ptx::smem_u32(&pv_done[t]), 1);
        }
        for (int s = 0; s < KSTAGES; ++s) {
            ptx::mbar_init(ptx::smem_u32(&k_full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&k_empty[s]), 1);
        }
        for (int s = 0; s < VSTAGES; ++s) {
            ptx::mbar_init(ptx::smem_u32(&v_full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&v_empty[s]), 1);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
        ptx::prefetch_tensormap(&tma_q);
        ptx::prefetch_tensormap(&tma_k);
        ptx::prefetch_tensormap(&tma_v);
    }
    if (warp == 9) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 8) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            for (int t = 0; t < 2; ++t) {
                if (n_tiles[t] == 0) continue;
                const uint32_t bar = ptx::smem_u32(&q_full[t]);
                ptx::mbar_expect_tx(bar, kQBytes);
                ptx::tma_load_2d(ptx::smem_u32(q_smem + t * kQBytes), &tma_q, bar, 0, q_row0 + t * QT);
                ptx::tma_load_2d(ptx::smem_u32(q_smem + t * kQBytes + kQBytes / 2), &tma_q, bar, 64, q_row0 + t * QT);
            }
            for (int j = 0; j < n_max; ++j) {
                const int ks = j % KSTAGES, vs = j % VSTAGES;
                const int row = kv_row0 + j * KT;
                if (!ptx::mbar_wait(ptx::smem_u32(&k_empty[ks]), ((j / KSTAGES) & 1) ^ 1, abort_flag, p.status, kCodeAttn | 1)) break;
                const uint32_t kb = ptx::smem_u32(&k_full[ks]);
                ptx::mbar_expect_tx(kb, kKBytes);
                ptx::tma_load_2d(ptx::smem_u32(k_smem + ks * kKBytes), &tma_k, kb, 0, row);
                ptx::tma_load_2d(ptx::smem_u32(k_smem + ks * kKBytes + kKBytes / 2), &tma_k, kb, 64, row);
                if (!ptx::mbar_wait(ptx::smem_u32(&v_empty[vs]), ((j / VSTAGES) & 1) ^ 1, abort_flag, p.status, kCodeAttn | 1)) break;
                const uint32_t vb = ptx::smem_u32(&v_full[vs]);
                ptx::mbar_expect_tx(vb, kVBytes);
                ptx::tma_load_2d(ptx::smem_u32(v_smem + vs * kVBytes), &tma_v, vb, 0, row);
                ptx::tma_load_2d(ptx::smem_u32(v_smem + vs * kVBytes + kVBytes / 2), &tma_v, vb, 64, row);
            }
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = ptx::umma_idesc_bf16(QT, KT, 0, 0);
            constexpr uint32_t idesc_pv = ptx::umma_idesc_bf16(QT, D, 0, 1);
            auto issue_qk = [&](int t, int j) {  // S_t[j & 1] = Q_t . K_j^T
                const int s = j % KSTAGES;
                const uint32_t qa = ptx::smem_u32(q_smem + t * kQBytes), ka = ptx::smem_u32(k_smem + s * kKBytes);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint64_t da = ptx::umma_desc_k_sw128(qa + (kk / 4) * (kQBytes / 2) + (kk % 4) * 32);
                    const uint64_t db = ptx::umma_desc_k_sw128(ka + (kk / 4) * (kKBytes / 2) + (kk % 4) * 32);
                    ptx::umma_bf16(tmem_base + (2 * t + (j & 1)) * KT, da, db, idesc_qk, kk != 0);
                }
                ptx::umma_commit(ptx::smem_u32(&s_full[2 * t + (j & 1)]));
            };
            auto issue_pv = [&](int t, int j) {  // O_t += P_t . V_j
                const int s = j % VSTAGES;
                const uint32_t pa = ptx::smem_u32(p_smem + t * kPBytes), va = ptx::smem_u32(v_smem + s * kVBytes);
#pragma unroll
                for (int kk = 0; kk < KT / 16; ++kk) {
                    const uint64_t da = ptx::umma_desc_k_sw128(pa + kk * 32);
                    const uint64_t db = ptx::umma_desc_mn_sw128(va + kk * 16 * 128, kVBytes / 2, 1024);
                    ptx::umma_bf16(tmem_base + kOCol + t * D, da, db, idesc_pv, (j | kk) != 0);
                }
                ptx::umma_commit(ptx::smem_u32(&pv_done[t]));
            };
            bool ok = true;
            for (int t = 0; t < 2 && ok; ++t)
                if (n_tiles[t] > 0) ok = ptx::mbar_wait(ptx::smem_u32(&q_full[t]), 0, abort_flag, p.status, kCodeAttn | 2);
            // prologue: scores of KV tiles 0 and 1 for both Q tiles
            for (int j = 0; ok && j < min(2, n_max); ++j) {
                ok = ptx::mbar_wait(ptx::smem_u32(&k_full[j % KSTAGES]), (j / KSTAGES) & 1, abort_flag, p.status, kCodeAttn | 2);
                if (!ok) break;
                ptx::tc_fence_after();
                for (int t = 0; t < 2; ++t)
                    if (j < n_tiles[t]) issue_qk(t, j);
                ptx::umma_commit(ptx::smem_u32(&k_empty[j % KSTAGES]));
            }
            for (int j = 0; ok && j < n_max; ++j) {
                const int vs = j % VSTAGES;
                for (int t = 0; ok && t < 2; ++t) {
                    if (j >= n_tiles[t]) continue;
                    ok = ptx::mbar_wait(ptx::smem_u32(&p_full[t]), j & 1, abort_flag, p.status, kCodeAttn | 2) &&
                         ptx::mbar_wait(ptx::smem_u32(&v_full[vs]), (j / VSTAGES) & 1, abort_flag, p.status, kCodeAttn | 2);
                    if (!ok) break;
                    ptx::tc_fence_after();
                    issue_pv(t, j);
                    if (j + 2 < n_tiles[t]) {  // S_t[j & 1] has been consumed: next scores into it
                        ok = ptx::mbar_wait(ptx::smem_u32(&k_full[(j + 2) % KSTAGES]), ((j + 2) / KSTAGES) & 1, abort_flag,
                                            p.status, kCodeAttn | 2);
                        if (!ok) break;
                        ptx::tc_fence_after();
                        issue_qk(t, j + 2);
                    }
                }
                if (ok) {
                    ptx::umma_commit(ptx::smem_u32(&v_empty[vs]));
                    if (j + 2 < n_max) ptx::umma_commit(ptx::smem_u32(&k_empty[(j + 2) % KSTAGES]));
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax groups
        const int t = warp >> 2;                 // Q tile of this group
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;       // row inside the tile == tensor-memory lane
        const int qi = q0 + t * QT + r;          // query index inside the sequence
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t s_addr0 = tmem_base + lane_base + 2 * t * KT;
        const uint32_t o_addr = tmem_base + lane_base + kOCol + t * D;
        uint8_t* p_row = p_smem + t * kPBytes + r * 128;
        const int nt = n_tiles[t];
        float m_used = -INFINITY, row_sum = 0.0F;
        bool ok = true;
        for (int j = 0; ok && j < nt; ++j) {
            ok = ptx::mbar_wait(ptx::smem_u32(&s_full[2 * t + (j & 1)]), (j >> 1) & 1, abort_flag, p.status, kCodeAttn | 4);
            if (!ok) break;
            ptx::tc_fence_after();
            const uint32_t s_addr = s_addr0 + (j & 1) * KT;
            uint32_t raw[2][32];
            ptx::tmem_ld_32x32(s_addr, raw[0]);
            ptx::tmem_ld_32x32(s_addr + 32, raw[1]);
            ptx::tmem_ld_wait();
            float x[64];
#pragma unroll
            for (int i = 0; i < 64; ++i) x[i] = __uint_as_float(raw[i >> 5][i & 31]) * p.scale_log2;
            const int key0 = j * KT;
            const bool needs_mask = (p.causal && key0 + KT - 1 > offset + q0 + t * QT) || key0 + KT > p.seq_kv;
            if (needs_mask) {
                const int limit = p.causal ? min(p.seq_kv - 1, offset + qi) : p.seq_kv - 1;
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    if (key0 + i > limit) x[i] = -INFINITY;
            }
            float tile_max = x[0];
#pragma unroll
            for (int i = 1; i < 64; ++i) tile_max = fmaxf(tile_max, x[i]);
            // lazy running maximum: move it only when the row maximum outgrows it by 2^8
            const bool grow = tile_max > m_used + kRescaleThreshold;
            if (j > 0) {
                // O_t and the P tile may be touched only after the previous P.V of this tile has finished
                ok = ptx::mbar_wait(ptx::smem_u32(&pv_done[t]), (j - 1) & 1, abort_flag, p.status, kCodeAttn | 4);
                if (!ok) break;
                if (__any_sync(0xffffffffu, grow)) {
                    const float alpha = grow ? fast_exp2(m_used - tile_max) : 1.0F;  // 2^(-inf) = 0 for a fresh row
                    ptx::tc_fence_after();
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t o[32];
                        ptx::tmem_ld_32x32(o_addr + c * 32, o);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        ptx::tmem_st_32x32(o_addr + c * 32, o);
                    }
                    ptx::tmem_st_wait();
                    row_sum *= alpha;
                }
            }
            if (grow) m_used = tile_max;
            float tile_sum = 0.0F;
            if (m_used == -INFINITY) {
#pragma unroll
                for (int i = 0; i < 64; ++i) x[i] = 0.0F;  // nothing visible yet for this row
            } else {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    x[i] = fast_exp2(x[i] - m_used);
                    tile_sum += x[i];
                }
            }
            row_sum += tile_sum;
            // P row (64 bf16 = 128 bytes) into the 128-byte-swizzled K-major tile: 16-byte chunk c of
            // row r lives at chunk position c ^ (r % 8)
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint4 packed;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(x[8 * c + 2 * i], x[8 * c + 2 * i + 1]);
                *reinterpret_cast<uint4*>(p_row + ((c ^ (r & 7)) << 4)) = packed;
            }
            ptx::fence_proxy_async();
            ptx::tc_fence_before();
            ptx::mbar_arrive(ptx::smem_u32(&p_full[t]));
        }
        if (ok && nt > 0)
            ok = ptx::mbar_wait(ptx::smem_u32(&pv_done[t]), (nt - 1) & 1, abort_flag, p.status, kCodeAttn | 4);
        if (ok && nt > 0) {
            ptx::tc_fence_after();
            const float inv = 1.0F / row_sum;
            bf16* dst;
            if (p.token_major)
                dst = p.out + (static_cast<size_t>(b) * p.seq_q + qi) * (p.q_heads * D) + head * D;
            else
                dst = p.out + ((static_cast<size_t>(b) * p.q_heads + head) * p.seq_q + qi) * D;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t o[32];
                ptx::tmem_ld_32x32(o_addr + c * 32, o);
                ptx::tmem_ld_wait();
                if (qi < p.seq_q) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 packed;
                        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            h[k] = __floats2bfloat162_rn(__uint_as_float(o[8 * i + 2 * k]) * inv,
                                                         __uint_as_float(o[8 * i + 2 * k + 1]) * inv);
                        reinterpret_cast<uint4*>(dst + c * 32)[i] = packed;
                    }
                }
            }
        }
    }

    __syncwarp();
    ptx::tc_fence_before();
    __syncthreads();
    if (*abort_flag)
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    if (warp == 9) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace

bool attention_prefill_tcgen05_supported(const sfb_attention_args& a) {
    return a.dtype == SFB_BF16 && a.head_dim == D && a.head_dim_value == D &&
           (reinterpret_cast<uintptr_t>(a.q) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.key) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(a.value) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15) == 0;
}

sfb_status attention_prefill_tcgen05(const sfb_attention_args& a, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        SFB_CUDA(cudaFuncSetAttribute(attention_prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSmemBytes));
        configured = true;
    }
    CUtensorMap map_q, map_k, map_v;
    const uint64_t q_rows = static_cast<uint64_t>(a.batch) * a.q_heads * a.seq_q;
    const uint64_t kv_rows = static_cast<uint64_t>(a.batch) * a.kv_heads * a.seq_kv;
    if (!encode_tensor_map_bf16_2d(&map_q, a.q, q_rows, D, QT, 64) ||
        !encode_tensor_map_bf16_2d(&map_k, a.key, kv_rows, D, KT, 64) ||
        !encode_tensor_map_bf16_2d(&map_v, a.value, kv_rows, D, KT, 64))
        return SFB_CUDA_ERROR;
    FaParams p{};
    p.out = static_cast<bf16*>(a.out);
    p.batch = a.batch; p.q_heads = a.q_heads; p.kv_heads = a.kv_heads; p.seq_q = a.seq_q; p.seq_kv = a.seq_kv;
    p.causal = a.causal; p.token_major = a.token_major;
    p.scale_log2 = a.scale * 1.4426950408889634F;
    p.status = device_status_word();
    const int q_blocks = ceil_div(a.seq_q, 2 * QT);
    const int grid = a.batch * a.q_heads * q_blocks;
    attention_prefill_tcgen05_kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_q, map_k, map_v, p);
    return check_launch("attention_prefill_tcgen05");
}

}  // namespace sfb
