// Flash-attention prefill on the 5th-generation tensor cores (bf16, head_dim = 128 or 64).
//
// One CTA owns 256 consecutive query rows of one (batch, head) as two 128-row Q tiles and walks
// the keys in tiles of 128.  384 threads, 320 of them in four roles:
//   warps 0-3   softmax group of Q tile 0: thread r owns query row r (= tensor-memory lane r), so
//   warps 4-7   (tile 1)  no cross-thread reduction is ever needed.  Per KV tile it reads its 128
//               scores from tensor memory once into registers (row maximum, then exponentials),
//               and writes p = 2^(s*c - m) as packed bf16 back into tensor memory OVER the
//               scores; the next MMA reads P from there as its A operand.
//   warp 8      TMA producer: Q tiles once, then K and V tiles through two 2-deep rings.
//   warp 9      MMA issuer (one thread): S_t = Q_t.K^T (M128 N128 K128, both operands in shared
//               memory) and O_t += P_t.V (M128 N128 K128, A = P_t from tensor memory, B = V as an
//               MN-major shared-memory operand), accumulators in tensor memory
//               (S0 S1 O0 O1 = 512 columns).  The two Q tiles alternate on the tensor pipe, so
//               while one group does exponentials the pipe works for the other.
// Keeping P in tensor memory and using 128-key tiles halves the shared-memory operand traffic per
// key compared with a 64-key tile and a P tile in shared memory; that traffic, not the MMA rate,
// bounded the first version of this kernel.
// Running maxima move lazily: the accumulator is rescaled (by the owning softmax group, with
// tcgen05.ld/st) only when a row maximum grows by more than 2^8; the final division by the row
// sum makes the result exact regardless.
// Causal masking follows the reference: key j is visible to query i iff j <= Sk - Sq + i; KV
// tiles above the frontier of a Q tile are never loaded or multiplied for it.
// Every wait is bounded (see ptx_sm100.cuh).
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace sfb {
namespace {

constexpr int QT = 128;         // rows per Q tile
constexpr int KT = 128;         // keys per KV tile
constexpr int KSTAGES = 2;
constexpr int VSTAGES = 2;
constexpr int kThreads = 384;         // three warpgroups; warps 10 and 11 only take part in the register hand-over
constexpr int kHalfBytes = 128 * 64 * 2;   // 128 rows of 64 dims: the unit every Q, K and V tile is made of
// D = head_dim == head_dim_value, 128 or 64: a tile is D / 64 such halves (32 or 16 KiB)
template <int D>
struct Fa {
    static constexpr int kHalves = D / 64;
    static constexpr int kQBytes = kHalves * kHalfBytes;
    static constexpr int kKBytes = kHalves * kHalfBytes;
    static constexpr int kVBytes = kHalves * kHalfBytes;
    static constexpr int kSmemBytes = 2 * kQBytes + KSTAGES * kKBytes + VSTAGES * kVBytes + 512 + 1024;
};
constexpr uint32_t kTmemCols = 512;        // S_t (and P_t over its first 64 columns) at t*128; O_t at 256 + t*D
constexpr uint32_t kOCol = 256;
constexpr uint32_t kCodeAttn = 0x10;
constexpr float kRescaleThreshold = 8.0F;  // log2 units

struct FaParams {
    bf16* out;
    int batch, q_heads, kv_heads, seq_q, seq_kv;
    int q_head_rows, kv_head_rows;  // rows between two heads in memory (>= seq_q / seq_kv for a slice of longer sequences)
    int causal, token_major;
    float scale_log2;  // scale * log2(e)
    uint32_t* status;
};

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                                 const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ FaParams p) {
    constexpr int kHalves = Fa<D>::kHalves, kQBytes = Fa<D>::kQBytes, kKBytes = Fa<D>::kKBytes, kVBytes = Fa<D>::kVBytes;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_smem = smem;                                  // [2][halves][128][64]
    uint8_t* k_smem = q_smem + 2 * kQBytes;                  // [KSTAGES][halves][128 keys][64 dims]
    uint8_t* v_smem = k_smem + KSTAGES * kKBytes;            // [VSTAGES][halves][128 keys][64 dv]
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_smem + VSTAGES * kVBytes);
    uint64_t* q_full = bars;                 // [2]
    uint64_t* k_full = bars + 2;             // [KSTAGES]
    uint64_t* k_empty = k_full + KSTAGES;    // [KSTAGES]
    uint64_t* v_full = k_empty + KSTAGES;    // [VSTAGES]
    uint64_t* v_empty = v_full + VSTAGES;    // [VSTAGES]
    uint64_t* s_full = v_empty + VSTAGES;    // [2]
    uint64_t* p_full = s_full + 2;           // [2]
    uint64_t* o_full = p_full + 2;           // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 2);
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
    const int q_row0 = (b * p.q_heads + head) * p.q_head_rows + q0;   // row in the [B*Hq*rows, D] view
    const int kv_row0 = (b * p.kv_heads + kvh) * p.kv_head_rows;      // row in the [B*Hkv*rows, D] view

    if (threadIdx.x == 0) {
        for (int t = 0; t < 2; ++t) {
            ptx::mbar_init(ptx::smem_u32(&q_full[t]), 1);
            ptx::mbar_init(ptx::smem_u32(&s_full[t]), 1);
            ptx::mbar_init(ptx::smem_u32(&p_full[t]), QT);
            ptx::mbar_init(ptx::smem_u32(&o_full[t]), 1);
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

    // The softmax threads keep a whole 128-score row in registers; the third warpgroup (copy and
    // MMA issue, one thread each) hands its share of the register file over to them.
    if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 8) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            for (int t = 0; t < 2; ++t) {
                if (n_tiles[t] == 0) continue;
                const uint32_t bar = ptx::smem_u32(&q_full[t]);
                ptx::mbar_expect_tx(bar, kQBytes);
#pragma unroll
                for (int h = 0; h < kHalves; ++h)
                    ptx::tma_load_2d(ptx::smem_u32(q_smem + t * kQBytes + h * kHalfBytes), &tma_q, bar, 64 * h, q_row0 + t * QT);
            }
            for (int j = 0; j < n_max; ++j) {
                const int ks = j % KSTAGES, vs = j % VSTAGES;
                const int row = kv_row0 + j * KT;
                if (!ptx::mbar_wait(ptx::smem_u32(&k_empty[ks]), ((j / KSTAGES) & 1) ^ 1, abort_flag, p.status, kCodeAttn | 1)) break;
                const uint32_t kb = ptx::smem_u32(&k_full[ks]);
                ptx::mbar_expect_tx(kb, kKBytes);
#pragma unroll
                for (int h = 0; h < kHalves; ++h)
                    ptx::tma_load_2d(ptx::smem_u32(k_smem + ks * kKBytes + h * kHalfBytes), &tma_k, kb, 64 * h, row);
                if (!ptx::mbar_wait(ptx::smem_u32(&v_empty[vs]), ((j / VSTAGES) & 1) ^ 1, abort_flag, p.status, kCodeAttn | 1)) break;
                const uint32_t vb = ptx::smem_u32(&v_full[vs]);
                ptx::mbar_expect_tx(vb, kVBytes);
#pragma unroll
                for (int h = 0; h < kHalves; ++h)
                    ptx::tma_load_2d(ptx::smem_u32(v_smem + vs * kVBytes + h * kHalfBytes), &tma_v, vb, 64 * h, row);
            }
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = ptx::umma_idesc_bf16(QT, KT, 0, 0);
            constexpr uint32_t idesc_pv = ptx::umma_idesc_bf16(QT, D, 0, 1);
            auto issue_qk = [&](int t, int j) {  // S_t = Q_t . K_j^T
                const uint32_t qa = ptx::smem_u32(q_smem + t * kQBytes);
                const uint32_t ka = ptx::smem_u32(k_smem + (j % KSTAGES) * kKBytes);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint64_t da = ptx::umma_desc_k_sw128(qa + (kk / 4) * kHalfBytes + (kk % 4) * 32);
                    const uint64_t db = ptx::umma_desc_k_sw128(ka + (kk / 4) * kHalfBytes + (kk % 4) * 32);
                    ptx::umma_bf16(tmem_base + t * KT, da, db, idesc_qk, kk != 0);
                }
                ptx::umma_commit(ptx::smem_u32(&s_full[t]));
            };
            auto issue_pv = [&](int t, int j) {  // O_t += P_t . V_j, P_t read from tensor memory
                const uint32_t va = ptx::smem_u32(v_smem + (j % VSTAGES) * kVBytes);
#pragma unroll
                for (int kk = 0; kk < KT / 16; ++kk) {
                    const uint64_t db = ptx::umma_desc_mn_sw128(va + kk * 16 * 128, kHalfBytes, 1024);
                    ptx::umma_bf16_ts(tmem_base + kOCol + t * D, tmem_base + t * KT + kk * 8, db, idesc_pv, (j | kk) != 0);
                }
            };
            bool ok = true;
            for (int t = 0; t < 2 && ok; ++t)
                if (n_tiles[t] > 0) ok = ptx::mbar_wait(ptx::smem_u32(&q_full[t]), 0, abort_flag, p.status, kCodeAttn | 2);
            if (ok && n_max > 0) ok = ptx::mbar_wait(ptx::smem_u32(&k_full[0]), 0, abort_flag, p.status, kCodeAttn | 2);
            if (ok && n_max > 0) {
                ptx::tc_fence_after();
                for (int t = 0; t < 2; ++t)
                    if (n_tiles[t] > 0) issue_qk(t, 0);
                ptx::umma_commit(ptx::smem_u32(&k_empty[0]));
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
                    if (j + 1 == n_tiles[t]) ptx::umma_commit(ptx::smem_u32(&o_full[t]));
                    if (j + 1 < n_tiles[t]) {  // the tensor pipe runs in order: P_t is consumed before S_t is overwritten
                        ok = ptx::mbar_wait(ptx::smem_u32(&k_full[(j + 1) % KSTAGES]), ((j + 1) / KSTAGES) & 1, abort_flag,
                                            p.status, kCodeAttn | 2);
                        if (!ok) break;
                        ptx::tc_fence_after();
                        issue_qk(t, j + 1);
                    }
                }
                if (ok) {
                    ptx::umma_commit(ptx::smem_u32(&v_empty[vs]));
                    if (j + 1 < n_max) ptx::umma_commit(ptx::smem_u32(&k_empty[(j + 1) % KSTAGES]));
                }
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
        // ---------------------------------------------------------------- softmax groups
        const int t = warp >> 2;                 // Q tile of this group
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;       // row inside the tile == tensor-memory lane
        const int qi = q0 + t * QT + r;          // query index inside the sequence
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t s_addr = tmem_base + lane_base + t * KT;   // scores, and P over their first 64 columns
        const uint32_t o_addr = tmem_base + lane_base + kOCol + t * D;
        const int nt = n_tiles[t];
        float m_used = -INFINITY, row_sum = 0.0F;
        bool ok = true;
        for (int j = 0; ok && j < nt; ++j) {
            ok = ptx::mbar_wait(ptx::smem_u32(&s_full[t]), j & 1, abort_flag, p.status, kCodeAttn | 4);
            if (!ok) break;
            ptx::tc_fence_after();
            const int key0 = j * KT;
            const bool needs_mask = (p.causal && key0 + KT - 1 > offset + q0 + t * QT) || key0 + KT > p.seq_kv;
            const int limit = p.causal ? min(p.seq_kv - 1, offset + qi) : p.seq_kv - 1;  // last visible key
            // The 128 scores of the row are read from tensor memory ONCE and stay in registers: the
            // second half is in flight while the maximum of the first half is taken.
            uint32_t raw[KT / 32][32];
            ptx::tmem_ld_32x32(s_addr, raw[0]);
            ptx::tmem_ld_32x32(s_addr + 32, raw[1]);
            ptx::tmem_ld_32x32(s_addr + 64, raw[2]);
            ptx::tmem_ld_32x32(s_addr + 96, raw[3]);
            ptx::tmem_ld_wait();  // one load latency (~400 cycles) for the whole row
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int c = 0; c < KT / 64; ++c) {
                if (needs_mask) {
#pragma unroll
                    for (int i = 0; i < 64; ++i)
                        if (key0 + c * 64 + i > limit) raw[2 * c + (i >> 5)][i & 31] = 0xff800000u;  // -inf, and 2^-inf = 0 below
                }
#pragma unroll
                for (int i = 0; i < 64; i += 8) {  // three-input maximum: half the instructions of fmaxf chains
                    const uint32_t* v = &raw[2 * c + (i >> 5)][i & 31];
                    mx0 = max3(mx0, __uint_as_float(v[0]), __uint_as_float(v[1]));
                    mx1 = max3(mx1, __uint_as_float(v[2]), __uint_as_float(v[3]));
                    mx2 = max3(mx2, __uint_as_float(v[4]), __uint_as_float(v[5]));
                    mx3 = max3(mx3, __uint_as_float(v[6]), __uint_as_float(v[7]));
                }
            }
            // (scale > 0, so the maximum commutes with scaling)
            const float tile_max = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
            // lazy running maximum: move it only when the row maximum outgrows it by 2^8.  S_t(j) is
            // complete, so every earlier MMA of this tile (including P.V of tile j-1) has finished and
            // O_t may be touched.
            const bool grow = tile_max > m_used + kRescaleThreshold;
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
                const float alpha = grow ? fast_exp2(m_used - tile_max) : 1.0F;  // 2^(-inf) = 0 for a fresh row
#pragma unroll 1
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
            if (grow) m_used = tile_max;
            // exponentials, row sum, packed bf16 P written over the consumed scores
            const float neg_m = m_used == -INFINITY ? 0.0F : -m_used;
            float s0 = 0.0F, s1 = 0.0F, s2 = 0.0F, s3 = 0.0F;
#pragma unroll
            for (int c = 0; c < KT / 32; ++c) {
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const float x0 = fast_exp2(fmaf(__uint_as_float(raw[c][i]), p.scale_log2, neg_m));
                    const float x1 = fast_exp2(fmaf(__uint_as_float(raw[c][i + 1]), p.scale_log2, neg_m));
                    const float x2 = fast_exp2(fmaf(__uint_as_float(raw[c][i + 2]), p.scale_log2, neg_m));
                    const float x3 = fast_exp2(fmaf(__uint_as_float(raw[c][i + 3]), p.scale_log2, neg_m));
                    s0 += x0; s1 += x1; s2 += x2; s3 += x3;
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(x0, x1), hi = __floats2bfloat162_rn(x2, x3);
                    packed[i / 2] = *reinterpret_cast<const uint32_t*>(&lo);
                    packed[i / 2 + 1] = *reinterpret_cast<const uint32_t*>(&hi);
                }
                ptx::tmem_st_32x16(s_addr + c * 16, packed);
            }
            ptx::tmem_st_wait();
            row_sum += (s0 + s1) + (s2 + s3);
            ptx::tc_fence_before();
            ptx::mbar_arrive(ptx::smem_u32(&p_full[t]));
        }
        if (ok && nt > 0) ok = ptx::mbar_wait(ptx::smem_u32(&o_full[t]), 0, abort_flag, p.status, kCodeAttn | 4);
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
    return a.dtype == SFB_BF16 && (a.head_dim == 128 || a.head_dim == 64) && a.head_dim_value == a.head_dim &&
           (reinterpret_cast<uintptr_t>(a.q) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.key) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(a.value) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15) == 0;
}

namespace {
template <int D>
sfb_status launch_prefill(const sfb_attention_args& a, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        SFB_CUDA(cudaFuncSetAttribute(attention_prefill_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Fa<D>::kSmemBytes));
        configured = true;
    }
    CUtensorMap map_q, map_k, map_v;
    const int q_head_rows = a.q_head_rows > 0 ? a.q_head_rows : a.seq_q;
    const int kv_head_rows = a.kv_head_rows > 0 ? a.kv_head_rows : a.seq_kv;
    // (a slice that starts inside the stored sequence ends before the last head's rows do)
    const uint64_t q_rows = static_cast<uint64_t>(a.batch) * a.q_heads * q_head_rows - (q_head_rows - a.seq_q);
    const uint64_t kv_rows = static_cast<uint64_t>(a.batch) * a.kv_heads * kv_head_rows - (kv_head_rows - a.seq_kv);
    if (!encode_tensor_map_bf16_2d(&map_q, a.q, q_rows, D, QT, 64) ||
        !encode_tensor_map_bf16_2d(&map_k, a.key, kv_rows, D, KT, 64) ||
        !encode_tensor_map_bf16_2d(&map_v, a.value, kv_rows, D, KT, 64))
        return SFB_CUDA_ERROR;
    FaParams p{};
    p.out = static_cast<bf16*>(a.out);
    p.batch = a.batch; p.q_heads = a.q_heads; p.kv_heads = a.kv_heads; p.seq_q = a.seq_q; p.seq_kv = a.seq_kv;
    p.q_head_rows = q_head_rows; p.kv_head_rows = kv_head_rows;
    p.causal = a.causal; p.token_major = a.token_major;
    p.scale_log2 = a.scale * 1.4426950408889634F;
    p.status = device_status_word();
    const int q_blocks = ceil_div(a.seq_q, 2 * QT);
    const int grid = a.batch * a.q_heads * q_blocks;
    attention_prefill_tcgen05_kernel<D><<<grid, kThreads, Fa<D>::kSmemBytes, stream>>>(map_q, map_k, map_v, p);
    return check_launch("attention_prefill_tcgen05");
}
}  // namespace

sfb_status attention_prefill_tcgen05(const sfb_attention_args& a, cudaStream_t stream) {
    return a.head_dim == 64 ? launch_prefill<64>(a, stream) : launch_prefill<128>(a, stream);
}

}  // namespace sfb
