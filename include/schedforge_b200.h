/*
 * schedforge_b200 — C ABI of the B200 (sm_100a) decoder-layer executor.
 *
 * Two groups of entry points live in libschedforge_b200.so:
 *
 *   1. Kernel entry points (`sfb_k_*`): one call = one (or a fixed short chain of) CUDA
 *      kernel launch(es) on the caller's stream.  All pointers are DEVICE pointers, shapes
 *      are int32 (the reference uses `int`), nothing is allocated, nothing synchronises.
 *      Each replaces one CPU function of the reference's decoder hot path; the reference
 *      location is cited beside each declaration (paths are relative to the reference
 *      repository root).
 *
 *   2. Plan entry points (`sfb_decoder_*`, `sfb_attention_*`, `sfb_paged_*`, `sfb_moe_*`,
 *      `sfb_import_*`): the reference's public C++ API for this path restated as a C ABI
 *      with HOST buffers (float32, the reference's `std::vector<float>` contents).  They
 *      are thin wrappers around the C++20 host runtime in this library, which owns device
 *      memory, builds the plan once and runs the kernels of group 1.
 *
 * Every function returns an `sfb_status`.  SFB_INVALID_ARGUMENT corresponds to the
 * reference throwing std::invalid_argument for the same condition, SFB_RUNTIME_ERROR to
 * std::runtime_error.  `sfb_last_error()` returns the message of the calling thread's
 * last failure.  The library has no CPU fallback: without a CUDA device every compute
 * entry point fails with SFB_CUDA_ERROR.
 *
 * The only C ABIs in the reference are its JIT/AOT matmul symbol
 * `schedforge_matmul_v1(A, B, bias, residual, C, M, N, K)` (src/llvm_backend.cpp:39-40,
 * src/aot_runtime.cpp:23-24) and `schedforge_fused_attention(q, k, v, out, row_begin,
 * row_end)` (src/attention_llvm_backend.cpp:36-37): raw pointers plus integer extents.
 * This header keeps that convention and adds a status return.
 */
#ifndef SCHEDFORGE_B200_H
#define SCHEDFORGE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum sfb_status {
    SFB_OK = 0,
    SFB_INVALID_ARGUMENT = -1, /* reference: std::invalid_argument */
    SFB_RUNTIME_ERROR = -2,    /* reference: std::runtime_error    */
    SFB_CUDA_ERROR = -3,       /* a CUDA runtime/driver call failed, or no device */
    SFB_UNSUPPORTED = -4,      /* shape/dtype outside what the kernels cover */
    SFB_DEVICE_TIMEOUT = -5    /* a bounded device-side wait gave up (status word set) */
} sfb_status;

typedef enum sfb_dtype { SFB_F32 = 0, SFB_BF16 = 1 } sfb_dtype;

typedef void* sfb_stream; /* cudaStream_t */

const char* sfb_last_error(void);
const char* sfb_version(void);
/* Number of kernels this library has launched in this process (for launch accounting). */
uint64_t sfb_launch_count(void);
/* Reads and clears the device status word that bounded waits set when they give up.
 * 0 = no device-side wait timed out since the last call. */
sfb_status sfb_device_status(uint32_t* status_word);

/* ======================================================================================
 * 1. Kernel entry points (device pointers)
 * ====================================================================================== */

/* y[r,:] = x[r,:] * (1/sqrt(mean(x[r,:]^2) + eps)) * weight[:].
 * f32: sum of squares in double, (x*inv)*w order.  weight is always float32.
 * Replaces rms_norm, src/decoder_compiler.cpp:41-62. */
sfb_status sfb_k_rms_norm(const void* x, const float* weight, void* y, int rows, int width,
                          float epsilon, sfb_dtype dtype, sfb_stream stream);

/* Elementwise z = x + y.  Replaces add, src/decoder_compiler.cpp:176-181. */
sfb_status sfb_k_add(const void* x, const void* y, void* z, int64_t count, sfb_dtype dtype,
                     sfb_stream stream);

/* out[r,j] = silu(gate_up[r,j]) * gate_up[r, I+j], gate = first I columns.
 * Replaces swiglu, src/decoder_compiler.cpp:183-194. */
sfb_status sfb_k_swiglu(const void* gate_up, void* out, int rows, int intermediate,
                        sfb_dtype dtype, sfb_stream stream);

/* float32 <-> bfloat16 (round to nearest even, as convert_to_bf16, src/compiler.cpp:34-43). */
sfb_status sfb_k_convert(const void* src, sfb_dtype src_dtype, void* dst, sfb_dtype dst_dtype,
                         int64_t count, sfb_stream stream);

/* C[m,n] = A[m,k] . B[k,n], float32 row-major, one FMA chain per output over ascending k:
 * the rounding sequence of the reference's native GEMM (execute -> register_kernel_16/8,
 * src/runtime.cpp:581-626, 278-370), so results are bit-identical to it. */
sfb_status sfb_k_gemm_f32(const float* a, const float* b, float* c, int m, int n, int k,
                          sfb_stream stream);

typedef enum sfb_gemm_epilogue {
    SFB_EPI_STORE = 0,      /* out[m,n] = acc                                              */
    SFB_EPI_RESIDUAL = 1,   /* out[m,n] = acc + residual[m,n]                               */
    SFB_EPI_SWIGLU = 2,     /* out[m,n/2]: weight rows come in blocks of 2*swiglu_block:    */
                            /* swiglu_block gate rows then swiglu_block up rows;            */
                            /* out = silu(gate) * up                                        */
    SFB_EPI_ROPE_SPLIT = 3  /* n = hidden + 2*kv: rotary on Q,K and scatter to head-major   */
} sfb_gemm_epilogue;

#define SFB_MAX_PEERS 8

typedef enum sfb_gemm_backend {
    SFB_GEMM_AUTO = 0,
    SFB_GEMM_SIMT = 1,     /* CUDA-core tiles, any shape                                   */
    SFB_GEMM_TCGEN05 = 2   /* tcgen05.mma + TMEM + TMA, needs k % 8 == 0                   */
} sfb_gemm_backend;

/* bf16 GEMM with fp32 accumulation.  A is [m,k] row-major bf16.  The weight is passed
 * TRANSPOSED: bt is [n,k] row-major bf16 (k contiguous), i.e. y = x . W with W = bt^T.
 * Grouped mode (group_offsets != NULL): rows [group_offsets[g], group_offsets[g+1]) of A
 * use weight slab g (bt + g*n*k); groups = number of slabs.  Replaces the four decoder
 * GEMMs (execute calls at src/decoder_compiler.cpp:230,252,272,276) and the variable-M
 * expert GEMMs (execute_loop_kernel / compute_task, src/moe_compiler.cpp:64-155). */
typedef struct sfb_gemm_args {
    const void* a;
    const void* bt;
    void* out;              /* bf16 unless out_f32 != 0                                    */
    int m, n, k;
    int epilogue;           /* sfb_gemm_epilogue                                           */
    int backend;            /* sfb_gemm_backend                                            */
    int out_f32;
    const void* residual;   /* SFB_EPI_RESIDUAL: [m,n] bf16                                */
    int swiglu_block;       /* SFB_EPI_SWIGLU: gate/up interleave block in weight rows     */
    /* SFB_EPI_ROPE_SPLIT */
    void* q;                /* [batch, q_heads, seq, head_dim] bf16                        */
    void* key;              /* [batch, kv_heads, seq, head_dim]                            */
    void* value;            /* [batch, kv_heads, seq, head_dim]                            */
    const float* rope_cos;  /* [seq, head_dim/2]                                           */
    const float* rope_sin;
    int batch, seq, q_heads, kv_heads, head_dim;
    /* grouped mode */
    const int* group_offsets; /* device int32[groups+1], NULL for a dense GEMM             */
    int groups;
    void* tile_table;       /* grouped tcgen05: device scratch, int32[4*(m/128 + groups + 1)] */
    /* optional scratch for GEMMs with m <= 128 (decode): with it the tcgen05 kernel gives every
     * SM an equal share of the K blocks and sums partial tiles here.  Device memory, 16-byte
     * aligned, at least sfb_gemm_stream_workspace_bytes(n) bytes, ZERO-FILLED before its first
     * use; every call leaves it zero-filled again.  NULL = whole tiles per SM. */
    void* split_workspace;
    size_t split_workspace_bytes;
    /* bt_tiled != 0: bt holds the weight in 64x64 blocks (sfb_k_tile_weight_bf16) so that a
     * weight-streaming GEMM reads 8 KB contiguous runs; tcgen05 backend, dense mode only */
    int bt_tiled;
    /* SFB_EPI_STORE / SFB_EPI_RESIDUAL with bf16 output, tcgen05 backend: every finished piece of
     * the output is also stored to these peer_count buffers (same [m,n] layout; memory of other GPUs
     * mapped into this process), so that a sum all-reduce of the sharded layer moves its data under
     * the GEMM; sfb_k_peer_allreduce_finish completes it. */
    void* peer_out[SFB_MAX_PEERS - 1];
    int peer_count;
    /* Two-shot form (scatter_rows > 0; SFB_EPI_STORE / SFB_EPI_RESIDUAL, bf16, tcgen05): row r belongs to rank
     * r / scatter_rows and is stored ONLY to scatter_out[that rank] at row r % scatter_rows (layout
     * [scatter_rows, n]; the entry of this rank points into its own memory); `out` is not written.
     * sfb_k_peer_reduce_gather on the owner completes the sum. */
    void* scatter_out[SFB_MAX_PEERS];
    int scatter_rows;
    /* SFB_EPI_ROPE_SPLIT on a row chunk: row r of A is token (r + rope_row_offset) of the
     * [batch, seq] grid (q/key/value stay the full tensors) */
    int rope_row_offset;
    /* weight-only INT8 (m <= 128, dense, tcgen05): bt_scales != NULL says that bt holds int8 values in
     * 64x64 blocks (sfb_k_quantize_weight_int8) and bt_scales one fp32 factor per output column,
     * padded with anything up to a multiple of 128 entries; y = (x . q^T) * scale, then the epilogue.
     * Follows quantize_matmul_weights / quantized_invoke, src/next_milestones.cpp:611-637, 50-69. */
    const float* bt_scales;
    /* RMSNorm folded into the GEMM (tcgen05 backend, dense mode).  The caller has multiplied the norm weight
     * into the weight (bt[n, k] *= norm_weight[k]) and passes A un-normalised; row r of the accumulator is
     * multiplied by 1 / sqrt(ss[r] / k + rms_epsilon) before the epilogue, which is rms_norm
     * (src/decoder_compiler.cpp:41-62) moved behind the product.  row_ss: device memory, one sum of squares
     * per row of A: float32, or with row_ss_fixed != 0 the unsigned 64-bit fixed-point sums (24 fraction
     * bits) that ss_out of the producing GEMM left.  NULL = no scaling. */
    const void* row_ss;
    int row_ss_fixed;
    float rms_epsilon;
    /* SFB_EPI_STORE / SFB_EPI_RESIDUAL with bf16 output (tcgen05): the kernel also adds the squares of the values
     * it stored to ss_out[row], unsigned 64-bit fixed point with 24 fraction bits (integer atomics: the total
     * does not depend on the order in which the tiles finish).  The caller zero-fills it before the launch
     * (or lets an earlier GEMM do it, see clear).  The next GEMM takes it as row_ss.  NULL = not collected. */
    void* ss_out;
    /* clear != NULL: this launch zero-fills clear_bytes bytes (8-byte aligned, a multiple of 8) after it has
     * waited for the kernels before it: how a chain of launches resets the sums a later GEMM adds to. */
    void* clear;
    size_t clear_bytes;
    /* owner_flags != NULL (tcgen05, dense, more than 128 rows): A is being all-gathered while the GEMM runs.  Rows
     * [o * owner_rows, (o + 1) * owner_rows) (owner_rows a multiple of 128) may be read once owner_flags[o] has reached
     * owner_epoch (device words that another GPU or a copy engine writes after the rows, and after their row_ss
     * entries); the rows of owner_self are complete at launch and their tiles are visited first.  The wait is
     * bounded; when it gives up bit 0x100 of sfb_device_status is set and the kernel drains. */
    const uint32_t* owner_flags;
    uint32_t owner_epoch;
    int owner_rows, owner_self;
    /* SFB_EPI_ROPE_SPLIT of a decode step (tcgen05): kv_k_pool != NULL also writes the rotated key and the
     * value of token t of sequence b into the paged cache at position kv_position + t (block
     * kv_table[b * kv_max_blocks + position / kv_block_tokens], pool layout of sfb_decode_args).  A position
     * past the table or a block id outside [0, kv_num_blocks) is skipped and sets bit 0x200 of
     * sfb_device_status.  This is the copy loop of append_paged_kv (src/next_milestones.cpp:502-522) done where
     * K and V are produced.  (A step at position p passes rope_cos / rope_sin advanced by p rows.) */
    void* kv_k_pool;
    void* kv_v_pool;
    const int* kv_table;
    int kv_position, kv_block_tokens, kv_max_blocks, kv_num_blocks;
} sfb_gemm_args;

sfb_status sfb_k_gemm_bf16(const sfb_gemm_args* args, sfb_stream stream);
size_t sfb_gemm_stream_workspace_bytes(int n);

/* dst[r, :] = bf16(src[r, :]) and ss[r] = sum of squares of the rounded row: the float32 -> bf16 conversion of
 * the layer input that also prepares the folded RMSNorm of the first GEMM (row_ss with one slot per row).
 * sfb_k_row_sumsq computes ss alone from a bf16 tensor (after an all-reduce through a library). */
sfb_status sfb_k_convert_rows_sumsq(const float* src, void* dst_bf16, float* ss, int rows, int width, sfb_stream stream);
sfb_status sfb_k_row_sumsq(const void* x_bf16, float* ss, int rows, int width, sfb_stream stream);

/* Blocked weight layout for decode-shaped (few rows, HBM-bound) GEMMs.  The [n,k] row-major
 * bf16 weight is cut into 64x64 blocks; block (j, b) = rows [64j, 64j+64) x columns
 * [64b, 64b+64), zero padded at the edges, stored row-major (64 rows of 128 bytes) at element
 * offset (j * ceil(k/64) + b) * 4096.  sfb_tiled_weight_elems gives the element count of the
 * blocked copy.  src and dst must not overlap.  No counterpart in the reference, whose CPU
 * packing is the plain transpose of pack_transposed (src/decoder_compiler.cpp:57-66). */
int64_t sfb_tiled_weight_elems(int n, int k);
/* Per-output-channel symmetric INT8 quantization of a [n,k] bf16 weight (quantize_matmul_weights,
 * src/next_milestones.cpp:611-637: scale = max|w| / 127 or 1 for an all-zero row, q = round-half-away(w / scale)
 * clamped to [-127, 127]) written in the blocked layout of sfb_k_tile_weight_bf16 with one byte per
 * element (sfb_tiled_weight_elems(n, k) bytes); scales: n floats.  sfb_k_dequantize_weight_int8 writes
 * q * scale back as a [n,k] row-major bf16 weight. */
sfb_status sfb_k_quantize_weight_int8(const void* bt, void* q_tiled, float* scales, int n, int k, sfb_stream stream);
sfb_status sfb_k_dequantize_weight_int8(const void* q_tiled, const float* scales, void* bt, int n, int k,
                                        sfb_stream stream);
sfb_status sfb_k_tile_weight_bf16(const void* bt, void* tiled, int n, int k, sfb_stream stream);

/* cos/sin tables for interleaved-pair rotary embedding, computed on the HOST with the
 * same powf/cosf/sinf calls as apply_rope, src/decoder_compiler.cpp:96-114:
 * freq = powf(theta, -float(d)/float(dim)), angle = float(t)*freq for even d.
 * cos_out/sin_out are HOST float32 [seq, dim/2]. */
sfb_status sfb_rope_table(int seq, int head_dim, float theta, float* cos_out, float* sin_out);

/* fused[T, hidden+2*kv] -> Q [B,Hq,S,D], K,V [B,Hkv,S,D] with rotary on Q and K; token
 * positions restart at 0 for every batch element.  Replaces split_qkv + apply_rope,
 * src/decoder_compiler.cpp:96-148. */
sfb_status sfb_k_rope_split(const void* fused, void* q, void* key, void* value,
                            const float* rope_cos, const float* rope_sin, int batch, int seq,
                            int q_heads, int kv_heads, int head_dim, sfb_dtype dtype,
                            sfb_stream stream);

/* Exact causal/non-causal GQA softmax attention, online softmax over KV tiles.
 * q [B,Hq,Sq,D], key [B,Hkv,Sk,D], value [B,Hkv,Sk,Dv].  Key j is visible to query i iff
 * !causal or j <= Sk - Sq + i; kv_head = head*Hkv/Hq; scale 0 means 1/sqrt(D).
 * out is [B,Hq,Sq,Dv] (token_major == 0) or [B*Sq, Hq*Dv] (token_major != 0, the layout
 * merge_attention produces, src/decoder_compiler.cpp:150-174).
 * Replaces execute_attention -> execute_streaming (IO-aware branch),
 * src/attention_compiler.cpp:879-885, 286-376. */
typedef struct sfb_attention_args {
    const void* q;
    const void* key;
    const void* value;
    void* out;
    int batch, q_heads, kv_heads, seq_q, seq_kv, head_dim, head_dim_value;
    int causal;
    float scale;
    int token_major;
    int dtype;    /* sfb_dtype of q/key/value/out */
    int backend;  /* 0 auto, 1 SIMT, 2 tcgen05 */
    /* A slice of longer sequences (tcgen05 kernel only; 0 = dense): rows between two heads of q
     * and of key/value in memory, when seq_q / seq_kv cover only part of the stored sequence.  With
     * causal masking query i of the slice is row seq_kv - seq_q + i of the sequence, so a prefill can
     * run in row chunks: chunk [r0, r1) passes q + r0 rows, seq_q = r1 - r0, seq_kv = r1. */
    int q_head_rows, kv_head_rows;
} sfb_attention_args;

sfb_status sfb_k_attention_prefill(const sfb_attention_args* args, sfb_stream stream);

/* Split-KV decode over a paged KV cache, one new query token per sequence.
 * Pool layout: k_pool/v_pool [num_blocks][kv_heads][block_tokens][dim] (the reference's
 * [page][batch][kv_head][page_tokens][dim], src/next_milestones.cpp:29-33, with the
 * per-sequence caches of a batch folded into one pool: batch == 1 per page).
 * block_table[b*max_blocks + i] = physical block of logical block i of sequence b;
 * context_len[b] = live tokens.  Each (sequence, kv head, split) block writes a partial
 * (max, sum, numerator) into `partials`; a second kernel merges the splits with the
 * log-sum-exp rule (merge_online, src/attention_compiler.cpp:132-145; empty splits are
 * skipped).  Replaces execute_decode_attention / execute_paged_decode_attention,
 * src/attention_compiler.cpp:968-1007, src/next_milestones.cpp:583-609, 137-184.
 * `partials` needs sfb_attention_decode_workspace() bytes.  splits <= 0 picks a value.
 * A context_len[b] beyond what the table covers (max_blocks * block_tokens, or max_context) is
 * cut to that bound and a block id outside [0, num_blocks) is skipped; either sets bit 0x200 of
 * sfb_device_status instead of reading out of bounds. */
typedef struct sfb_decode_args {
    const void* q;          /* [batch, q_heads, head_dim]                                  */
    const void* k_pool;
    const void* v_pool;
    const int* block_table; /* int32 [batch, max_blocks]                                   */
    const int* context_len; /* int32 [batch]                                               */
    void* out;              /* [batch, q_heads, head_dim_value]                            */
    void* partials;
    int batch, q_heads, kv_heads, head_dim, head_dim_value;
    int block_tokens, max_blocks, num_blocks;
    int max_context;        /* upper bound of context_len, sizes the split count           */
    int splits;
    float scale;
    int dtype;
    int uniform_context;    /* > 0: every sequence holds this many tokens and context_len is not read (may be
                               NULL): the case of a batch that decodes in lock step, whose length the host knows */
} sfb_decode_args;

size_t sfb_attention_decode_workspace(int batch, int q_heads, int head_dim_value, int splits);
int sfb_attention_decode_default_splits(int batch, int kv_heads, int max_context);
sfb_status sfb_k_attention_decode_paged(const sfb_decode_args* args, sfb_stream stream);

/* Writes `tokens` new tokens per sequence into the paged pool.  new_k/new_v are
 * [batch, kv_heads, tokens, dim]; the token at logical position start_len[b] + t goes to
 * block block_table[b][pos / block_tokens], slot pos % block_tokens.  start_len and block_table
 * live on the device and may have been written by another kernel, so the kernel checks them: a
 * position past the table (pos / block_tokens >= max_blocks) or a block id outside [0, num_blocks)
 * is skipped and bit 0x200 of sfb_device_status is set (num_blocks <= 0 switches the block check off).
 * Replaces the copy loop of append_paged_kv, src/next_milestones.cpp:502-522. */
sfb_status sfb_k_paged_kv_append(const void* new_k, const void* new_v, void* k_pool, void* v_pool,
                                 const int* block_table, const int* start_len, int batch,
                                 int kv_heads, int tokens, int head_dim, int head_dim_value,
                                 int block_tokens, int max_blocks, int num_blocks, sfb_dtype dtype,
                                 sfb_stream stream);

/* Paged pool -> contiguous [batch, kv_heads, length, dim] (all sequences `length` long).
 * Replaces gather_paged_kv, src/next_milestones.cpp:552-581. */
sfb_status sfb_k_paged_kv_gather(const void* k_pool, const void* v_pool, void* keys, void* values,
                                 const int* block_table, int batch, int kv_heads, int length,
                                 int head_dim, int head_dim_value, int block_tokens,
                                 int max_blocks, sfb_dtype dtype, sfb_stream stream);

/* Router: logits[t,e] = sum_f x[t,f]*router[f,e] accumulated sequentially in float32
 * (multiply rounded, then add rounded, f ascending) + optional bias[e]; softmax
 * numerators p = exp(logit - max); top-k by descending p (ties: lower expert id);
 * weights (p/den)/sum_selected(p/den); per-expert histogram.  router is float32 [H,E].
 * counts must be zeroed by the caller's stream before the call (the entry point does it).
 * Replaces route_topk, src/moe_compiler.cpp:412-455.  Limits: experts <= 64, top_k <= 8. */
sfb_status sfb_k_moe_route(const void* x, sfb_dtype x_dtype, const float* router,
                           const float* bias, int tokens, int hidden, int experts, int top_k,
                           int* expert_ids, float* expert_weights, int* counts,
                           sfb_stream stream);

/* Exclusive prefix sum of counts -> offsets[E+1], then the stable counting-sort scatter in
 * (token, slot) order: dest = offsets[e] + rank of the assignment among earlier
 * assignments to e.  Writes values[dest,:] = x[token,:], token_ids, route_slots,
 * routing_weights, and dest_of[token*k+slot] = dest.  Deterministic (no atomics).
 * Replaces the prefix loop and dispatch_tokens, src/moe_compiler.cpp:496-528.
 * scratch: device int32[(ceil(tokens*top_k/1024) + 1) * experts]. */
sfb_status sfb_k_moe_dispatch(const void* x, sfb_dtype dtype, const int* expert_ids,
                              const float* expert_weights, const int* counts, int tokens,
                              int hidden, int experts, int top_k, void* values, int* offsets,
                              int* token_ids, int* route_slots, float* routing_weights,
                              int* dest_of, int* scratch, sfb_stream stream);
size_t sfb_moe_dispatch_scratch_bytes(int tokens, int experts, int top_k);

/* Same dispatch for callers that must not allocate device memory (a host process whose memory
 * pool owns every byte, a plugin under a "no cudaMalloc after start-up" rule, a latency-critical
 * loop): the scratch is a 66 816-byte array that lives inside the library image on every GPU that
 * loads it, so the call takes no scratch pointer and never calls cudaMalloc/cudaFree.
 * This entry point has no counterpart in the reference.
 *   - limit: tokens * top_k <= 262144 and experts <= 64, else SFB_UNSUPPORTED;
 *   - the first call on each device looks up the array's device address (with that device
 *     current); make that first call before starting any stream capture;
 *   - all calls on one GPU share the array: two calls whose kernels can overlap on the GPU
 *     (different streams, no dependency) race on it; issue them on one stream or order them;
 *   - the array keeps the last call's contents; nothing in it needs clearing between calls. */
sfb_status sfb_k_moe_dispatch_static(const void* x, sfb_dtype dtype, const int* expert_ids,
                                     const float* expert_weights, const int* counts, int tokens,
                                     int hidden, int experts, int top_k, void* values, int* offsets,
                                     int* token_ids, int* route_slots, float* routing_weights,
                                     int* dest_of, sfb_stream stream);

/* out[t,:] = (residual ? residual[t,:] : 0) + sum over the token's assignments, in
 * ascending dispatched position (= the reference's expert-major accumulation order), of
 * routing_weights[pos] * y[pos,:].
 * Replaces the weighted combine, src/moe_compiler.cpp:219-226 (+ the FFN residual add,
 * src/decoder_compiler.cpp:285). */
sfb_status sfb_k_moe_combine(const void* y, const int* dest_of, const float* routing_weights,
                             const void* residual, void* out, int tokens, int hidden, int top_k,
                             sfb_dtype dtype, sfb_stream stream);

/* ======================================================================================
 * 2. Plan entry points (host float32 buffers; mirror of the reference's C++ API)
 * ====================================================================================== */

/* DecoderConfig, include/schedforge/decoder_compiler.h:17-32. */
typedef struct sfb_decoder_config {
    int batch, sequence, hidden, intermediate, query_heads, kv_heads, head_dim;
    float rms_epsilon, rope_theta;
    int causal;
    int ffn_moe;           /* DecoderFFNKind: 0 Dense, 1 MoE */
    int experts, top_k;
    int context_sequence;  /* > 0: decode over cached K/V of this length */
} sfb_decoder_config;

/* DecoderData, include/schedforge/decoder_compiler.h:34-49 (+ MoeData, moe_compiler.h:79-85).
 * All weights are [in, out] row-major float32, y = x . W.  Unused members may be NULL.
 * router_bias has no counterpart in the reference (its router has no bias term). */
typedef struct sfb_decoder_data {
    const float* rms1_weight;
    const float* query_weight;
    const float* key_weight;
    const float* value_weight;
    const float* output_weight;
    const float* rms2_weight;
    const float* gate_weight;
    const float* up_weight;
    const float* down_weight;
    const float* router_weight; /* [H, E]   */
    const float* router_bias;   /* [E]      */
    const float* w1;            /* [E, H, I] */
    const float* w3;            /* [E, H, I] */
    const float* w2;            /* [E, I, H] */
    const float* cached_key;    /* [B, Hkv, context, D] */
    const float* cached_value;
} sfb_decoder_data;

/* DecoderCompileOptions + DecoderPlanPolicy, include/schedforge/decoder_compiler.h:55-65,132-138,
 * reduced to what applies to a GPU plan, plus the sharding this build adds. */
typedef struct sfb_compile_options {
    int dtype;            /* sfb_dtype: SFB_F32 = exact-order fp32 path, SFB_BF16 = tensor cores */
    int token_major_attention; /* DecoderIntermediateLayout::TokenMajor (1) or HeadMajor (0) */
    int fuse_epilogues;   /* bf16: RoPE/residual/SwiGLU inside the GEMM epilogues (1) or as
                             separate kernels (0, the "materialize" policy) */
    int gemm_backend;     /* sfb_gemm_backend */
    int attention_backend;
    int page_tokens;      /* decode: KV block size of the paged cache (0 -> 16) */
    int tp_rank, tp_size; /* tensor parallel shard of this plan (heads / FFN columns) */
    int seed_block_table; /* decode: != 0 permutes the physical block order with this seed */
    int no_workspace_reuse; /* != 0: every intermediate keeps its own bytes (DecoderPlanPolicy::
                               reuse_workspace = false), so tests can read any of them back */
    int no_pipeline;      /* != 0: sfb_decoder_execute copies the whole input, runs, copies the whole output;
                             0: dense bf16 prefill plans overlap the host copies of one row chunk with the
                             computation of another (chunks of whole sequences, or, for causal head_dim-128
                             plans of one shard, row ranges sized to whole rounds of GEMM tiles) */
    int append_new_token; /* decode plans (sequence == 1, context_sequence > 0).  0 = the reference's
                             semantics (src/decoder_compiler.cpp:238-241): RoPE position 0, the new token's
                             K/V are dropped, attention sees the cached context only.  != 0 = a real
                             autoregressive step: RoPE at position context_sequence, K/V of the new token
                             appended to the paged cache (append_paged_kv, src/next_milestones.cpp:486-524)
                             and attention over context_sequence + 1 keys.  sfb_decoder_execute can be run
                             again (it appends at the current cache length without advancing it);
                             sfb_decoder_step advances. */
    int weight_int8;      /* != 0 (bf16 plans, dense FFN): per-output-channel symmetric INT8 weights as
                             quantize_decoder_weights / execute_quantized_decoder_layer
                             (src/next_milestones.cpp:660-697).  Plans of at most 128 rows keep the four
                             projections as int8 and stream half the bytes; larger plans (compute bound)
                             multiply by the dequantised q * scale weights in bf16.  The quantizer sees the
                             bf16-rounded weights. */
    int kv_capacity;      /* decode plans with append_new_token: tokens the paged cache can hold (0 -> context_sequence
                             + 1); sfb_decoder_step appends one token per call until the cache is full */
    int norm_fusion;      /* > 0: bf16 plans with fused epilogues fold both RMSNorms into the GEMM that follows (norm
                             weight multiplied into the packed weight, 1/rms applied to the accumulator rows, sums of
                             squares taken where the rows are produced); < 0: stand-alone RMSNorm kernels; 0: folded
                             for sharded plans (tp_size > 1), where the stand-alone norms are replicated work that
                             does not shrink with the rank count, stand-alone for a single shard, where they measured
                             faster on B200 */
    int local_expert_weights; /* MoE plans with tp_size > 1: != 0 says that w1 / w3 / w2 of sfb_decoder_data hold
                             only this rank's experts/tp_size experts (expert tp_rank * experts/tp_size first), so
                             that a rank never has to materialise the other ranks' expert weights on its host;
                             0 = the full [experts, ...] arrays, of which the rank takes its slice. */
    int fixed_order;      /* != 0: the weight-streaming GEMMs of plans of at most 128 rows never cut an output tile
                             between CTAs, so no fp32 partial sums meet at L2 in arrival order: the plan's output is
                             bitwise the same from run to run.  Slower: the tiles left over after the last full
                             round of the SMs are then computed by one CTA each.  0: left-over tiles are shared. */
} sfb_compile_options;

/* DecoderBenchmarkResult, include/schedforge/decoder_compiler.h:119-130 (device-event times). */
typedef struct sfb_decoder_result {
    double milliseconds;
    double attention_milliseconds;
    double projection_milliseconds;
    double norm_rope_milliseconds;
    double ffn_milliseconds;
    double residual_milliseconds;
    double h2d_milliseconds;
    double d2h_milliseconds;
    double tokens_per_second;
    uint64_t kernel_launches;
} sfb_decoder_result;

/* StableHLOImporter::importText + DecoderFusionPass::run, src/graph_compiler.cpp:1129-1198,
 * src/decoder_compiler.cpp:380-410. */
typedef struct sfb_graph_summary {
    int operations, values, inputs, matmuls;
    int fused_qkv, fused_gate_up, fused_rope;
} sfb_graph_summary;

sfb_status sfb_import_stablehlo(const char* text, sfb_graph_summary* summary);
/* graph dump ("graph @model { ... }") of the imported text into buffer. */
sfb_status sfb_import_stablehlo_dump(const char* text, char* buffer, size_t capacity);

typedef struct sfb_decoder_plan sfb_decoder_plan;

/* DecoderCompiler::compile, src/decoder_compiler.cpp:518-620: validates the configuration,
 * runs the fusion pass on the imported graph (NULL/empty text = the canonical graph) and
 * fails with SFB_INVALID_ARGUMENT ("decoder graph is missing required fusion patterns") when
 * a pattern is missing, packs Wq|Wk|Wv and Wgate|Wup, uploads every weight once and lays
 * all activations out in one device workspace. */
sfb_status sfb_decoder_compile(const sfb_decoder_config* config, const sfb_decoder_data* data,
                               const char* stablehlo_text, const sfb_compile_options* options,
                               sfb_decoder_plan** plan);
void sfb_decoder_destroy(sfb_decoder_plan* plan);

/* execute_decoder_layer, src/decoder_compiler.cpp:675-692, one repetition: copies
 * input [T,H] float32 from host, runs the layer, copies output [T,H] float32 back.
 * routing trace (optional, MoE): expert_ids/expert_weights [T*k] and counts [E] replace the
 * router, like DecoderData::routing_trace (include/schedforge/decoder_compiler.h:48).
 * Dense bf16 prefill plans run the pass in row chunks whose host copies overlap the kernels of other chunks (see
 * no_pipeline of sfb_compile_options); the numbers equal the one-shot pass.  result == NULL skips the stage marks
 * between the kernels, which cost the chunked pass a few per cent beside saturated PCIe traffic. */
sfb_status sfb_decoder_execute(sfb_decoder_plan* plan, const float* input, float* output,
                               const int* trace_expert_ids, const float* trace_expert_weights,
                               const int* trace_counts, sfb_decoder_result* result);
/* The row chunks of that pipelined pass for a causal head_dim-128 plan of one shard with `rows` tokens and `hidden`
 * columns on a device of sm_count SMs, in blocks of 128 rows (host arithmetic, no device needed): returns the number
 * of chunks and fills up to `capacity` of them; 0 = the shape is chunked by whole sequences or not at all.  A chunk
 * is a multiple of the row blocks that fill one round of the SMs with the 128 x 256 output tiles of the O and Down
 * GEMMs, 4 blocks at the head and 4 + remainder at the tail (rows 8192, hidden 4096, 148 SMs: 4 9 18 18 9 6). */
int sfb_decoder_row_chunks(int rows, int hidden, int sm_count, int* blocks, int capacity);

/* execute_decoder_layer for a rank of a sharded plan that owns rows [row_begin, row_begin + row_count) of the
 * [T,H] input: only these rows cross this rank's PCIe link (input_rows in, the same rows of the output out).
 * The ranks' ranges must be disjoint and cover all rows; the plan's all-reduce hook gathers the input (each
 * row is zero on every other rank, so the sum is exact).  bf16 plans with a hook; the full range works on
 * any plan and equals sfb_decoder_execute without the row-chunk pipeline.  No counterpart in the reference,
 * which is a single-process library. */
sfb_status sfb_decoder_execute_rows(sfb_decoder_plan* plan, const float* input_rows, float* output_rows,
                                    int row_begin, int row_count, sfb_decoder_result* result);

/* Autoregressive decode loop on a plan compiled with append_new_token (sequence == 1, context_sequence > 0):
 * one call = one token per sequence.  The step rotates the token at position `length`, appends its K/V to the
 * paged cache there, attends over length + 1 keys and then advances the length; a token that opens a page takes
 * it from the BACK of the free list, like append_paged_kv (src/next_milestones.cpp:486-524).  The cache has ONE
 * page table and ONE length for the whole batch, like the reference's PagedKVCache.  SFB_INVALID_ARGUMENT
 * "paged KV capacity exceeded" when the cache (kv_capacity of sfb_compile_options) is full.
 * sfb_decoder_execute on such a plan runs the same pass WITHOUT advancing (it can be repeated).
 * sfb_decoder_kv_info: info[0..3] = length, pages in the table, free pages, total pages (as sfb_paged_info).
 * sfb_decoder_kv_truncate / sfb_decoder_kv_release: truncate_paged_kv / release_paged_kv_pages
 * (src/next_milestones.cpp:526-550) with the same guards and messages. */
sfb_status sfb_decoder_step(sfb_decoder_plan* plan, const float* input, float* output, sfb_decoder_result* result);
sfb_status sfb_decoder_kv_info(const sfb_decoder_plan* plan, int* info, int* page_table, int table_capacity,
                               int* free_pages, int free_capacity);
sfb_status sfb_decoder_kv_truncate(sfb_decoder_plan* plan, int new_length);
sfb_status sfb_decoder_kv_release(sfb_decoder_plan* plan, const int* pages, int count);

/* The same layer with the input already resident (last sfb_decoder_execute /
 * sfb_decoder_upload_input) and the output left on the device: kernels only. */
sfb_status sfb_decoder_upload_input(sfb_decoder_plan* plan, const float* input);
sfb_status sfb_decoder_execute_resident(sfb_decoder_plan* plan, sfb_stream stream);
sfb_status sfb_decoder_download_output(sfb_decoder_plan* plan, float* output);

/* ExecutablePlanOptimizer::optimize (include/schedforge/decoder_compiler.h:140-178,
 * src/decoder_compiler.cpp:726-861) on the GPU: 16 policies (fused or materialised epilogues x
 * tensor-core or CUDA-core GEMM family x tensor-core or CUDA-core attention x workspace reuse) ranked
 * analytically; the baseline (base_options) and the best-ranked measurement_budget candidates are
 * measured with three warm-up passes and `repetitions` timed passes (median) on `input` (host
 * float32 [T,H]); a faster winner is confirmed by three interleaved baseline/winner measurements.
 * *plan receives the winning plan (the baseline when nothing beat it).  candidates_out (optional,
 * `capacity` entries) receives the baseline followed by the ranked candidates. */
typedef struct sfb_plan_cost {
    double measured_milliseconds;
    double analytical_score;
    size_t workspace_bytes;
    size_t materialization_bytes;
    int measured;
} sfb_plan_cost;
typedef struct sfb_plan_candidate {
    sfb_compile_options options;
    sfb_plan_cost cost;
} sfb_plan_candidate;
typedef struct sfb_optimization_result {
    sfb_plan_cost baseline;
    sfb_plan_cost winner;
    sfb_compile_options winner_options;
    int candidates;
    int hardware_measurements;
    double speedup;
} sfb_optimization_result;
sfb_status sfb_decoder_optimize(const sfb_decoder_config* config, const sfb_decoder_data* data,
                                const char* stablehlo_text, const sfb_compile_options* base_options,
                                const float* input, int measurement_budget, int repetitions,
                                sfb_optimization_result* result, sfb_plan_candidate* candidates_out, int capacity,
                                sfb_decoder_plan** plan);

/* ---- decoder benchmark matrix ---------------------------------------------------------------------
 * realistic_decoder_profiles / benchmark_decoder_profile / write_decoder_benchmark_csv /
 * write_decoder_plan_candidates_csv (include/schedforge/decoder_compiler.h:180-203,236-247;
 * src/decoder_compiler.cpp:864-1060): the same 24 profiles (3 scales x {prefill 128, 512, 2048; decode over
 * 128, 512, 2048, 4096 cached tokens} + 3 tiny MoE layers), the same estimates, synthetic data (seed 101, routing
 * trace seed 103), evidence kinds and CSV columns.  A profile above either budget is recorded as compile-only
 * without touching the device; the others are measured on the device plan (median of `repetitions` passes after
 * one warm-up, host buffers), after sfb_decoder_optimize with a budget of 6 when optimize_plan != 0.
 * CSV columns without a device counterpart keep their place: llvm_compile_ms and memory_planning_ms are 0,
 * threads 0, placement "compact"; dispatch_ms holds the host<->device copy time of a pass. */
#define SFB_MAX_PLAN_CANDIDATES 17
enum { SFB_EVIDENCE_SKIPPED = 0, SFB_EVIDENCE_COMPILE_ONLY = 1, SFB_EVIDENCE_MEASURED = 2 }; /* DecoderEvidenceKind */
typedef struct sfb_decoder_profile {
    char name[64];
    sfb_decoder_config config;
    int routing;                      /* RoutingDistribution: 0 uniform, 1 moderate-skew, 2 heavy-skew */
    uint64_t estimated_flops;
    uint64_t estimated_weight_bytes;
    uint64_t estimated_activation_bytes;
} sfb_decoder_profile;
typedef struct sfb_decoder_benchmark_record {
    sfb_decoder_profile profile;
    int evidence;
    sfb_decoder_result measured;
    double max_error;                 /* 0: the device run is not compared with a scalar layer here */
    sfb_plan_cost plan_cost;
    double compile_milliseconds, llvm_compile_milliseconds, memory_planning_milliseconds;
    double optimizer_speedup, optimizer_baseline_milliseconds;
    int hardware_measurements;
    int candidate_count;
    sfb_plan_candidate candidates[SFB_MAX_PLAN_CANDIDATES];
    char selected_policy[192];
    char note[96];
} sfb_decoder_benchmark_record;
int sfb_decoder_profile_count(void);
sfb_status sfb_decoder_profile_get(int index, sfb_decoder_profile* out);
sfb_status sfb_benchmark_decoder_profile(const sfb_decoder_profile* profile, const char* stablehlo_text,
                                         const sfb_compile_options* options, uint64_t max_real_flops,
                                         uint64_t max_real_weight_bytes, int optimize_plan, int repetitions,
                                         sfb_decoder_benchmark_record* record);
sfb_status sfb_write_decoder_benchmark_csv(const char* path, const sfb_decoder_benchmark_record* records, int count);
sfb_status sfb_write_decoder_plan_candidates_csv(const char* path, const sfb_decoder_benchmark_record* records,
                                                 int count);
/* DecoderExecutablePlan::compile_milliseconds: host time of sfb_decoder_compile for this plan. */
double sfb_decoder_compile_milliseconds(const sfb_decoder_plan* plan);

/* ---- sum all-reduce over NVLink peer memory, fused with the producing GEMM -----------------------
 * Replaces, for the sharded plan, the collective that the reference does not have (it is a
 * single-process CPU library); the unfused form is the sfb_allreduce_fn hook below.
 * data: this rank's partial sums in, the sum out (bf16 [count]).  recv: this rank's receive buffer,
 * slot s (slot_elems elements apart) holds rank s's partial sums, pushed there by rank s's GEMM
 * epilogue (sfb_gemm_args.peer_out).  local_flags[s] is written by rank s; peer_flags[s] is the
 * address of local_flags[rank] inside rank s's memory as mapped into this process.  epoch must
 * grow by one with every use of the same buffers.  The wait is bounded (about two seconds); when
 * it gives up, bit 0x100 of sfb_device_status is set and data keeps this rank's partial sums. */
typedef struct sfb_peer_allreduce_args {
    void* data;
    const void* recv;
    uint32_t* local_flags;
    uint32_t* peer_flags[SFB_MAX_PEERS];
    int rank, size;
    uint32_t epoch;
    int64_t count;
    int64_t slot_elems;
} sfb_peer_allreduce_args;
sfb_status sfb_k_peer_allreduce_finish(const sfb_peer_allreduce_args* args, sfb_stream stream);

/* Two-shot form of the same all-reduce for large outputs on several ranks (no counterpart in the reference):
 * rank r owns rows [r * rows_own, (r + 1) * rows_own) of a [size * rows_own, width] bf16 tensor.
 *   1. reduce-scatter: either under the GEMM (with sfb_gemm_args.scatter_rows = rows_own the O / Down projection stores
 *      each output piece only to scatter_out[owner of the row], this rank's slot in the owner's receive buffer, row-local
 *      layout [rows_own, width]) or by the owners themselves (pull, below); a rank moves (size - 1) / size of the tensor;
 *   2. this kernel on the owner: waits (bounded) until every peer has delivered, adds the `slots` partial rows in
 *      rank order in fp32 (+ the owner's rows of `residual`), rounds to bf16, writes the finished rows into
 *      gathered[rank] (its own full tensor) and, when gather != 0, into gathered[s] of every peer with plain peer
 *      stores (the all-gather), together with the per-row sums of squares of the rounded rows in ss[s] (optional;
 *      what the folded RMSNorm of the next GEMM consumes), then waits (bounded) for the peers' rows.
 * slots == 0: all-gather of rows the rank already holds (`source`, [rows_own, width]; source_ss optional).
 * local_flags: 2 * SFB_MAX_PEERS words of this collective in this rank's memory ([s] = partial sums of rank s
 * delivered, [SFB_MAX_PEERS + s] = finished rows of rank s delivered); peer_flags[s] = the address of entry
 * [rank] of rank s's local_flags, as mapped into this process.  done_counter: one zeroed word per collective.
 * epoch grows by one with every use.  A wait that gives up sets bit 0x100 of sfb_device_status. */
typedef struct sfb_peer_gather_args {
    const void* recv;
    int64_t slot_elems;
    int slots;
    /* pull[0] != NULL: the partial rows of rank s are READ from pull[s] ([rows_own, width], this owner's row range inside
     * rank s's partial tensor, mapped into this process; pull[rank] is local) instead of from recv.  The producing GEMM
     * then stores its whole partial tensor locally with its ordinary epilogue and the owners fetch their rows with wide
     * peer loads: small peer stores from a GEMM epilogue use NVLink poorly. */
    const void* pull[SFB_MAX_PEERS];
    const void* source;
    const float* source_ss;
    const void* residual;
    void* gathered[SFB_MAX_PEERS];
    float* ss[SFB_MAX_PEERS];
    uint32_t* local_flags;
    uint32_t* peer_flags[SFB_MAX_PEERS];
    uint32_t* done_counter;
    int rank, size;
    uint32_t epoch;
    int rows_own, width;
    int gather;
    uint32_t* epoch_out;   /* gather == 0: optional device word that receives `epoch` when the rows are done; a caller
                              that moves the rows to the peers with copy engines copies this word into the peers' flag
                              arrays after the rows ("rows sent") */
} sfb_peer_gather_args;
sfb_status sfb_k_peer_reduce_gather(const sfb_peer_gather_args* args, sfb_stream stream);
/* Bounded wait (one thread) until local_flags[s] has reached epoch for every peer s: closes an all-gather whose rows
 * travel by copy engine while other kernels run.  Bit 0x100 of sfb_device_status when it gives up. */
sfb_status sfb_k_peer_wait(const uint32_t* local_flags, int rank, int size, uint32_t epoch, sfb_stream stream);
/* Bounded wait (one thread) until the device word *flag has reached epoch (wrap-around compare).  The word is
 * written by a copy that a copy engine runs behind the data it announces (sfb_decoder_execute: the upload of a row
 * chunk, then a 4-byte copy of the epoch), so the stream of kernels needs no event from the copy stream.  Bit 0x100 of
 * sfb_device_status when it gives up. */
sfb_status sfb_k_flag_wait(const uint32_t* flag, uint32_t epoch, sfb_stream stream);

/* ---- token-sharded expert parallelism: all-to-all dispatch and combine over peer stores --------------------
 * No counterpart in the reference (a single-process library); what must be preserved is the order of its
 * dispatch_tokens (src/moe_compiler.cpp:496-528: per expert, rows in (token, slot) order) and of its weighted
 * combine (:219-226).  Rank r owns tokens [r * rows_own, (r + 1) * rows_own) and experts [r * E / size, ...).
 * Every rank routes and dispatches its own tokens (sfb_k_moe_route, sfb_k_moe_dispatch with values = NULL), then
 *   sfb_k_moe_ep_plan    exchanges the per-expert histograms and derives send_base[E] (first row, on the expert's
 *                        owner, of this rank's rows of that expert), recv_offsets[E / size + 1] (segment starts of
 *                        this rank's experts = group_offsets of the grouped GEMMs) and return_table
 *                        [E / size * size][4] = (receive start, rows, source rank, first row at the source);
 *   sfb_k_moe_ep_send    copies every locally dispatched token row to its final position in the owner's receive
 *                        buffer (a segment holds rank 0's rows, then rank 1's, ...: the reference's order), with
 *                        the global token id and the route slot;
 *   sfb_k_moe_ep_return  copies every expert output row back to the source rank, to the row's position in that
 *                        rank's local dispatched order, where sfb_k_moe_combine of that rank reads it.
 * Each call ends with an announcement to every peer and a bounded wait for theirs (sfb_ep_sync: local_flags[s] is
 * written by rank s, peer_flags[s] is the address of entry [rank] of rank s's local_flags, done_counter one
 * zeroed word, epoch grows by one per use); a wait that gives up sets bit 0x100 of sfb_device_status. */
typedef struct sfb_ep_sync {
    uint32_t* local_flags;
    uint32_t* peer_flags[SFB_MAX_PEERS];
    uint32_t* done_counter;
    uint32_t epoch;
    int rank, size;
} sfb_ep_sync;
typedef struct sfb_moe_ep_plan_args {
    const int* counts;                 /* this rank's histogram [experts] (sfb_k_moe_route on its tokens) */
    int* counts_all[SFB_MAX_PEERS];    /* every rank's table [size][experts]; entry [rank] is local */
    int experts;
    int* send_base;
    int* recv_offsets;
    int* return_table;
    sfb_ep_sync sync;
} sfb_moe_ep_plan_args;
typedef struct sfb_moe_ep_send_args {
    const void* rows;                  /* this rank's token rows [rows_own, hidden] bf16 */
    const int* offsets;                /* local dispatch: segment starts [experts + 1] */
    const int* token_ids;              /* local dispatch: token of every dispatched row */
    const int* route_slots;
    const int* send_base;
    void* recv_rows[SFB_MAX_PEERS];    /* every rank's receive buffer [capacity, hidden] bf16 */
    int* recv_tokens[SFB_MAX_PEERS];   /* ... and the global token id / route slot of every received row */
    int* recv_slots[SFB_MAX_PEERS];
    int assignments, hidden, experts, first_token;
    sfb_ep_sync sync;
} sfb_moe_ep_send_args;
typedef struct sfb_moe_ep_return_args {
    const void* rows;                  /* expert outputs in receive order [received, hidden] bf16 */
    const int* recv_offsets;
    const int* return_table;
    void* back[SFB_MAX_PEERS];         /* every rank's [rows_own * top_k, hidden] buffer in its local dispatched order */
    int hidden, experts_local;
    int max_rows;                      /* upper bound of the received rows (sizes the launch) */
    sfb_ep_sync sync;
} sfb_moe_ep_return_args;
sfb_status sfb_k_moe_ep_plan(const sfb_moe_ep_plan_args* args, sfb_stream stream);
/* The table arithmetic of sfb_k_moe_ep_plan on the HOST (no device needed), from the complete histogram table
 * counts_all[size][experts]: the same send_base, recv_offsets and return_table for rank `rank`. */
sfb_status sfb_moe_ep_tables(const int* counts_all, int size, int experts, int rank, int* send_base, int* recv_offsets,
                             int* return_table);
sfb_status sfb_k_moe_ep_send(const sfb_moe_ep_send_args* args, sfb_stream stream);
sfb_status sfb_k_moe_ep_return(const sfb_moe_ep_return_args* args, sfb_stream stream);

/* Device memory that other processes of this node can map (CUDA IPC): allocate + export a 64-byte
 * handle, map a peer's handle, unmap, free. */
sfb_status sfb_peer_alloc(size_t bytes, void** ptr, void* handle64);
sfb_status sfb_peer_open(const void* handle64, void** ptr);
sfb_status sfb_peer_close(void* ptr);
sfb_status sfb_peer_free(void* ptr);

/* Sharded plan (tp_size > 1): use the fused form for the all-reduces after the O and Down
 * projections.  local_base: this rank's buffer of sfb_decoder_peer_bytes(plan) bytes from
 * sfb_peer_alloc (zero-filled); peer_bases[s]: rank s's buffer mapped with sfb_peer_open (entry
 * tp_rank ignored).  Every rank of the group must make the same calls in the same order. */
size_t sfb_decoder_peer_bytes(const sfb_decoder_plan* plan);
sfb_status sfb_decoder_set_peer_allreduce(sfb_decoder_plan* plan, void* local_base, void* const* peer_bases);

/* The same with the form chosen: mode 1 = the one-shot form above (each rank pushes its whole partial tensor to
 * every peer: two ranks, or the small outputs of decode plans), mode 2 = the two-shot form (sfb_k_peer_reduce_gather:
 * reduce-scatter under the GEMM, then the row owners add the residual, sum, take the sums of squares for the folded
 * RMSNorm and all-gather the finished rows with peer stores; needs rows % tp_size == 0), mode 3 = the two-shot form
 * with the all-gather moved to copy engines (peer-to-peer copies on a side stream of the plan) so that it runs UNDER
 * the next GEMM, which waits per owner for the rows it has not got yet (sfb_gemm_args.owner_flags; dense plans with
 * 128-row multiples per rank), mode 0 = mode 3 or 2 for more than two ranks and more than 128 rows, else one-shot.  With the two-shot form sfb_decoder_execute_rows gathers
 * the input rows with peer stores as well instead of going through the hook. */
sfb_status sfb_decoder_set_peer_collective(sfb_decoder_plan* plan, void* local_base, void* const* peer_bases, int mode);

/* Tensor-parallel hook: called on the plan's stream after the O projection and after the
 * Down projection partial sums are in `buffer` (`count` elements of `dtype`); the callee
 * must all-reduce (sum) in place on `stream`.  NULL = single shard. */
typedef void (*sfb_allreduce_fn)(void* user, void* buffer, int64_t count, int dtype,
                                 sfb_stream stream);
sfb_status sfb_decoder_set_allreduce(sfb_decoder_plan* plan, sfb_allreduce_fn fn, void* user);

/* Introspection: text dump in the reference's `sfe.decoder_executable` layout
 * (DecoderExecutablePlan::dump, src/decoder_compiler.cpp:694-717), workspace bytes, the
 * device pointer of a named intermediate ("normalized2", "attention_residual", "output",
 * ...) and its element count, for tests that feed the oracle the very same tensor. */
sfb_status sfb_decoder_dump(const sfb_decoder_plan* plan, char* buffer, size_t capacity);
size_t sfb_decoder_workspace_bytes(const sfb_decoder_plan* plan);
sfb_status sfb_decoder_read_tensor(sfb_decoder_plan* plan, const char* name, float* host_out,
                                   int64_t capacity, int64_t* count);
sfb_stream sfb_decoder_stream(sfb_decoder_plan* plan);

/* AttentionConfig, include/schedforge/attention_compiler.h:23-33. */
typedef struct sfb_attention_config {
    int batch, query_heads, kv_heads, sequence_query, sequence_kv, head_dim, head_dim_value;
    int causal;
    float scale;
} sfb_attention_config;

/* execute_attention, src/attention_compiler.cpp:879-885 (host q/k/v/out, float32). */
sfb_status sfb_attention_execute(const sfb_attention_config* config, const float* q,
                                 const float* key, const float* value, float* out, int dtype,
                                 int backend, double* milliseconds);

/* make_kv_cache + append_kv + execute_decode_attention (contiguous cache),
 * src/attention_compiler.cpp:923-1007: keys/values [B,Hkv,length,D]; guard
 * 0 < length <= config.sequence_kv else SFB_INVALID_ARGUMENT. */
sfb_status sfb_attention_decode(const sfb_attention_config* config, const float* q,
                                const float* keys, const float* values, int length, float* out,
                                int dtype, double* milliseconds);

/* PagedKVCache, include/schedforge/next_milestones.h:15-43, kept on the device.  One page
 * table and one length for the whole batch, pages handed out from the BACK of the free
 * list, like the reference. */
typedef struct sfb_paged_kv sfb_paged_kv;
sfb_status sfb_paged_create(int batch, int kv_heads, int head_dim, int head_dim_value,
                            int page_tokens, int capacity, int dtype, sfb_paged_kv** cache);
void sfb_paged_destroy(sfb_paged_kv* cache);
sfb_status sfb_paged_set_free_pages(sfb_paged_kv* cache, const int* pages, int count);
sfb_status sfb_paged_append(sfb_paged_kv* cache, const float* keys, const float* values, int tokens);
sfb_status sfb_paged_truncate(sfb_paged_kv* cache, int new_length);
sfb_status sfb_paged_release(sfb_paged_kv* cache, const int* pages, int count);
/* info[0..3] = length, pages in table, free pages, total pages. */
sfb_status sfb_paged_info(const sfb_paged_kv* cache, int* info, int* page_table, int table_capacity,
                          int* free_pages, int free_capacity);
sfb_status sfb_paged_gather(sfb_paged_kv* cache, float* keys, float* values);
/* execute_paged_decode_attention, src/next_milestones.cpp:583-609 (guards :98-120). */
sfb_status sfb_paged_decode(sfb_paged_kv* cache, const sfb_attention_config* config,
                            const float* q, float* out, double* milliseconds);

/* MoeConfig, include/schedforge/moe_compiler.h:71-77. */
typedef struct sfb_moe_config {
    int tokens, hidden, intermediate, experts, top_k;
} sfb_moe_config;

/* route_topk, src/moe_compiler.cpp:412-455 (host buffers; input dtype selects whether the
 * activations are rounded to bf16 before routing). */
sfb_status sfb_moe_route_topk(const sfb_moe_config* config, const float* input, int tokens,
                              const float* router_weight, const float* router_bias, int dtype,
                              int* expert_ids, float* expert_weights, int* counts);
/* dispatch_tokens, src/moe_compiler.cpp:496-528. values may be NULL. */
sfb_status sfb_moe_dispatch_tokens(const sfb_moe_config* config, const float* input, int tokens,
                                   const int* expert_ids, const float* expert_weights,
                                   const int* counts, int dtype, float* values, int* offsets,
                                   int* token_ids, int* route_slots, float* routing_weights);
/* execute_moe with a routing trace, src/moe_compiler.cpp:691-718 (guard: tokens <=
 * config.tokens).  Weights w1,w3 [E,H,I], w2 [E,I,H]. */
sfb_status sfb_moe_execute(const sfb_moe_config* config, const float* input, int tokens,
                           const float* w1, const float* w3, const float* w2,
                           const int* expert_ids, const float* expert_weights, const int* counts,
                           int dtype, int gemm_backend, float* out, double* milliseconds);
/* quantize_moe_weights + execute_quantized_moe, src/next_milestones.cpp:699-738 (per expert matrix,
 * per output channel: scale = max|w| / 127, q = round-half-away(w / scale) clamped to +-127; the experts
 * then multiply by q * scale).  bf16 arithmetic on the grouped tcgen05 GEMMs; per_channel = 0 (one scale per
 * matrix) is rejected with SFB_INVALID_ARGUMENT.  The reference's bar is 0.2 absolute against reference_moe
 * on the unquantized weights (tests/test_schedforge.cpp:911). */
sfb_status sfb_moe_execute_quantized(const sfb_moe_config* config, const float* input, int tokens,
                                     const float* w1, const float* w3, const float* w2,
                                     const int* expert_ids, const float* expert_weights, const int* counts,
                                     int per_channel, int gemm_backend, float* out, double* milliseconds);
/* MoeCompiler::compile + execute_moe on a compiled plan (include/schedforge/moe_compiler.h:181-212,
 * src/moe_compiler.cpp:684-818): the expert weights (w1, w3 [E,H,I]; w2 [E,I,H]) are packed and uploaded ONCE and stay
 * on the device with every buffer a pass needs; sfb_moe_plan_execute then only moves the tokens.  With a routing
 * trace (all three arrays) the router is skipped; with none the plan routes with router_weight [H,E] (+ optional
 * router_bias [E], which the reference does not have) and the time includes the routing, like the reference's
 * untraced overload.  Guard: tokens <= config.tokens ("runtime token count exceeds compiled MoE guard").
 * weight_int8 != 0: the experts of quantize_moe_weights (bf16 plans).  sfb_moe_execute above builds such a plan for
 * one call. */
typedef struct sfb_moe_plan sfb_moe_plan;
sfb_status sfb_moe_compile(const sfb_moe_config* config, const float* w1, const float* w3, const float* w2,
                           const float* router_weight, const float* router_bias, int dtype, int gemm_backend,
                           int weight_int8, sfb_moe_plan** plan);
void sfb_moe_destroy(sfb_moe_plan* plan);
sfb_status sfb_moe_plan_execute(sfb_moe_plan* plan, const float* input, int tokens, const int* expert_ids,
                                const float* expert_weights, const int* counts, float* out, double* milliseconds);
/* plan_moe_tasks, src/moe_compiler.cpp:530-558: rows (expert, begin, end, bucket). */
sfb_status sfb_moe_plan_tasks(const sfb_moe_config* config, const int* counts, int split_threshold,
                              int* tasks, int capacity, int* task_count);
/* make_routing_trace (src/moe_compiler.cpp:457-489; distribution 0 uniform, 1 moderate-skew, 2 heavy-skew) and the
 * input tensor of make_decoder_data (src/decoder_compiler.cpp:483-492): the reference's seeded generators
 * (std::mt19937), so that a benchmark run here and one of the reference see the same tokens and routes. */
sfb_status sfb_make_routing_trace(const sfb_moe_config* config, int distribution, unsigned seed, int* expert_ids,
                                  float* expert_weights, int* counts);
sfb_status sfb_make_decoder_input(const sfb_decoder_config* config, unsigned seed, float* input);
/* The whole of make_decoder_data (src/decoder_compiler.cpp:483-514, with make_moe_data, src/moe_compiler.cpp:
 * 393-406, for MoE layers): one std::mt19937(seed) stream, uniform in (-0.15, 0.15), drawn in the order input,
 * Wq, Wk, Wv, Wo, Wgate, Wup, Wdown, then (decode) cached K and V; RMSNorm weights 1; MoE layers add a second
 * stream std::mt19937(seed + 1), uniform in (-0.2, 0.2), in the order (unused input), router, W1, W3, W2.
 * Bit-identical to the reference's generator, so a benchmark here and one of the reference see the same layer.
 * Destinations are HOST float32 buffers of the DecoderData sizes; a NULL destination is skipped (its values are
 * still drawn). */
typedef struct sfb_decoder_data_buffers {
    float* rms1_weight;
    float* query_weight;
    float* key_weight;
    float* value_weight;
    float* output_weight;
    float* rms2_weight;
    float* gate_weight;
    float* up_weight;
    float* down_weight;
    float* router_weight;
    float* w1;
    float* w3;
    float* w2;
    float* cached_key;
    float* cached_value;
} sfb_decoder_data_buffers;
sfb_status sfb_make_decoder_data(const sfb_decoder_config* config, unsigned seed, float* input,
                                 const sfb_decoder_data_buffers* out);

/* Column shard of a [rows, cols] row-major host matrix / row shard, used by the
 * tensor-parallel plan build and exposed for tests: copies shard `rank` of `size`. */
sfb_status sfb_shard_columns(const float* src, int rows, int cols, int rank, int size, float* dst);
sfb_status sfb_shard_rows(const float* src, int rows, int cols, int rank, int size, float* dst);

#ifdef __cplusplus
}
#endif
#endif /* SCHEDFORGE_B200_H */
