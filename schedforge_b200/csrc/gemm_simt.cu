// CUDA-core GEMMs.
//
//  * gemm_f32_kernel: the fp32 plan's GEMM.  Every output is ONE fused-multiply-add chain
//    over ascending k, which is exactly the rounding sequence of the reference's AVX2
//    register kernels, so the result is bit-identical to the reference's native path.
//  * gemm_bf16_simt_kernel: shape-agnostic bf16 GEMM (fp32 accumulate) with the same
//    epilogues as the tensor-core kernel.  It is the path for shapes the tcgen05 kernel
//    does not take (k % 8 != 0, tiny head sizes) and the cross-check for it in tests.
#include <algorithm>

#include "common.cuh"

namespace sfb {

sfb_status gemm_bf16_tcgen05(const sfb_gemm_args& args, cudaStream_t stream);  // gemm_tcgen05.cu
bool gemm_bf16_tcgen05_supported(const sfb_gemm_args& args);

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

// Computes columns [0, n_cols) of the [m, n] output (n is the leading dimension).
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                int m, int n, int k, int n_cols) {
    __shared__ float as[TK][TM + 4];
    __shared__ float bs[TK][TN + 4];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int row0 = blockIdx.y * TM, col0 = blockIdx.x * TN;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < k; k0 += TK) {
        for (int i = threadIdx.x; i < TM * TK; i += 256) {
            const int r = i / TK, kk = i % TK;
            const int gr = row0 + r, gk = k0 + kk;
            as[kk][r] = (gr < m && gk < k) ? a[static_cast<size_t>(gr) * k + gk] : 0.0F;
        }
        for (int i = threadIdx.x; i < TK * TN; i += 256) {
            const int kk = i / TN, cidx = i % TN;
            const int gk = k0 + kk, gc = col0 + cidx;
            bs[kk][cidx] = (gk < k && gc < n_cols) ? b[static_cast<size_t>(gk) * n + gc] : 0.0F;
        }
        __syncthreads();
        const int kmax = min(TK, k - k0);
        for (int kk = 0; kk < kmax; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = as[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gr = row0 + ty * 4 + i;
        if (gr >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gc = col0 + tx * 4 + j;
            if (gc < n_cols) c[static_cast<size_t>(gr) * n + gc] = acc[i][j];
        }
    }
}

// The n % 8 tail columns of the reference's native GEMM are a scalar loop that rounds the
// product and the sum separately; one thread per output reproduces that sequence.
__global__ void gemm_f32_tail_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                     float* __restrict__ c, int m, int n, int k, int col_begin) {
    const int tail = n - col_begin;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= m * tail) return;
    const int row = idx / tail, col = col_begin + idx % tail;
    float acc = 0.0F;
    for (int kk = 0; kk < k; ++kk)
        acc = __fadd_rn(acc, __fmul_rn(a[static_cast<size_t>(row) * k + kk], b[static_cast<size_t>(kk) * n + col]));
    c[static_cast<size_t>(row) * n + col] = acc;
}

struct SimtParams {
    const bf16* a;
    const bf16* bt;
    void* out;
    int m, n, k;
    int epilogue, out_f32;
    const bf16* residual;
    int swiglu_block;
    bf16 *q, *key, *value;
    const float *rope_cos, *rope_sin;
    int batch, seq, q_heads, kv_heads, head_dim;
    const int* group_offsets;
    int groups;
    int rope_row_offset;
};

__device__ __forceinline__ void store_out(const SimtParams& p, size_t index, float v) {
    if (p.out_f32) static_cast<float*>(p.out)[index] = v;
    else static_cast<bf16*>(p.out)[index] = from_float<bf16>(v);
}

// Writes the outputs of column pair (c0, c1) of `row` according to the epilogue of `p`.
__device__ __forceinline__ void apply_epilogue(const SimtParams& p, int row, int pair, int c0, int c1, float acc0,
                                               float acc1) {
    switch (p.epilogue) {
        case SFB_EPI_STORE:
        case SFB_EPI_RESIDUAL: {
            const size_t i0 = static_cast<size_t>(row) * p.n + c0;
            const bool res = p.epilogue == SFB_EPI_RESIDUAL;
            store_out(p, i0, acc0 + (res ? to_float(p.residual[i0]) : 0.0F));
            if (c1 < p.n) store_out(p, i0 + 1, acc1 + (res ? to_float(p.residual[i0 + 1]) : 0.0F));
            break;
        }
        case SFB_EPI_SWIGLU:
            store_out(p, static_cast<size_t>(row) * (p.n / 2) + pair, acc0 / (1.0F + __expf(-acc0)) * acc1);
            break;
        case SFB_EPI_ROPE_SPLIT: {
            const int hidden = p.q_heads * p.head_dim, kvw = p.kv_heads * p.head_dim;
            const int token = row + p.rope_row_offset;
            const int b = token / p.seq, t = token % p.seq;
            bf16* dst;
            int heads, local;
            bool rotate = true;
            if (c0 < hidden) { dst = p.q; heads = p.q_heads; local = c0; }
            else if (c0 < hidden + kvw) { dst = p.key; heads = p.kv_heads; local = c0 - hidden; }
            else { dst = p.value; heads = p.kv_heads; local = c0 - hidden - kvw; rotate = false; }
            const int head = local / p.head_dim, d = local % p.head_dim;
            const size_t o = ((static_cast<size_t>(b) * heads + head) * p.seq + t) * p.head_dim + d;
            if (rotate) {
                const float c = p.rope_cos[t * (p.head_dim / 2) + d / 2];
                const float s = p.rope_sin[t * (p.head_dim / 2) + d / 2];
                dst[o] = from_float<bf16>(acc0 * c - acc1 * s);
                dst[o + 1] = from_float<bf16>(acc0 * s + acc1 * c);
            } else {
                dst[o] = from_float<bf16>(acc0);
                dst[o + 1] = from_float<bf16>(acc1);
            }
            break;
        }
    }
}

// 16x16 threads; thread (ty, tx) owns row `row0 + ty` and the column PAIR `pair0 + tx`.
// A pair is two adjacent columns (2j, 2j+1), or for SwiGLU a gate column and its up column.
__global__ void __launch_bounds__(256)
gemm_bf16_simt_kernel(SimtParams p) {
    constexpr int BK = 32;
    __shared__ float as[16][BK + 1];
    __shared__ float b0[16][BK + 1];
    __shared__ float b1[16][BK + 1];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    int row_begin = 0, row_end = p.m;
    const bf16* bt = p.bt;
    if (p.group_offsets) {
        const int g = blockIdx.z;
        row_begin = p.group_offsets[g];
        row_end = p.group_offsets[g + 1];
        bt += static_cast<size_t>(g) * p.n * p.k;
    }
    const int row0 = row_begin + blockIdx.y * 16;
    if (row0 >= row_end) return;
    const int pairs = (p.n + 1) / 2;
    const int pair0 = blockIdx.x * 16;
    auto columns = [&](int pair, int& c0, int& c1) {
        if (p.epilogue == SFB_EPI_SWIGLU) {
            const int blk = pair / p.swiglu_block, w = pair % p.swiglu_block;
            c0 = blk * 2 * p.swiglu_block + w;
            c1 = c0 + p.swiglu_block;
        } else {
            c0 = 2 * pair;
            c1 = 2 * pair + 1;
        }
    };
    float acc0 = 0.0F, acc1 = 0.0F;
    for (int k0 = 0; k0 < p.k; k0 += BK) {
        for (int i = threadIdx.x; i < 16 * BK; i += 256) {
            const int r = i / BK, kk = i % BK;
            const int gr = row0 + r, gk = k0 + kk;
            as[r][kk] = (gr < row_end && gk < p.k) ? to_float(p.a[static_cast<size_t>(gr) * p.k + gk]) : 0.0F;
            const int pair = pair0 + r;
            int c0 = 0, c1 = 0;
            columns(pair, c0, c1);
            const bool live = pair < pairs && gk < p.k;
            b0[r][kk] = (live && c0 < p.n) ? to_float(bt[static_cast<size_t>(c0) * p.k + gk]) : 0.0F;
            b1[r][kk] = (live && c1 < p.n) ? to_float(bt[static_cast<size_t>(c1) * p.k + gk]) : 0.0F;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            acc0 = fmaf(as[ty][kk], b0[tx][kk], acc0);
            acc1 = fmaf(as[ty][kk], b1[tx][kk], acc1);
        }
        __syncthreads();
    }
    const int row = row0 + ty, pair = pair0 + tx;
    if (row >= row_end || pair >= pairs) return;
    int c0 = 0, c1 = 0;
    columns(pair, c0, c1);
    apply_epilogue(p, row, pair, c0, c1, acc0, acc1);
}

sfb_status validate_gemm(const sfb_gemm_args& g) {
    SFB_REQUIRE(g.a && g.bt && g.m > 0 && g.n > 0 && g.k > 0, "gemm: invalid shape or null operand");
    switch (g.epilogue) {
        case SFB_EPI_STORE:
            SFB_REQUIRE(g.out, "gemm: null output");
            break;
        case SFB_EPI_RESIDUAL:
            SFB_REQUIRE(g.out && g.residual, "gemm: residual epilogue needs out and residual");
            break;
        case SFB_EPI_SWIGLU:
            SFB_REQUIRE(g.out && g.swiglu_block > 0 && g.n % (2 * g.swiglu_block) == 0,
                        "gemm: SwiGLU epilogue needs n to be a multiple of 2*swiglu_block");
            break;
        case SFB_EPI_ROPE_SPLIT:
            SFB_REQUIRE(g.q && g.key && g.value && g.rope_cos && g.rope_sin, "gemm: RoPE epilogue needs q/key/value and tables");
            SFB_REQUIRE(g.batch > 0 && g.seq > 0 && g.rope_row_offset >= 0 &&
                            g.rope_row_offset + g.m <= g.batch * g.seq && g.head_dim % 2 == 0 &&
                        g.n == (g.q_heads + 2 * g.kv_heads) * g.head_dim,
                        "gemm: RoPE epilogue shape mismatch");
            SFB_REQUIRE(!g.group_offsets, "gemm: RoPE epilogue is not available in grouped mode");
            break;
        default:
            return fail(SFB_INVALID_ARGUMENT, "gemm: unknown epilogue");
    }
    if (g.group_offsets) SFB_REQUIRE(g.groups > 0, "gemm: grouped mode needs groups > 0");
    return SFB_OK;
}

// One thread per 16-byte piece (8 elements) of the blocked copy.
__global__ void tile_weight_kernel(const bf16* __restrict__ bt, bf16* __restrict__ tiled, int n, int k,
                                   long long pieces) {
    const int k_blocks = (k + 63) / 64;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < pieces;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long block = i >> 9;               // 512 pieces per 64x64 block
        const int within = static_cast<int>(i & 511);
        const int r = within >> 3, c8 = (within & 7) * 8;
        const int row = static_cast<int>(block / k_blocks) * 64 + r;
        const int col = static_cast<int>(block % k_blocks) * 64 + c8;
        bf16 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            v[j] = (row < n && col + j < k) ? bt[static_cast<size_t>(row) * k + col + j] : from_float<bf16>(0.0F);
        *reinterpret_cast<uint4*>(tiled + i * 8) = *reinterpret_cast<const uint4*>(v);
    }
}

// One block per output row: absolute maximum over k, then the rounded quotients into the blocked layout.
__global__ void __launch_bounds__(256)
quantize_weight_int8_kernel(const bf16* __restrict__ bt, int8_t* __restrict__ q, float* __restrict__ scales, int n,
                            int k) {
    __shared__ float partial[8];
    const int row = blockIdx.x;
    const bf16* src = bt + static_cast<size_t>(row) * k;
    float maximum = 0.0F;
    for (int c = threadIdx.x; c < k; c += 256) maximum = fmaxf(maximum, fabsf(to_float(src[c])));
    maximum = warp_max(maximum);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = maximum;
    __syncthreads();
    maximum = partial[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) maximum = fmaxf(maximum, partial[i]);
    const float scale = maximum > 0.0F ? __fdiv_rn(maximum, 127.0F) : 1.0F;
    if (threadIdx.x == 0) scales[row] = scale;
    const int k_blocks = (k + 63) / 64, k_padded = k_blocks * 64;
    int8_t* block_row = q + (static_cast<size_t>(row / 64) * k_blocks) * 4096 + (row % 64) * 64;
    for (int c = threadIdx.x; c < k_padded; c += 256) {
        float value = 0.0F;
        if (c < k) value = fminf(fmaxf(roundf(__fdiv_rn(to_float(src[c]), scale)), -127.0F), 127.0F);
        block_row[static_cast<size_t>(c / 64) * 4096 + (c % 64)] = static_cast<int8_t>(value);
    }
}

// rows of the last 64-row block that do not exist
__global__ void zero_int8_rows_kernel(int8_t* __restrict__ q, int n, int k) {
    const int k_blocks = (k + 63) / 64, rows = (n + 63) / 64 * 64;
    const long long total = static_cast<long long>(rows - n) * k_blocks * 64;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int row = n + static_cast<int>(i / (static_cast<long long>(k_blocks) * 64));
        const int c = static_cast<int>(i % (static_cast<long long>(k_blocks) * 64));
        q[(static_cast<size_t>(row / 64) * k_blocks + c / 64) * 4096 + (row % 64) * 64 + (c % 64)] = 0;
    }
}

__global__ void dequantize_weight_int8_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales,
                                              bf16* __restrict__ bt, int n, int k) {
    const int k_blocks = (k + 63) / 64;
    const long long total = static_cast<long long>(n) * k;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int row = static_cast<int>(i / k), c = static_cast<int>(i % k);
        const int8_t value = q[(static_cast<size_t>(row / 64) * k_blocks + c / 64) * 4096 + (row % 64) * 64 + (c % 64)];
        bt[i] = from_float<bf16>(__fmul_rn(static_cast<float>(value), scales[row]));
    }
}

}  // namespace

}  // namespace sfb

using namespace sfb;

extern "C" {

sfb_status sfb_k_gemm_f32(const float* a, const float* b, float* c, int m, int n, int k,
                          sfb_stream stream) {
    SFB_REQUIRE(a && b && c && m > 0 && n > 0 && k > 0, "gemm_f32: invalid shape or null operand");
    const int n_main = n / 8 * 8;
    if (n_main > 0) {
        dim3 grid(ceil_div(n_main, TN), ceil_div(m, TM));
        gemm_f32_kernel<<<grid, 256, 0, as_stream(stream)>>>(a, b, c, m, n, k, n_main);
        SFB_TRY(check_launch("gemm_f32"));
    }
    if (n_main < n) {
        gemm_f32_tail_kernel<<<ceil_div(m * (n - n_main), 128), 128, 0, as_stream(stream)>>>(a, b, c, m, n, k, n_main);
        SFB_TRY(check_launch("gemm_f32_tail"));
    }
    return SFB_OK;
}

int64_t sfb_tiled_weight_elems(int n, int k) {
    if (n <= 0 || k <= 0) return 0;
    return static_cast<int64_t>(ceil_div(n, 64)) * ceil_div(k, 64) * 4096;
}

sfb_status sfb_k_tile_weight_bf16(const void* bt, void* tiled, int n, int k, sfb_stream stream) {
    SFB_REQUIRE(bt && tiled && n > 0 && k > 0, "tile_weight: invalid shape or null operand");
    SFB_REQUIRE((reinterpret_cast<uintptr_t>(tiled) & 15) == 0, "tile_weight: destination must be 16-byte aligned");
    const long long pieces = sfb_tiled_weight_elems(n, k) / 8;
    const int grid = static_cast<int>(std::min<long long>((pieces + 255) / 256, static_cast<long long>(sm_count()) * 16));
    tile_weight_kernel<<<grid, 256, 0, as_stream(stream)>>>(static_cast<const bf16*>(bt), static_cast<bf16*>(tiled), n,
                                                            k, pieces);
    return check_launch("tile_weight");
}

sfb_status sfb_k_quantize_weight_int8(const void* bt, void* q_tiled, float* scales, int n, int k, sfb_stream stream) {
    SFB_REQUIRE(bt && q_tiled && scales && n > 0 && k > 0, "quantize_weight: invalid shape or null operand");
    cudaStream_t s = as_stream(stream);
    quantize_weight_int8_kernel<<<n, 256, 0, s>>>(static_cast<const bf16*>(bt), static_cast<int8_t*>(q_tiled), scales, n, k);
    SFB_TRY(check_launch("quantize_weight_int8"));
    if (n % 64 != 0) {
        zero_int8_rows_kernel<<<64, 256, 0, s>>>(static_cast<int8_t*>(q_tiled), n, k);
        SFB_TRY(check_launch("quantize_weight_int8_pad"));
    }
    return SFB_OK;
}

sfb_status sfb_k_dequantize_weight_int8(const void* q_tiled, const float* scales, void* bt, int n, int k,
                                        sfb_stream stream) {
    SFB_REQUIRE(bt && q_tiled && scales && n > 0 && k > 0, "dequantize_weight: invalid shape or null operand");
    const long long total = static_cast<long long>(n) * k;
    const int grid = static_cast<int>(std::min<long long>((total + 255) / 256, static_cast<long long>(sm_count()) * 16));
    dequantize_weight_int8_kernel<<<grid, 256, 0, as_stream(stream)>>>(static_cast<const int8_t*>(q_tiled), scales,
                                                                       static_cast<bf16*>(bt), n, k);
    return check_launch("dequantize_weight_int8");
}

sfb_status sfb_k_gemm_bf16(const sfb_gemm_args* args, sfb_stream stream) {
    SFB_REQUIRE(args, "gemm: null arguments");
    SFB_TRY(validate_gemm(*args));
    SFB_REQUIRE(!args->bt_tiled || (!args->group_offsets && args->backend != SFB_GEMM_SIMT),
                "gemm: the blocked weight layout needs the dense tcgen05 kernel");
    int backend = args->backend;
    if (args->bt_tiled || args->peer_count != 0 || args->scatter_rows != 0 || args->bt_scales || args->row_ss || args->ss_out ||
        args->kv_k_pool || args->clear || args->owner_flags)
        backend = SFB_GEMM_TCGEN05;  // only that kernel knows these
    if (backend == SFB_GEMM_AUTO)
        backend = gemm_bf16_tcgen05_supported(*args) ? SFB_GEMM_TCGEN05 : SFB_GEMM_SIMT;
    if (backend == SFB_GEMM_TCGEN05) {
        if (!gemm_bf16_tcgen05_supported(*args))
            return fail(SFB_UNSUPPORTED, "gemm: shape not supported by the tcgen05 kernel");
        return gemm_bf16_tcgen05(*args, as_stream(stream));
    }
    SimtParams p{static_cast<const bf16*>(args->a), static_cast<const bf16*>(args->bt), args->out,
                 args->m, args->n, args->k, args->epilogue, args->out_f32,
                 static_cast<const bf16*>(args->residual), args->swiglu_block,
                 static_cast<bf16*>(args->q), static_cast<bf16*>(args->key), static_cast<bf16*>(args->value),
                 args->rope_cos, args->rope_sin, args->batch, args->seq, args->q_heads, args->kv_heads,
                 args->head_dim, args->group_offsets, args->groups, args->rope_row_offset};
    dim3 grid(ceil_div((args->n + 1) / 2, 16), ceil_div(args->m, 16), args->group_offsets ? args->groups : 1);
    gemm_bf16_simt_kernel<<<grid, 256, 0, as_stream(stream)>>>(p);
    return check_launch("gemm_bf16_simt");
}

}  // extern "C"
