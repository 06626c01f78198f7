// HBM-bound row and elementwise kernels of the decoder layer: RMSNorm, residual add,
// SwiGLU, dtype conversion, RoPE + head split.  Each is a coalesced streaming kernel;
// in the bf16 plan RoPE/SwiGLU/residual are normally fused into GEMM epilogues instead
// and these stand-alone versions serve the fp32 plan and the unfused policy.
#include "common.cuh"

#include <cmath>
#include <vector>

namespace sfb {
namespace {

// One warp per row.  fp32: sum of squares in double and (x*inv)*w, as the reference.
template <class T>
__global__ void rms_norm_kernel(const T* __restrict__ x, const float* __restrict__ weight,
                                T* __restrict__ y, int rows, int width, float epsilon) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= rows) return;
    const T* row = x + static_cast<size_t>(warp) * width;
    T* out = y + static_cast<size_t>(warp) * width;
    if constexpr (sizeof(T) == 4) {
        double ss = 0.0;
        for (int c = lane; c < width; c += 32) {
            const double v = static_cast<double>(row[c]);
            ss += v * v;
        }
        ss = warp_sum(ss);
        const float inv = 1.0F / sqrtf(static_cast<float>(ss / static_cast<double>(width)) + epsilon);
        for (int c = lane; c < width; c += 32)
            out[c] = __fmul_rn(__fmul_rn(row[c], inv), weight[c]);
    } else {
        float ss = 0.0F;
        if ((width & 7) == 0) {
            const uint4* row4 = reinterpret_cast<const uint4*>(row);
            for (int c = lane; c < width / 8; c += 32) {
                const uint4 packed = row4[c];
                const bf16* v = reinterpret_cast<const bf16*>(&packed);
#pragma unroll
                for (int i = 0; i < 8; ++i) { const float f = to_float(v[i]); ss += f * f; }
            }
            ss = warp_sum(ss);
            const float inv = 1.0F / sqrtf(ss / static_cast<float>(width) + epsilon);
            uint4* out4 = reinterpret_cast<uint4*>(out);
            for (int c = lane; c < width / 8; c += 32) {
                const uint4 packed = row4[c];
                const bf16* v = reinterpret_cast<const bf16*>(&packed);
                const float4 w0 = reinterpret_cast<const float4*>(weight)[2 * c];
                const float4 w1 = reinterpret_cast<const float4*>(weight)[2 * c + 1];
                const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                uint4 result;
                bf16* r = reinterpret_cast<bf16*>(&result);
#pragma unroll
                for (int i = 0; i < 8; ++i) r[i] = from_float<bf16>(to_float(v[i]) * inv * w[i]);
                out4[c] = result;
            }
        } else {
            for (int c = lane; c < width; c += 32) { const float f = to_float(row[c]); ss += f * f; }
            ss = warp_sum(ss);
            const float inv = 1.0F / sqrtf(ss / static_cast<float>(width) + epsilon);
            for (int c = lane; c < width; c += 32)
                out[c] = from_float<T>(to_float(row[c]) * inv * weight[c]);
        }
    }
}

// bf16, few rows (decode): one 256-thread block per row, so that a row is read by 256 threads
// at once instead of 32 threads sixteen times over.  width % 8 == 0.
__global__ void __launch_bounds__(256)
rms_norm_row_block_kernel(const bf16* __restrict__ x, const float* __restrict__ weight, bf16* __restrict__ y,
                          int width, float epsilon) {
    __shared__ float partial[8];
    grid_dependents_may_launch();  // the GEMM that follows can start fetching its weights
    grid_dependency_wait();
    const uint4* row4 = reinterpret_cast<const uint4*>(x + static_cast<size_t>(blockIdx.x) * width);
    uint4* out4 = reinterpret_cast<uint4*>(y + static_cast<size_t>(blockIdx.x) * width);
    const int pieces = width / 8;
    float ss = 0.0F;
    for (int c = threadIdx.x; c < pieces; c += 256) {
        const uint4 packed = row4[c];
        const bf16* v = reinterpret_cast<const bf16*>(&packed);
#pragma unroll
        for (int i = 0; i < 8; ++i) { const float f = to_float(v[i]); ss += f * f; }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.0F;
#pragma unroll
    for (int i = 0; i < 8; ++i) total += partial[i];
    const float inv = 1.0F / sqrtf(total / static_cast<float>(width) + epsilon);
    for (int c = threadIdx.x; c < pieces; c += 256) {
        const uint4 packed = row4[c];
        const bf16* v = reinterpret_cast<const bf16*>(&packed);
        const float4 w0 = reinterpret_cast<const float4*>(weight)[2 * c];
        const float4 w1 = reinterpret_cast<const float4*>(weight)[2 * c + 1];
        const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        uint4 result;
        bf16* r = reinterpret_cast<bf16*>(&result);
#pragma unroll
        for (int i = 0; i < 8; ++i) r[i] = from_float<bf16>(to_float(v[i]) * inv * w[i]);
        out4[c] = result;
    }
}

// float32 rows -> bf16 rows plus the sum of squares of each rounded row (SRC = float), or the sum of squares
// of bf16 rows alone (SRC = bf16, dst unused).  One 256-thread block per row for at most 128 rows (decode), one warp per row
// otherwise; width % 8 == 0 takes 16/32-byte accesses.
template <class SRC, bool BLOCK_PER_ROW>
__global__ void __launch_bounds__(256)
rows_sumsq_kernel(const SRC* __restrict__ src, bf16* __restrict__ dst, float* __restrict__ ss, int rows, int width) {
    __shared__ float partial[8];
    const int lane = threadIdx.x & 31;
    const int row = BLOCK_PER_ROW ? blockIdx.x : (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int first = BLOCK_PER_ROW ? threadIdx.x : lane, step = BLOCK_PER_ROW ? 256 : 32;
    float sum = 0.0F;
    if (row < rows) {
        const SRC* in = src + static_cast<size_t>(row) * width;
        if ((width & 7) == 0) {
            for (int c = first; c < width / 8; c += step) {
                float f[8];
                if constexpr (sizeof(SRC) == 4) {
                    const float4 a = reinterpret_cast<const float4*>(in)[2 * c], b = reinterpret_cast<const float4*>(in)[2 * c + 1];
                    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
                    uint4 packed;
                    bf16* r = reinterpret_cast<bf16*>(&packed);
#pragma unroll
                    for (int i = 0; i < 8; ++i) { r[i] = from_float<bf16>(f[i]); f[i] = to_float(r[i]); }
                    reinterpret_cast<uint4*>(dst + static_cast<size_t>(row) * width)[c] = packed;
                } else {
                    const uint4 packed = reinterpret_cast<const uint4*>(in)[c];
                    const bf16* v = reinterpret_cast<const bf16*>(&packed);
#pragma unroll
                    for (int i = 0; i < 8; ++i) f[i] = to_float(v[i]);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) sum = fmaf(f[i], f[i], sum);
            }
        } else {
            for (int c = first; c < width; c += step) {
                float f = to_float(in[c]);
                if constexpr (sizeof(SRC) == 4) {
                    const bf16 r = from_float<bf16>(f);
                    dst[static_cast<size_t>(row) * width + c] = r;
                    f = to_float(r);
                }
                sum = fmaf(f, f, sum);
            }
        }
    }
    sum = warp_sum(sum);
    if constexpr (BLOCK_PER_ROW) {
        if (lane == 0) partial[threadIdx.x >> 5] = sum;
        __syncthreads();
        if (threadIdx.x == 0) {
            float total = 0.0F;
#pragma unroll
            for (int i = 0; i < 8; ++i) total += partial[i];
            ss[row] = total;
        }
    } else if (lane == 0 && row < rows) {
        ss[row] = sum;
    }
}

template <class T>
__global__ void add_kernel(const T* __restrict__ x, const T* __restrict__ y, T* __restrict__ z,
                           int64_t count) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
        z[i] = from_float<T>(to_float(x[i]) + to_float(y[i]));
}

template <class T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int rows,
                              int intermediate) {
    const int64_t total = static_cast<int64_t>(rows) * intermediate;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t r = i / intermediate, j = i % intermediate;
        const float g = to_float(gate_up[r * 2 * intermediate + j]);
        const float u = to_float(gate_up[r * 2 * intermediate + intermediate + j]);
        out[i] = from_float<T>(g / (1.0F + expf(-g)) * u);
    }
}

template <class S, class D>
__global__ void convert_kernel(const S* __restrict__ src, D* __restrict__ dst, int64_t count) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
        dst[i] = from_float<D>(to_float(src[i]));
}

// One thread per (row, column pair) of the fused projection.  Q and K pairs are rotated
// with the table entry of the token's position inside its sequence; V pairs are copied.
template <class T>
__global__ void rope_split_kernel(const T* __restrict__ fused, T* __restrict__ q, T* __restrict__ key,
                                  T* __restrict__ value, const float* __restrict__ rope_cos,
                                  const float* __restrict__ rope_sin, int batch, int seq,
                                  int q_heads, int kv_heads, int dim) {
    const int hidden = q_heads * dim, kvw = kv_heads * dim, total = hidden + 2 * kvw;
    const int pairs_per_row = total / 2;
    const int64_t pairs = static_cast<int64_t>(batch) * seq * pairs_per_row;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < pairs; i += stride) {
        const int64_t row = i / pairs_per_row;
        const int col = static_cast<int>(i % pairs_per_row) * 2;
        const int b = static_cast<int>(row / seq), t = static_cast<int>(row % seq);
        const float even = to_float(fused[row * total + col]);
        const float odd = to_float(fused[row * total + col + 1]);
        T* dst;
        int heads, local;
        bool rotate = true;
        if (col < hidden) { dst = q; heads = q_heads; local = col; }
        else if (col < hidden + kvw) { dst = key; heads = kv_heads; local = col - hidden; }
        else { dst = value; heads = kv_heads; local = col - hidden - kvw; rotate = false; }
        const int head = local / dim, d = local % dim;
        const size_t o = ((static_cast<size_t>(b) * heads + head) * seq + t) * dim + d;
        if (rotate) {
            const float c = rope_cos[t * (dim / 2) + d / 2], s = rope_sin[t * (dim / 2) + d / 2];
            // even*cos - odd*sin and even*sin + odd*cos, each product rounded separately
            dst[o] = from_float<T>(__fsub_rn(__fmul_rn(even, c), __fmul_rn(odd, s)));
            dst[o + 1] = from_float<T>(__fadd_rn(__fmul_rn(even, s), __fmul_rn(odd, c)));
        } else {
            dst[o] = from_float<T>(even);
            dst[o + 1] = from_float<T>(odd);
        }
    }
}

int grid_for(int64_t work, int block) {
    const int64_t blocks = ceil_div64(work, block);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace
}  // namespace sfb

using namespace sfb;

extern "C" {

sfb_status sfb_k_rms_norm(const void* x, const float* weight, void* y, int rows, int width,
                          float epsilon, sfb_dtype dtype, sfb_stream stream) {
    SFB_REQUIRE(x && weight && y && rows > 0 && width > 0, "RMSNorm shape mismatch");
    const int block = 256, grid = ceil_div(rows, block / 32);
    if (dtype == SFB_BF16 && rows <= 2048 && width % 8 == 0 && width >= 2048 &&
        (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(weight) & 15) == 0) {
        SFB_CUDA(launch_dependent(rms_norm_row_block_kernel, dim3(rows), dim3(256), 0, as_stream(stream),
                                  static_cast<const bf16*>(x), weight, static_cast<bf16*>(y), width, epsilon));
        return check_launch("rms_norm");
    }
    if (dtype == SFB_F32)
        rms_norm_kernel<float><<<grid, block, 0, as_stream(stream)>>>(
            static_cast<const float*>(x), weight, static_cast<float*>(y), rows, width, epsilon);
    else
        rms_norm_kernel<bf16><<<grid, block, 0, as_stream(stream)>>>(
            static_cast<const bf16*>(x), weight, static_cast<bf16*>(y), rows, width, epsilon);
    return check_launch("rms_norm");
}

sfb_status sfb_k_add(const void* x, const void* y, void* z, int64_t count, sfb_dtype dtype,
                     sfb_stream stream) {
    SFB_REQUIRE(x && y && z && count > 0, "residual shape mismatch");
    const int block = 256, grid = grid_for(count, block);
    if (dtype == SFB_F32)
        add_kernel<float><<<grid, block, 0, as_stream(stream)>>>(
            static_cast<const float*>(x), static_cast<const float*>(y), static_cast<float*>(z), count);
    else
        add_kernel<bf16><<<grid, block, 0, as_stream(stream)>>>(
            static_cast<const bf16*>(x), static_cast<const bf16*>(y), static_cast<bf16*>(z), count);
    return check_launch("add");
}

sfb_status sfb_k_swiglu(const void* gate_up, void* out, int rows, int intermediate,
                        sfb_dtype dtype, sfb_stream stream) {
    SFB_REQUIRE(gate_up && out && rows > 0 && intermediate > 0, "SwiGLU shape mismatch");
    const int block = 256, grid = grid_for(static_cast<int64_t>(rows) * intermediate, block);
    if (dtype == SFB_F32)
        swiglu_kernel<float><<<grid, block, 0, as_stream(stream)>>>(
            static_cast<const float*>(gate_up), static_cast<float*>(out), rows, intermediate);
    else
        swiglu_kernel<bf16><<<grid, block, 0, as_stream(stream)>>>(
            static_cast<const bf16*>(gate_up), static_cast<bf16*>(out), rows, intermediate);
    return check_launch("swiglu");
}

sfb_status sfb_k_convert(const void* src, sfb_dtype src_dtype, void* dst, sfb_dtype dst_dtype,
                         int64_t count, sfb_stream stream) {
    SFB_REQUIRE(src && dst && count > 0, "convert: empty tensor");
    const int block = 256, grid = grid_for(count, block);
    cudaStream_t s = as_stream(stream);
    if (src_dtype == SFB_F32 && dst_dtype == SFB_BF16)
        convert_kernel<float, bf16><<<grid, block, 0, s>>>(static_cast<const float*>(src), static_cast<bf16*>(dst), count);
    else if (src_dtype == SFB_BF16 && dst_dtype == SFB_F32)
        convert_kernel<bf16, float><<<grid, block, 0, s>>>(static_cast<const bf16*>(src), static_cast<float*>(dst), count);
    else if (src_dtype == SFB_F32)
        convert_kernel<float, float><<<grid, block, 0, s>>>(static_cast<const float*>(src), static_cast<float*>(dst), count);
    else
        convert_kernel<bf16, bf16><<<grid, block, 0, s>>>(static_cast<const bf16*>(src), static_cast<bf16*>(dst), count);
    return check_launch("convert");
}

sfb_status sfb_k_convert_rows_sumsq(const float* src, void* dst_bf16, float* ss, int rows, int width, sfb_stream stream) {
    SFB_REQUIRE(src && dst_bf16 && ss && rows > 0 && width > 0, "convert: empty tensor");
    cudaStream_t s = as_stream(stream);
    if (rows <= 128) rows_sumsq_kernel<float, true><<<rows, 256, 0, s>>>(src, static_cast<bf16*>(dst_bf16), ss, rows, width);
    else rows_sumsq_kernel<float, false><<<ceil_div(rows, 8), 256, 0, s>>>(src, static_cast<bf16*>(dst_bf16), ss, rows, width);
    return check_launch("convert_rows_sumsq");
}

sfb_status sfb_k_row_sumsq(const void* x_bf16, float* ss, int rows, int width, sfb_stream stream) {
    SFB_REQUIRE(x_bf16 && ss && rows > 0 && width > 0, "row sums of squares: empty tensor");
    cudaStream_t s = as_stream(stream);
    const bf16* x = static_cast<const bf16*>(x_bf16);
    if (rows <= 128) rows_sumsq_kernel<bf16, true><<<rows, 256, 0, s>>>(x, nullptr, ss, rows, width);
    else rows_sumsq_kernel<bf16, false><<<ceil_div(rows, 8), 256, 0, s>>>(x, nullptr, ss, rows, width);
    return check_launch("row_sumsq");
}

sfb_status sfb_rope_table(int seq, int head_dim, float theta, float* cos_out, float* sin_out) {
    SFB_REQUIRE(seq > 0 && head_dim > 0 && cos_out && sin_out, "invalid rope table shape");
    const int half = head_dim / 2;
    for (int t = 0; t < seq; ++t)
        for (int d = 0; d + 1 < head_dim; d += 2) {
            const float frequency = std::pow(theta, -static_cast<float>(d) / static_cast<float>(head_dim));
            const float angle = static_cast<float>(t) * frequency;
            cos_out[static_cast<size_t>(t) * half + d / 2] = std::cos(angle);
            sin_out[static_cast<size_t>(t) * half + d / 2] = std::sin(angle);
        }
    return SFB_OK;
}

sfb_status sfb_k_rope_split(const void* fused, void* q, void* key, void* value,
                            const float* rope_cos, const float* rope_sin, int batch, int seq,
                            int q_heads, int kv_heads, int head_dim, sfb_dtype dtype,
                            sfb_stream stream) {
    SFB_REQUIRE(fused && q && key && value && rope_cos && rope_sin, "rope_split: null tensor");
    SFB_REQUIRE(batch > 0 && seq > 0 && q_heads > 0 && kv_heads > 0 && head_dim > 0 && head_dim % 2 == 0,
                "rope_split: head_dim must be even");
    const int64_t pairs = static_cast<int64_t>(batch) * seq * (q_heads + 2 * kv_heads) * head_dim / 2;
    const int block = 256, grid = grid_for(pairs, block);
    if (dtype == SFB_F32)
        rope_split_kernel<float><<<grid, block, 0, as_stream(stream)>>>(
            static_cast<const float*>(fused), static_cast<float*>(q), static_cast<float*>(key),
            static_cast<float*>(value), rope_cos, rope_sin, batch, seq, q_heads, kv_heads, head_dim);
    else
        rope_split_kernel<bf16><<<grid, block, 0, as_stream(stream)>>>(
            static_cast<const bf16*>(fused), static_cast<bf16*>(q), static_cast<bf16*>(key),
            static_cast<bf16*>(value), rope_cos, rope_sin, batch, seq, q_heads, kv_heads, head_dim);
    return check_launch("rope_split");
}

}  // extern "C"
