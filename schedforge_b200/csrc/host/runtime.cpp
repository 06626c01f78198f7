#include "runtime.hpp"

#include <cuda_bf16.h>

#include <algorithm>
#include <cstring>

#include "../common.cuh"

namespace sfb {

void throw_on(sfb_status status) {
    if (status == SFB_OK) return;
    const std::string message = sfb_last_error();
    if (status == SFB_INVALID_ARGUMENT) throw std::invalid_argument(message);
    throw DeviceError(status, message);
}

void cuda_check(cudaError_t error, const char* what) {
    if (error != cudaSuccess)
        throw DeviceError(SFB_CUDA_ERROR, std::string(what) + ": " + cudaGetErrorString(error));
}

void DeviceBuffer::allocate(std::size_t bytes) {
    release();
    if (bytes == 0) return;
    cuda_check(cudaMalloc(&ptr_, bytes), "cudaMalloc");
    bytes_ = bytes;
}

void DeviceBuffer::release() {
    if (ptr_) cudaFree(ptr_);
    ptr_ = nullptr;
    bytes_ = 0;
}

int WorkspacePlanner::add(std::string name, std::size_t bytes, int first_step, int last_step) {
    constexpr std::size_t kAlign = 1024;
    bytes = (bytes + kAlign - 1) / kAlign * kAlign;
    naive_ += bytes;
    std::size_t offset = 0;
    if (!reuse_) {
        offset = total_;
    } else {
        // first fit: lowest offset that does not collide with a tensor alive at the same time
        std::vector<std::pair<std::size_t, std::size_t>> busy;
        for (const auto& slot : slots_)
            if (!(slot.last < first_step || last_step < slot.first)) busy.emplace_back(slot.offset, slot.offset + slot.bytes);
        std::sort(busy.begin(), busy.end());
        for (const auto& [begin, end] : busy) {
            if (offset + bytes <= begin) break;
            offset = std::max(offset, end);
        }
    }
    slots_.push_back({std::move(name), offset, bytes, first_step, last_step});
    total_ = std::max(total_, offset + bytes);
    return static_cast<int>(slots_.size()) - 1;
}

int WorkspacePlanner::find(const std::string& name) const {
    for (std::size_t i = 0; i < slots_.size(); ++i)
        if (slots_[i].name == name) return static_cast<int>(i);
    return -1;
}

void shard_columns(const float* src, int rows, int cols, int rank, int size, float* dst) {
    const int width = cols / size;
    for (int r = 0; r < rows; ++r)
        std::memcpy(dst + static_cast<std::size_t>(r) * width,
                    src + static_cast<std::size_t>(r) * cols + static_cast<std::size_t>(rank) * width,
                    static_cast<std::size_t>(width) * sizeof(float));
}

void validate_routing_trace(int tokens, int top_k, int experts, const int* expert_ids, const float* expert_weights,
                            const int* counts) {
    const char* message = "routing trace does not match MoE configuration";
    if (!expert_ids || !expert_weights || !counts || tokens <= 0 || top_k <= 0 || experts <= 0)
        throw std::invalid_argument(message);
    std::vector<long long> histogram(static_cast<std::size_t>(experts), 0);
    const long long assignments = static_cast<long long>(tokens) * top_k;
    for (long long i = 0; i < assignments; ++i) {
        const int e = expert_ids[i];
        if (e < 0 || e >= experts) throw std::invalid_argument(message);
        ++histogram[static_cast<std::size_t>(e)];
    }
    for (int e = 0; e < experts; ++e)
        if (counts[e] != histogram[static_cast<std::size_t>(e)]) throw std::invalid_argument(message);
}

void shard_rows(const float* src, int rows, int cols, int rank, int size, float* dst) {
    const int height = rows / size;
    std::memcpy(dst, src + static_cast<std::size_t>(rank) * height * cols,
                static_cast<std::size_t>(height) * cols * sizeof(float));
}

namespace {

// 32x32 shared-memory tile transpose with fp32 -> bf16 conversion.
__global__ void pack_weight_kernel(const float* __restrict__ src, int src_cols, int k_begin, int k_count,
                                   int c_begin, int c_count, __nv_bfloat16* __restrict__ dst, int block,
                                   int block_stride, int block_offset, const float* __restrict__ k_scale) {
    __shared__ float tile[32][33];
    const int c0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int k = k0 + i, c = c0 + threadIdx.x;
        float v = (k < k_count && c < c_count) ? src[static_cast<size_t>(k_begin + k) * src_cols + c_begin + c] : 0.0F;
        if (k_scale && k < k_count) v *= k_scale[k_begin + k];  // a per-input-feature factor (folded norm weight)
        tile[i][threadIdx.x] = v;
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int c = c0 + i, k = k0 + threadIdx.x;
        if (c < c_count && k < k_count) {
            const size_t row = static_cast<size_t>(c / block) * block_stride + block_offset + c % block;
            dst[row * k_count + k] = __float2bfloat16_rn(tile[threadIdx.x][i]);
        }
    }
}

}  // namespace

void pack_weight_transposed(const float* src_device, int src_cols, int k_begin, int k_count, int c_begin,
                            int c_count, void* dst_bf16, int block, int block_stride, int block_offset,
                            cudaStream_t stream, const float* k_scale_device) {
    dim3 grid((c_count + 31) / 32, (k_count + 31) / 32), threads(32, 8);
    pack_weight_kernel<<<grid, threads, 0, stream>>>(src_device, src_cols, k_begin, k_count, c_begin, c_count,
                                                     static_cast<__nv_bfloat16*>(dst_bf16), block, block_stride,
                                                     block_offset, k_scale_device);
    count_launch();
    cuda_check(cudaGetLastError(), "pack_weight");
}

}  // namespace sfb

extern "C" {

sfb_status sfb_shard_columns(const float* src, int rows, int cols, int rank, int size, float* dst) {
    if (!src || !dst || rows <= 0 || cols <= 0 || size <= 0 || rank < 0 || rank >= size || cols % size != 0)
        return sfb::fail(SFB_INVALID_ARGUMENT, "invalid column shard request");
    sfb::shard_columns(src, rows, cols, rank, size, dst);
    return SFB_OK;
}

sfb_status sfb_shard_rows(const float* src, int rows, int cols, int rank, int size, float* dst) {
    if (!src || !dst || rows <= 0 || cols <= 0 || size <= 0 || rank < 0 || rank >= size || rows % size != 0)
        return sfb::fail(SFB_INVALID_ARGUMENT, "invalid row shard request");
    sfb::shard_rows(src, rows, cols, rank, size, dst);
    return SFB_OK;
}

}  // extern "C"
