// Host runtime helpers shared by the plan code: status -> exception bridge (the host layer
// throws the same exception types as the reference, the C wrappers turn them back into
// status codes), owned device memory, and the lifetime-based workspace planner.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "schedforge_b200.h"

namespace sfb {

// Raised for CUDA / device failures; carries the status the C wrapper should return.
struct DeviceError : std::runtime_error {
    sfb_status status;
    DeviceError(sfb_status s, const std::string& message) : std::runtime_error(message), status(s) {}
};

void throw_on(sfb_status status);             // status of a kernel entry point -> exception
void cuda_check(cudaError_t error, const char* what);

// C-wrapper side: run `body`, map exceptions to status codes and record the message.
template <class F>
sfb_status guarded(F&& body);

class DeviceBuffer {
public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(std::size_t bytes) { allocate(bytes); }
    ~DeviceBuffer() { release(); }
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    DeviceBuffer(DeviceBuffer&& other) noexcept : ptr_(other.ptr_), bytes_(other.bytes_) { other.ptr_ = nullptr; other.bytes_ = 0; }
    DeviceBuffer& operator=(DeviceBuffer&& other) noexcept {
        if (this != &other) { release(); ptr_ = other.ptr_; bytes_ = other.bytes_; other.ptr_ = nullptr; other.bytes_ = 0; }
        return *this;
    }
    void allocate(std::size_t bytes);
    void release();
    void* get() const { return ptr_; }
    template <class T> T* as() const { return static_cast<T*>(ptr_); }
    std::size_t bytes() const { return bytes_; }
private:
    void* ptr_ = nullptr;
    std::size_t bytes_ = 0;
};

// Assigns every intermediate tensor an offset inside ONE device workspace.  Two tensors
// may share bytes when their live ranges [first_step, last_step] do not overlap (the idea
// of the reference's GraphBufferizer: first-fit slot reuse over value lifetimes,
// src/graph_compiler.cpp:698-760).  Offsets are 1024-byte aligned (TMA tiles).
class WorkspacePlanner {
public:
    explicit WorkspacePlanner(bool reuse) : reuse_(reuse) {}
    int add(std::string name, std::size_t bytes, int first_step, int last_step);
    std::size_t offset(int id) const { return slots_.at(static_cast<std::size_t>(id)).offset; }
    std::size_t bytes(int id) const { return slots_.at(static_cast<std::size_t>(id)).bytes; }
    std::size_t total_bytes() const { return total_; }
    std::size_t naive_bytes() const { return naive_; }
    int find(const std::string& name) const;
private:
    struct Slot { std::string name; std::size_t offset, bytes; int first, last; };
    std::vector<Slot> slots_;
    std::size_t total_ = 0, naive_ = 0;
    bool reuse_;
};

// A caller-supplied routing trace goes to kernels that index shared and global memory with its expert ids and
// place rows by its counts, so it is checked on the host first (O(tokens * top_k)): all three arrays present,
// every id inside [0, experts), counts equal to the histogram of the ids.  Throws std::invalid_argument
// "routing trace does not match MoE configuration", the reference's message for a malformed trace
// (dispatch_tokens, src/moe_compiler.cpp:498-501).
void validate_routing_trace(int tokens, int top_k, int experts, const int* expert_ids, const float* expert_weights,
                            const int* counts);

// Host-side matrix shards used by the tensor-parallel plan build.
void shard_columns(const float* src, int rows, int cols, int rank, int size, float* dst);
void shard_rows(const float* src, int rows, int cols, int rank, int size, float* dst);

// Device: dst (bf16, [count_cols rows of packed layout][k_count]) = transpose of the fp32
// source block src[k_begin:k_begin+k_count, c_begin:c_begin+c_count] of a [*, src_cols]
// row-major matrix; source column c lands in destination row
// (c / block) * block_stride + block_offset + c % block.
void pack_weight_transposed(const float* src_device, int src_cols, int k_begin, int k_count, int c_begin,
                            int c_count, void* dst_bf16, int block, int block_stride, int block_offset,
                            cudaStream_t stream, const float* k_scale_device = nullptr);

// Whether the tensor-core GEMM takes these arguments (gemm_tcgen05.cu); the CUDA-core kernel covers the rest
// but knows neither the folded RMSNorm nor the paged K/V append of the RoPE epilogue.
bool gemm_bf16_tcgen05_supported(const sfb_gemm_args& args);

// first[i] *= silu(gate[i]) (fp32 MoE plan; defined in moe.cu).
void moe_silu_mul_f32(float* first, const float* gate, int64_t count, cudaStream_t stream);

}  // namespace sfb

#include <new>

namespace sfb {
void set_error(const std::string& message);

template <class F>
sfb_status guarded(F&& body) {
    try {
        body();
        return SFB_OK;
    } catch (const std::invalid_argument& e) {
        set_error(e.what());
        return SFB_INVALID_ARGUMENT;
    } catch (const DeviceError& e) {
        set_error(e.what());
        return e.status;
    } catch (const std::bad_alloc&) {
        set_error("host allocation failed");
        return SFB_RUNTIME_ERROR;
    } catch (const std::exception& e) {
        set_error(e.what());
        return SFB_RUNTIME_ERROR;
    }
}
}  // namespace sfb
