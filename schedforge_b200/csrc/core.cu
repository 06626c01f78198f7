// Error channel, launch accounting and the device status word shared by every
// translation unit of the library.
#include "common.cuh"

#include <atomic>
#include <mutex>

namespace sfb {
namespace {
thread_local std::string g_last_error;
std::atomic<uint64_t> g_launches{0};
constexpr int kMaxDevices = 64;
uint32_t* g_status_word[kMaxDevices] = {};  // one word per device, allocated with that device current
std::mutex g_status_mutex;
}  // namespace

void set_error(const std::string& message) { g_last_error = message; }

sfb_status fail(sfb_status status, const std::string& message) {
    g_last_error = message;
    return status;
}

sfb_status cuda_fail(cudaError_t error, const char* what) {
    g_last_error = std::string(what) + ": " + cudaGetErrorString(error);
    return SFB_CUDA_ERROR;
}

void count_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }

// One 4-byte word per device in that device's memory, zero-initialised.  Kernels with bounded
// waits OR a code into it when a wait runs out instead of spinning forever.  The word of the
// CURRENT device is returned, so a kernel always gets memory of the GPU it runs on.
uint32_t* device_status_word() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (!g_status_word[device]) {
        if (cudaMalloc(&g_status_word[device], sizeof(uint32_t)) != cudaSuccess) {
            g_status_word[device] = nullptr;
            return nullptr;
        }
        cudaMemset(g_status_word[device], 0, sizeof(uint32_t));
    }
    return g_status_word[device];
}

int sm_count() {
    static int cached = 0;
    if (cached == 0) {
        int device = 0, count = 0;
        if (cudaGetDevice(&device) == cudaSuccess &&
            cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && count > 0)
            cached = count;
        else
            return 148;
    }
    return cached;
}

}  // namespace sfb

extern "C" {

const char* sfb_last_error(void) { return sfb::g_last_error.c_str(); }

const char* sfb_version(void) { return "schedforge_b200 0.1.0 (sm_100a)"; }

uint64_t sfb_launch_count(void) { return sfb::g_launches.load(std::memory_order_relaxed); }

sfb_status sfb_device_status(uint32_t* status_word) {
    if (!status_word) return sfb::fail(SFB_INVALID_ARGUMENT, "null status pointer");
    uint32_t* word = sfb::device_status_word();
    if (!word) return sfb::fail(SFB_CUDA_ERROR, "no CUDA device");
    SFB_CUDA(cudaDeviceSynchronize());
    SFB_CUDA(cudaMemcpy(status_word, word, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    SFB_CUDA(cudaMemset(word, 0, sizeof(uint32_t)));
    return SFB_OK;
}

}  // extern "C"
