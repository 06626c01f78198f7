// Sum all-reduce over NVLink peer memory for the sharded decoder layer, fused with the GEMM that
// produces the partial sums.
//
// Every rank owns a receive buffer with one slot per rank.  The O and Down projections of a
// tensor-parallel plan (gemm_tcgen05.cu) store each finished output piece twice from their
// epilogue: into the local partial-sum buffer and, with plain peer stores, into this rank's slot of
// every other rank's receive buffer, so the transfer runs tile by tile under the GEMM.  The
// kernel below then (1) publishes "my partial sums are in your slot" with a system-scope release
// store of an epoch number into every peer's flag array, (2) waits, with a bound, for the same
// epoch from every peer and (3) replaces the local partial sums by the sum over all ranks, taken
// in rank order so that every rank computes bit-identical results.
//
// Each rank pushes (size - 1) x bytes: this is the form for small messages (decode) and for two
// ranks; larger groups with large outputs should use a two-shot collective instead.
//
// Reuse of a slot is safe without further handshakes when the same sequence of collectives
// runs on every rank: a rank starts pushing use n+1 of a slot only after it has passed the wait
// of a later collective on another slot set, which its peers signal after they have finished
// reading use n (stream order on the peer).  The decoder plan alternates two slot sets.
#include <algorithm>
#include <cstring>

#include "common.cuh"

namespace sfb {
namespace {

constexpr long long kPeerWaitCycles = 4000000000LL;  // ~2 s; then the status word is set and the sum is skipped
constexpr uint32_t kCodePeerWait = 0x100;

__device__ __forceinline__ void store_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

struct PeerParams {
    bf16* data;
    const bf16* recv;
    uint32_t* local_flags;
    uint32_t* peer_flags[SFB_MAX_PEERS];
    int rank, size;
    uint32_t epoch;
    long long count;
    long long slot_elems;
    uint32_t* status;
};

__global__ void __launch_bounds__(256)
peer_allreduce_finish_kernel(const PeerParams p) {
    __shared__ int proceed;
    if (blockIdx.x == 0 && threadIdx.x < p.size && static_cast<int>(threadIdx.x) != p.rank) {
        __threadfence_system();  // the partial sums pushed by the preceding GEMM come before the flag
        store_release_sys(p.peer_flags[threadIdx.x], p.epoch);
    }
    if (threadIdx.x == 0) {
        bool ok = true;
        const long long start = clock64();
        for (int s = 0; s < p.size && ok; ++s) {
            if (s == p.rank) continue;
            uint32_t spins = 0;
            while (static_cast<int>(load_acquire_sys(p.local_flags + s) - p.epoch) < 0) {
                if ((++spins & 0xFFu) == 0 && clock64() - start > kPeerWaitCycles) {
                    ok = false;
                    atomicOr(p.status, kCodePeerWait);
                    break;
                }
            }
        }
        proceed = ok ? 1 : 0;
    }
    __syncthreads();
    if (!proceed) return;
    const long long pieces = p.count / 8;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < pieces; i += stride) {
        float acc[8] = {0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F};
        for (int s = 0; s < p.size; ++s) {  // rank order: the same arithmetic on every rank
            const bf16* src = s == p.rank ? p.data : p.recv + s * p.slot_elems;
            const uint4 packed = *reinterpret_cast<const uint4*>(src + i * 8);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&packed);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 x = __bfloat1622float2(h[j]);
                acc[2 * j] += x.x;
                acc[2 * j + 1] += x.y;
            }
        }
        uint4 result;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&result);
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        *reinterpret_cast<uint4*>(p.data + i * 8) = result;
    }
    // ragged tail (count % 8), one thread
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        for (long long i = pieces * 8; i < p.count; ++i) {
            float acc = 0.0F;
            for (int s = 0; s < p.size; ++s) acc += to_float((s == p.rank ? p.data : p.recv + s * p.slot_elems)[i]);
            p.data[i] = from_float<bf16>(acc);
        }
    }
}

// ---- two-shot form: reduce-scatter by the GEMM epilogues, sum + all-gather by the row owners ---------
// Rank r owns rows [r * rows_own, (r + 1) * rows_own) of the [T, width] tensor.  The producing GEMM of every
// rank stores each finished output piece ONLY into its slot of the owner's receive buffer (sfb_gemm_args.
// scatter_out), so a rank sends (size - 1) / size of the tensor instead of (size - 1) times the tensor.  The
// kernel below runs on the owner: it (A) tells every peer that its partial sums have been delivered and waits
// for the same from them, then one warp per owned row adds the `slots` partial rows in rank order (fp32), adds
// the owner's rows of the residual stream, rounds to bf16, takes the row's sum of squares (the RMSNorm of the
// next GEMM is folded into that GEMM and only needs 1/rms), stores the finished row into its own copy of the
// full tensor and, with plain peer stores, into every other rank's copy (the all-gather), and (B) the block that
// finishes last tells every peer that this rank's rows have arrived and waits for theirs.  With slots == 0 the
// rows are taken from `source` as they are: an all-gather of rows each rank already holds (the layer input).
// Both waits are bounded; when one gives up the status word is set and the kernel returns.
struct GatherParams {
    const bf16* slot[SFB_MAX_PEERS];  // partial rows of rank s for this owner's row range (local slots, or peers' buffers)
    int slots;
    const bf16* source;
    const bf16* residual;
    bf16* gathered[SFB_MAX_PEERS];
    float* ss[SFB_MAX_PEERS];
    const float* source_ss;
    uint32_t* local_flags_a;
    uint32_t* local_flags_b;
    uint32_t* peer_flags_a[SFB_MAX_PEERS];
    uint32_t* peer_flags_b[SFB_MAX_PEERS];
    uint32_t* done_counter;
    int rank, size;
    uint32_t epoch;
    int rows_own, width, gather;
    uint32_t* epoch_out;  // optional: receives the epoch (the word a copy engine then hands to the peers as "rows sent")
    uint32_t* status;
};

__device__ __forceinline__ bool wait_peers(const uint32_t* flags, int rank, int size, uint32_t epoch, uint32_t* status) {
    const long long start = clock64();
    for (int s = 0; s < size; ++s) {
        if (s == rank) continue;
        uint32_t spins = 0;
        while (static_cast<int>(load_acquire_sys(flags + s) - epoch) < 0) {
            if ((++spins & 0xFFu) == 0 && clock64() - start > kPeerWaitCycles) {
                atomicOr(status, kCodePeerWait);
                return false;
            }
        }
    }
    return true;
}

__global__ void __launch_bounds__(256)
peer_reduce_gather_kernel(const GatherParams p) {
    __shared__ int proceed;
    if (blockIdx.x == 0 && threadIdx.x < p.size && static_cast<int>(threadIdx.x) != p.rank) {
        __threadfence_system();  // the partial sums pushed by the preceding GEMM come before the flag
        store_release_sys(p.peer_flags_a[threadIdx.x], p.epoch);
    }
    if (threadIdx.x == 0) proceed = wait_peers(p.local_flags_a, p.rank, p.size, p.epoch, p.status) ? 1 : 0;
    __syncthreads();
    if (!proceed) return;
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int pieces = p.width / 8;  // width % 8 == 0
    for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < p.rows_own; row += warps) {
        const size_t local = static_cast<size_t>(row) * p.width;
        const size_t global = (static_cast<size_t>(p.rank) * p.rows_own + row) * p.width;
        float sumsq = 0.0F;
        // Two 16-byte pieces per lane and pass, and every load of a pass is issued before the first value is used:
        // a peer load takes microseconds, so the bytes in flight per warp decide the NVLink rate.
        for (int c0 = lane; c0 < pieces; c0 += 64) {
            const int piece[2] = {c0, c0 + 32};
            const int live = piece[1] < pieces ? 2 : 1;
            uint4 packed[2][SFB_MAX_PEERS], extra[2], base[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (u >= live) break;
                if (p.slots == 0) base[u] = *reinterpret_cast<const uint4*>(p.source + local + piece[u] * 8);
#pragma unroll
                for (int s = 0; s < SFB_MAX_PEERS; ++s)
                    if (s < p.slots) packed[u][s] = *reinterpret_cast<const uint4*>(p.slot[s] + local + piece[u] * 8);
                if (p.residual) extra[u] = *reinterpret_cast<const uint4*>(p.residual + local + piece[u] * 8);
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (u >= live) break;
                float acc[8] = {0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F};
                auto add = [&](const uint4& value) {
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&value);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 x = __bfloat1622float2(h[j]);
                        acc[2 * j] += x.x;
                        acc[2 * j + 1] += x.y;
                    }
                };
                if (p.slots == 0) add(base[u]);
#pragma unroll
                for (int s = 0; s < SFB_MAX_PEERS; ++s) {  // rank order: one arithmetic everywhere
                    if (s >= p.slots) break;
                    add(packed[u][s]);
                }
                if (p.residual) add(extra[u]);
                uint4 result;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&result);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    h[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                    const float2 r = __bfloat1622float2(h[j]);
                    sumsq = fmaf(r.x, r.x, sumsq);
                    sumsq = fmaf(r.y, r.y, sumsq);
                }
                *reinterpret_cast<uint4*>(p.gathered[p.rank] + global + piece[u] * 8) = result;
                if (p.gather)
                    for (int s = 0; s < p.size; ++s)
                        if (s != p.rank) *reinterpret_cast<uint4*>(p.gathered[s] + global + piece[u] * 8) = result;  // peer stores over NVLink
            }
        }
        if (p.ss[p.rank]) {
            sumsq = p.source_ss ? p.source_ss[row] : warp_sum(sumsq);
            if (lane == 0) {
                const size_t at = static_cast<size_t>(p.rank) * p.rows_own + row;
                p.ss[p.rank][at] = sumsq;
                if (p.gather)
                    for (int s = 0; s < p.size; ++s)
                        if (s != p.rank) p.ss[s][at] = sumsq;
            }
        }
    }
    if (!p.gather) {
        if (p.epoch_out && blockIdx.x == 0 && threadIdx.x == 0) *p.epoch_out = p.epoch;
        return;
    }
    // (B) the last block to finish announces this rank's rows and waits for the peers' rows
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t ticket = atomicAdd(p.done_counter, 1u);
        proceed = ticket == gridDim.x - 1 ? 1 : 0;
    }
    __syncthreads();
    if (!proceed) return;
    if (threadIdx.x == 0) *p.done_counter = 0;
    if (threadIdx.x < p.size && static_cast<int>(threadIdx.x) != p.rank) {
        __threadfence_system();
        store_release_sys(p.peer_flags_b[threadIdx.x], p.epoch);
    }
    if (threadIdx.x == 0) wait_peers(p.local_flags_b, p.rank, p.size, p.epoch, p.status);
}

// Bounded wait until every peer's flag has reached `epoch` (one thread): the end of an all-gather whose rows were
// moved by copy engines, placed in the stream before the first kernel that needs all rows.
__global__ void peer_wait_kernel(const uint32_t* flags, int rank, int size, uint32_t epoch, uint32_t* status) {
    if (threadIdx.x == 0 && blockIdx.x == 0) wait_peers(flags, rank, size, epoch, status);
}

}  // namespace
}  // namespace sfb

using namespace sfb;

extern "C" {

sfb_status sfb_k_peer_allreduce_finish(const sfb_peer_allreduce_args* a, sfb_stream stream) {
    SFB_REQUIRE(a && a->data && a->recv && a->local_flags, "peer all-reduce: null buffer");
    SFB_REQUIRE(a->size >= 2 && a->size <= SFB_MAX_PEERS && a->rank >= 0 && a->rank < a->size && a->count > 0 &&
                    a->slot_elems >= a->count,
                "peer all-reduce: invalid group or size");
    SFB_REQUIRE((reinterpret_cast<uintptr_t>(a->data) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->recv) & 15) == 0 &&
                    a->slot_elems % 8 == 0,
                "peer all-reduce: buffers must be 16-byte aligned");
    PeerParams p{};
    p.data = static_cast<bf16*>(a->data);
    p.recv = static_cast<const bf16*>(a->recv);
    p.local_flags = a->local_flags;
    for (int s = 0; s < a->size; ++s) {
        SFB_REQUIRE(s == a->rank || a->peer_flags[s], "peer all-reduce: null peer flag");
        p.peer_flags[s] = a->peer_flags[s];
    }
    p.rank = a->rank;
    p.size = a->size;
    p.epoch = a->epoch;
    p.count = a->count;
    p.slot_elems = a->slot_elems;
    p.status = device_status_word();
    const long long pieces = a->count / 8 + 1;
    const int grid = static_cast<int>(std::min<long long>((pieces + 255) / 256, static_cast<long long>(sm_count()) * 4));
    peer_allreduce_finish_kernel<<<grid, 256, 0, as_stream(stream)>>>(p);
    return check_launch("peer_allreduce_finish");
}

sfb_status sfb_k_peer_reduce_gather(const sfb_peer_gather_args* a, sfb_stream stream) {
    SFB_REQUIRE(a && a->local_flags && a->done_counter, "peer reduce-gather: null buffer");
    SFB_REQUIRE(a->size >= 2 && a->size <= SFB_MAX_PEERS && a->rank >= 0 && a->rank < a->size && a->rows_own > 0 &&
                    a->width > 0 && a->width % 8 == 0 && a->slots >= 0 && a->slots <= a->size,
                "peer reduce-gather: invalid group or shape");
    SFB_REQUIRE(a->slots == 0 ? a->source != nullptr
                              : (a->pull[0] != nullptr || (a->recv != nullptr && a->slot_elems >= static_cast<int64_t>(a->rows_own) * a->width &&
                                                           a->slot_elems % 8 == 0)),
                "peer reduce-gather: missing source rows or receive slots");
    SFB_REQUIRE(a->gathered[a->rank], "peer reduce-gather: null destination");
    GatherParams p{};
    p.slots = a->slots;
    for (int s = 0; s < a->slots; ++s) {
        p.slot[s] = a->pull[0] ? static_cast<const bf16*>(a->pull[s]) : static_cast<const bf16*>(a->recv) + s * a->slot_elems;
        SFB_REQUIRE(p.slot[s] && (reinterpret_cast<uintptr_t>(p.slot[s]) & 15) == 0, "peer reduce-gather: null or misaligned partial rows");
    }
    p.source = static_cast<const bf16*>(a->source);
    p.residual = static_cast<const bf16*>(a->residual);
    p.source_ss = a->source_ss;
    for (int s = 0; s < a->size; ++s) {
        if (a->gather) SFB_REQUIRE(a->gathered[s] && (a->ss[a->rank] == nullptr || a->ss[s]), "peer reduce-gather: null peer destination");
        SFB_REQUIRE(s == a->rank || a->peer_flags[s], "peer reduce-gather: null peer flag");
        SFB_REQUIRE((reinterpret_cast<uintptr_t>(a->gathered[s]) & 15) == 0, "peer reduce-gather: buffers must be 16-byte aligned");
        p.gathered[s] = static_cast<bf16*>(a->gathered[s]);
        p.ss[s] = a->ss[s];
        // two flags per peer and collective: [0] partial sums delivered, [1] finished rows delivered
        p.peer_flags_a[s] = a->peer_flags[s];
        p.peer_flags_b[s] = a->peer_flags[s] ? a->peer_flags[s] + SFB_MAX_PEERS : nullptr;
    }
    p.local_flags_a = a->local_flags;
    p.local_flags_b = a->local_flags + SFB_MAX_PEERS;
    p.done_counter = a->done_counter;
    p.rank = a->rank;
    p.size = a->size;
    p.epoch = a->epoch;
    p.rows_own = a->rows_own;
    p.width = a->width;
    p.gather = a->gather;
    p.epoch_out = a->epoch_out;
    p.status = device_status_word();
    const int blocks = std::min((a->rows_own + 7) / 8, sm_count() * 4);
    peer_reduce_gather_kernel<<<blocks, 256, 0, as_stream(stream)>>>(p);
    return check_launch("peer_reduce_gather");
}

sfb_status sfb_k_flag_wait(const uint32_t* flag, uint32_t epoch, sfb_stream stream) {
    SFB_REQUIRE(flag, "flag wait: null flag");
    peer_wait_kernel<<<1, 32, 0, as_stream(stream)>>>(flag, -1, 1, epoch, device_status_word());
    return check_launch("flag_wait");
}

sfb_status sfb_k_peer_wait(const uint32_t* local_flags, int rank, int size, uint32_t epoch, sfb_stream stream) {
    SFB_REQUIRE(local_flags && size >= 2 && size <= SFB_MAX_PEERS && rank >= 0 && rank < size, "peer wait: invalid group");
    peer_wait_kernel<<<1, 32, 0, as_stream(stream)>>>(local_flags, rank, size, epoch, device_status_word());
    return check_launch("peer_wait");
}

// ---- peer-visible device memory (CUDA IPC) -----------------------------------------------------

sfb_status sfb_peer_alloc(size_t bytes, void** ptr, void* handle64) {
    SFB_REQUIRE(bytes > 0 && ptr && handle64, "peer alloc: invalid argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    SFB_CUDA(cudaMalloc(ptr, bytes));
    SFB_CUDA(cudaMemset(*ptr, 0, bytes));
    SFB_CUDA(cudaDeviceSynchronize());
    cudaIpcMemHandle_t handle;
    SFB_CUDA(cudaIpcGetMemHandle(&handle, *ptr));
    memcpy(handle64, &handle, sizeof(handle));
    return SFB_OK;
}

sfb_status sfb_peer_open(const void* handle64, void** ptr) {
    SFB_REQUIRE(handle64 && ptr, "peer open: invalid argument");
    cudaIpcMemHandle_t handle;
    memcpy(&handle, handle64, sizeof(handle));
    SFB_CUDA(cudaIpcOpenMemHandle(ptr, handle, cudaIpcMemLazyEnablePeerAccess));
    return SFB_OK;
}

sfb_status sfb_peer_close(void* ptr) {
    if (ptr) SFB_CUDA(cudaIpcCloseMemHandle(ptr));
    return SFB_OK;
}

sfb_status sfb_peer_free(void* ptr) {
    if (ptr) SFB_CUDA(cudaFree(ptr));
    return SFB_OK;
}

}  // extern "C"
