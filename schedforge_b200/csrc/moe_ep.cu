// Token-sharded expert parallelism for the MoE layer: all-to-all dispatch and combine over NVLink peer stores.
//
// Rank r owns tokens [r * rows_own, (r + 1) * rows_own) and the experts [r * E / size, (r + 1) * E / size).
// Every rank routes and dispatches ITS tokens locally (route_topk and the stable counting sort of
// dispatch_tokens, src/moe_compiler.cpp:412-455, 496-528, on rows_own tokens), then three kernels move the rows:
//
//   plan     every rank tells every rank its per-expert histogram; from the table counts_all[rank][expert] each rank
//            derives where its rows go and where the rows it receives come from.  Expert e's segment on its
//            owner holds rank 0's rows, then rank 1's, ... : because token ranges ascend with the rank and each
//            rank's rows are already in stable (token, slot) order, the segment is in the order the reference's
//            single-process dispatch_tokens produces.
//   send     one warp per locally dispatched row copies the (normalised) token row into the owner's receive
//            buffer at its final position, together with the global token id and the route slot;
//   return   after the grouped expert GEMMs one warp per received row copies the expert output back to the
//            source rank, to the row's position in that rank's LOCAL dispatched order, where the rank's own
//            weighted combine (moe_combine, expert-major order per token) finds it.
//
// Every kernel that hands data to peers ends with "announce + bounded wait" (the last block to finish publishes an
// epoch to every peer's flag array and waits for theirs), so the next kernel in the stream may read what the
// peers delivered.  No kernel waits for another kernel of the SAME GPU.  A wait that gives up sets bit 0x100 of
// the device status word and returns.
#include <algorithm>

#include "common.cuh"

namespace sfb {
namespace {

constexpr long long kPeerWaitCycles = 4000000000LL;  // ~2 s
constexpr uint32_t kCodePeerWait = 0x100;
constexpr int kMaxExperts = 64;

__device__ __forceinline__ void store_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

struct Sync {
    uint32_t* local_flags;                 // [s] written by rank s
    uint32_t* peer_flags[SFB_MAX_PEERS];   // entry [rank] of rank s's local_flags
    uint32_t* done_counter;
    uint32_t epoch;
    int rank, size;
    uint32_t* status;
};

// Called by every block at its end (all threads): the block that finishes last publishes the epoch to every peer and
// waits, with a bound, for every peer's epoch.
__device__ void announce_and_wait(const Sync& y) {
    __shared__ int last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(y.done_counter, 1u) == gridDim.x - 1 ? 1 : 0;
    __syncthreads();
    if (!last) return;
    if (threadIdx.x == 0) *y.done_counter = 0;
    if (static_cast<int>(threadIdx.x) < y.size && static_cast<int>(threadIdx.x) != y.rank) {
        __threadfence_system();
        store_release_sys(y.peer_flags[threadIdx.x], y.epoch);
    }
    if (threadIdx.x == 0) {
        const long long start = clock64();
        for (int s = 0; s < y.size; ++s) {
            if (s == y.rank) continue;
            uint32_t spins = 0;
            while (static_cast<int>(load_acquire_sys(y.local_flags + s) - y.epoch) < 0) {
                if ((++spins & 0xFFu) == 0 && clock64() - start > kPeerWaitCycles) {
                    atomicOr(y.status, kCodePeerWait);
                    return;
                }
            }
        }
    }
}

// The three tables of rank `rank` from the complete histogram table all[size][experts] (host and device).
//   send_base[e]       first row, in the receive buffer of expert e's owner, of THIS rank's rows of expert e: inside
//                      owner d the experts of d follow one another in ascending order, each holding the ranks' rows
//                      in ascending rank order;
//   recv_offsets[el]   segment starts of this rank's experts (the last entry is the number of received rows);
//   return_table       per (own expert, source rank): receive start, rows, source rank, first row of that expert's
//                      segment in the SOURCE's local dispatched order.
__host__ __device__ inline void ep_tables(const int* all, int size, int experts, int rank, int* send_base, int* recv_offsets,
                                          int* return_table) {
    const int local = experts / size;
    for (int d = 0; d < size; ++d) {
        int segment = 0;
        for (int e = d * local; e < (d + 1) * local; ++e) {
            int before = 0, total = 0;
            for (int s = 0; s < size; ++s) {
                if (s < rank) before += all[s * experts + e];
                total += all[s * experts + e];
            }
            send_base[e] = segment + before;
            segment += total;
        }
    }
    int start = 0, entry = 0;
    for (int el = 0; el < local; ++el) {
        const int e = rank * local + el;
        recv_offsets[el] = start;
        for (int s = 0; s < size; ++s) {
            int at_source = 0;
            for (int before = 0; before < e; ++before) at_source += all[s * experts + before];
            int* row = return_table + 4 * entry++;
            row[0] = start;
            row[1] = all[s * experts + e];
            row[2] = s;
            row[3] = at_source;
            start += all[s * experts + e];
        }
    }
    recv_offsets[local] = start;
}

struct PlanParams {
    const int* counts;                      // this rank's histogram [experts]
    int* counts_all[SFB_MAX_PEERS];         // every rank's table [size][experts] (index = rank that holds the table)
    int experts, experts_local;
    int* send_base;                         // [experts]: first destination row (on the expert's owner) of this rank's rows
    int* recv_offsets;                      // [experts_local + 1]: segment starts of this rank's experts
    int* return_table;                      // [experts_local * size][4]: receive start, rows, source rank, first row at the source
    Sync sync;
};

// One block.  Exchange of the histograms, then the three tables of this rank.
__global__ void __launch_bounds__(kMaxExperts)
ep_plan_kernel(const PlanParams p) {
    const int rank = p.sync.rank, size = p.sync.size, E = p.experts, El = p.experts_local;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int n = p.counts[e];
        for (int s = 0; s < size; ++s) p.counts_all[s][rank * E + e] = n;  // peer stores (and the local copy)
    }
    announce_and_wait(p.sync);   // one block: it is the last one
    __syncthreads();
    if (threadIdx.x != 0) return;
    ep_tables(p.counts_all[rank], size, E, rank, p.send_base, p.recv_offsets, p.return_table);
}

struct SendParams {
    const bf16* rows;              // this rank's normalised token rows [rows_own, hidden]
    const int* offsets;            // local dispatched order: segment starts [experts + 1]
    const int* token_ids;          // local token of every dispatched row
    const int* route_slots;
    const int* send_base;
    bf16* recv_rows[SFB_MAX_PEERS];
    int* recv_tokens[SFB_MAX_PEERS];
    int* recv_slots[SFB_MAX_PEERS];
    int assignments, hidden, experts, experts_local, first_token;
    Sync sync;
};

__global__ void __launch_bounds__(256)
ep_send_kernel(const SendParams p) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int pieces = p.hidden / 8;
    for (int a = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; a < p.assignments; a += warps) {
        int lo = 0, hi = p.experts;          // expert of dispatched row a: offsets[e] <= a < offsets[e + 1]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (p.offsets[mid] <= a) lo = mid; else hi = mid;
        }
        const int e = lo, owner = e / p.experts_local;
        const int dest = p.send_base[e] + (a - p.offsets[e]);
        const int token = p.token_ids[a];
        const uint4* src = reinterpret_cast<const uint4*>(p.rows + static_cast<size_t>(token) * p.hidden);
        uint4* dst = reinterpret_cast<uint4*>(p.recv_rows[owner] + static_cast<size_t>(dest) * p.hidden);
        for (int c = lane; c < pieces; c += 32) dst[c] = src[c];
        if (lane == 0) {
            p.recv_tokens[owner][dest] = p.first_token + token;
            p.recv_slots[owner][dest] = p.route_slots[a];
        }
    }
    announce_and_wait(p.sync);
}

struct ReturnParams {
    const bf16* rows;              // expert outputs in receive order [received, hidden]
    const int* recv_offsets;       // [experts_local + 1]; the last entry is the number of received rows
    const int* return_table;
    bf16* back[SFB_MAX_PEERS];     // every rank's buffer of expert outputs in ITS local dispatched order
    int hidden, experts_local;
    Sync sync;
};

__global__ void __launch_bounds__(256)
ep_return_kernel(const ReturnParams p) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int pieces = p.hidden / 8;
    const int received = p.recv_offsets[p.experts_local];
    const int entries = p.experts_local * p.sync.size;
    for (int j = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; j < received; j += warps) {
        int lo = 0, hi = entries;            // run of the table that holds received row j (runs may be empty)
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (p.return_table[4 * mid] <= j) lo = mid; else hi = mid;
        }
        const int* row = p.return_table + 4 * lo;
        const int source = row[2], at = row[3] + (j - row[0]);
        const uint4* src = reinterpret_cast<const uint4*>(p.rows + static_cast<size_t>(j) * p.hidden);
        uint4* dst = reinterpret_cast<uint4*>(p.back[source] + static_cast<size_t>(at) * p.hidden);
        for (int c = lane; c < pieces; c += 32) dst[c] = src[c];
    }
    announce_and_wait(p.sync);
}

Sync make_sync(const sfb_ep_sync& a, uint32_t* status) {
    Sync y{};
    y.local_flags = a.local_flags;
    for (int s = 0; s < SFB_MAX_PEERS; ++s) y.peer_flags[s] = a.peer_flags[s];
    y.done_counter = a.done_counter;
    y.epoch = a.epoch;
    y.rank = a.rank;
    y.size = a.size;
    y.status = status;
    return y;
}

bool sync_ok(const sfb_ep_sync& a) {
    if (!a.local_flags || !a.done_counter || a.size < 2 || a.size > SFB_MAX_PEERS || a.rank < 0 || a.rank >= a.size) return false;
    for (int s = 0; s < a.size; ++s)
        if (s != a.rank && !a.peer_flags[s]) return false;
    return true;
}

}  // namespace
}  // namespace sfb

using namespace sfb;

extern "C" {

sfb_status sfb_k_moe_ep_plan(const sfb_moe_ep_plan_args* a, sfb_stream stream) {
    SFB_REQUIRE(a && a->counts && a->send_base && a->recv_offsets && a->return_table && sync_ok(a->sync),
                "expert-parallel plan: null buffer or invalid group");
    SFB_REQUIRE(a->experts > 0 && a->experts <= kMaxExperts && a->experts % a->sync.size == 0,
                "expert-parallel plan: the experts must divide over the ranks (at most 64)");
    PlanParams p{};
    p.counts = a->counts;
    for (int s = 0; s < a->sync.size; ++s) {
        SFB_REQUIRE(a->counts_all[s], "expert-parallel plan: null histogram table");
        p.counts_all[s] = a->counts_all[s];
    }
    p.experts = a->experts;
    p.experts_local = a->experts / a->sync.size;
    p.send_base = a->send_base;
    p.recv_offsets = a->recv_offsets;
    p.return_table = a->return_table;
    p.sync = make_sync(a->sync, device_status_word());
    ep_plan_kernel<<<1, kMaxExperts, 0, as_stream(stream)>>>(p);
    return check_launch("moe_ep_plan");
}

sfb_status sfb_moe_ep_tables(const int* counts_all, int size, int experts, int rank, int* send_base, int* recv_offsets,
                             int* return_table) {
    SFB_REQUIRE(counts_all && send_base && recv_offsets && return_table, "expert-parallel tables: null buffer");
    SFB_REQUIRE(size >= 1 && size <= SFB_MAX_PEERS && rank >= 0 && rank < size && experts > 0 && experts % size == 0,
                "expert-parallel tables: the experts must divide over the ranks");
    ep_tables(counts_all, size, experts, rank, send_base, recv_offsets, return_table);
    return SFB_OK;
}

sfb_status sfb_k_moe_ep_send(const sfb_moe_ep_send_args* a, sfb_stream stream) {
    SFB_REQUIRE(a && a->rows && a->offsets && a->token_ids && a->route_slots && a->send_base && sync_ok(a->sync),
                "expert-parallel send: null buffer or invalid group");
    SFB_REQUIRE(a->assignments > 0 && a->hidden > 0 && a->hidden % 8 == 0 && a->experts > 0 && a->experts % a->sync.size == 0,
                "expert-parallel send: invalid shape");
    SendParams p{};
    p.rows = static_cast<const bf16*>(a->rows);
    p.offsets = a->offsets;
    p.token_ids = a->token_ids;
    p.route_slots = a->route_slots;
    p.send_base = a->send_base;
    for (int s = 0; s < a->sync.size; ++s) {
        SFB_REQUIRE(a->recv_rows[s] && a->recv_tokens[s] && a->recv_slots[s], "expert-parallel send: null receive buffer");
        p.recv_rows[s] = static_cast<bf16*>(a->recv_rows[s]);
        p.recv_tokens[s] = a->recv_tokens[s];
        p.recv_slots[s] = a->recv_slots[s];
    }
    p.assignments = a->assignments;
    p.hidden = a->hidden;
    p.experts = a->experts;
    p.experts_local = a->experts / a->sync.size;
    p.first_token = a->first_token;
    p.sync = make_sync(a->sync, device_status_word());
    const int blocks = std::min((a->assignments + 7) / 8, sm_count() * 8);
    ep_send_kernel<<<blocks, 256, 0, as_stream(stream)>>>(p);
    return check_launch("moe_ep_send");
}

sfb_status sfb_k_moe_ep_return(const sfb_moe_ep_return_args* a, sfb_stream stream) {
    SFB_REQUIRE(a && a->rows && a->recv_offsets && a->return_table && sync_ok(a->sync),
                "expert-parallel return: null buffer or invalid group");
    SFB_REQUIRE(a->hidden > 0 && a->hidden % 8 == 0 && a->experts_local > 0 && a->max_rows > 0, "expert-parallel return: invalid shape");
    ReturnParams p{};
    p.rows = static_cast<const bf16*>(a->rows);
    p.recv_offsets = a->recv_offsets;
    p.return_table = a->return_table;
    for (int s = 0; s < a->sync.size; ++s) {
        SFB_REQUIRE(a->back[s], "expert-parallel return: null destination");
        p.back[s] = static_cast<bf16*>(a->back[s]);
    }
    p.hidden = a->hidden;
    p.experts_local = a->experts_local;
    p.sync = make_sync(a->sync, device_status_word());
    const int blocks = std::min((a->max_rows + 7) / 8, sm_count() * 8);
    ep_return_kernel<<<blocks, 256, 0, as_stream(stream)>>>(p);
    return check_launch("moe_ep_return");
}

}  // extern "C"
