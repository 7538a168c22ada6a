// Column-sharded linear across the GPUs of one box: every rank owns a block of
// output features (rows of W are independent, so each rank's weights quantize
// exactly as the whole would) and computes y[:, block]; the blocks are then
// gathered so that every rank holds y[m][n_full]. The reference has no
// multi-GPU code (it runs on one Vulkan device); this is new.
//
// Two gathers:
//  * gq_all_gather_columns — NCCL over NVLink/NVSwitch. One ncclAllGather per
//    row of y inside a group: a rank's receive buffer for row r is row r of
//    y_full itself, so no transpose is needed. NCCL is loaded with dlopen the
//    first time a communicator is made; a single-GPU process never needs it.
//  * gq_peer_gather — this library's own put-and-signal collective over
//    peer-mapped memory (CUDA IPC): each rank stores its block straight into
//    every peer's y_full with ordinary peer stores, fences, and bumps a
//    counter in the peer's flag buffer; then waits — with a bound, reporting
//    through the context's status word — until every peer's counter has
//    reached this step. For the <= 230 KB this path moves it is latency, not
//    bandwidth, that matters, and a store + flag is one NVLink traversal.
//    No TMA and no multicast is involved: plain st.global to a peer pointer.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>

#include "async_common.cuh"
#include "gq_internal.h"

struct gq_comm {
    ncclComm_t comm = nullptr;
    int nranks = 0, rank = 0;
};

namespace gq {

namespace {

struct Nccl {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

Nccl& nccl() {
    static Nccl n;
    if (!n.lib) {
        n.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (!n.lib) fail("NCCL is needed for multi-GPU gathers but libnccl.so.2 could not be loaded: %s", dlerror());
        auto sym = [&](const char* name) {
            void* p = dlsym(n.lib, name);
            if (!p) fail("libnccl.so.2 lacks %s", name);
            return p;
        };
        n.GetUniqueId = reinterpret_cast<decltype(n.GetUniqueId)>(sym("ncclGetUniqueId"));
        n.CommInitRank = reinterpret_cast<decltype(n.CommInitRank)>(sym("ncclCommInitRank"));
        n.CommDestroy = reinterpret_cast<decltype(n.CommDestroy)>(sym("ncclCommDestroy"));
        n.AllGather = reinterpret_cast<decltype(n.AllGather)>(sym("ncclAllGather"));
        n.GroupStart = reinterpret_cast<decltype(n.GroupStart)>(sym("ncclGroupStart"));
        n.GroupEnd = reinterpret_cast<decltype(n.GroupEnd)>(sym("ncclGroupEnd"));
        n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(sym("ncclGetErrorString"));
    }
    return n;
}

void nccl_check(ncclResult_t r, const char* what) {
    if (r != ncclSuccess) fail("%s: %s", what, nccl().GetErrorString(r));
}

constexpr int kMaxRanks = 8;
constexpr uint32_t kPeerBlocks = 8;  // CTAs that copy (and signal) per destination rank
struct PeerArgs {
    float* y[kMaxRanks];         // every rank's y_full (own included), peer-mapped
    uint32_t* flag[kMaxRanks];   // every rank's counters, one per source rank
};

// grid = (blocks_per_peer, nranks): CTA (b, p) copies this rank's block into rank p's y_full, then
// signals. CTA (0, rank) afterwards waits for the peers' signals.
__global__ void __launch_bounds__(256) peer_gather_kernel(PeerArgs args, const float* __restrict__ src, uint32_t m, uint32_t n_shard,
                                                         uint32_t n_full, uint32_t rank, uint32_t nranks, uint32_t* status) {
    const uint32_t p = blockIdx.y;
    float* dst = args.y[p] + (size_t)rank * n_shard;
    const uint32_t total = m * n_shard;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const uint32_t r = i / n_shard, c = i - r * n_shard;
        dst[(size_t)r * n_full + c] = src[i];
    }
    __threadfence_system();  // the stores above are visible system-wide before the signal below
    __syncthreads();
    if (threadIdx.x == 0) atomicAdd_system(args.flag[p] + rank, 1u);
    if (p == rank && blockIdx.x == 0) {
        // The step number lives in the flag buffer (word nranks), so a captured launch counts on by
        // itself at every replay. Every source rank signals gridDim.x times per step.
        uint32_t* step_word = args.flag[rank] + nranks;
        const uint32_t step = *step_word + 1;
        __syncthreads();
        if (threadIdx.x < nranks) {
            const uint32_t want = step * gridDim.x;
            volatile uint32_t* f = args.flag[rank] + threadIdx.x;
            const long long start = clock64();
            while ((int32_t)(*f - want) < 0) {
                if (clock64() - start > 4000000000ll) {  // ~2 s: give up, tell the host
                    atomicCAS(status, 0u, 16u + threadIdx.x);
                    break;
                }
            }
            __threadfence_system();
        }
        __syncthreads();
        if (threadIdx.x == 0) *step_word = step;
    }
}

}  // namespace

void comm_unique_id(void* out128) {
    ncclUniqueId id;
    nccl_check(nccl().GetUniqueId(&id), "ncclGetUniqueId");
    memcpy(out128, &id, sizeof id);
}

gq_comm* comm_create(int nranks, int rank, const void* id128) {
    if (nranks < 1 || nranks > kMaxRanks || rank < 0 || rank >= nranks) fail("gq_comm_create: rank %d of %d is out of range (at most %d ranks)", rank, nranks, kMaxRanks);
    ncclUniqueId id;
    memcpy(&id, id128, sizeof id);
    auto c = new gq_comm();
    c->nranks = nranks, c->rank = rank;
    ncclResult_t r = nccl().CommInitRank(&c->comm, nranks, id, rank);
    if (r != ncclSuccess) {
        delete c;
        nccl_check(r, "ncclCommInitRank");
    }
    return c;
}

void comm_destroy(gq_comm* c) {
    if (!c) return;
    if (c->comm) nccl().CommDestroy(c->comm);
    delete c;
}

void comm_info(gq_comm* c, int* nranks, int* rank) { *nranks = c->nranks, *rank = c->rank; }

// y_full[r][rank * n_shard + c] = y_shard(rank)[r][c] on every rank.
void all_gather_columns(cudaStream_t s, gq_comm* c, const float* src, float* dst, uint64_t m, uint64_t n_shard) {
    const uint64_t n_full = n_shard * c->nranks;
    nccl_check(nccl().GroupStart(), "ncclGroupStart");
    for (uint64_t r = 0; r < m; ++r)
        nccl_check(nccl().AllGather(src + r * n_shard, dst + r * n_full, n_shard, ncclFloat, c->comm, s), "ncclAllGather");
    nccl_check(nccl().GroupEnd(), "ncclGroupEnd");
}

void launch_peer_gather(cudaStream_t s, float* const* y, uint32_t* const* flag, const float* src, uint64_t m, uint64_t n_shard,
                        int rank, int nranks, uint32_t* status) {
    PeerArgs args{};
    for (int i = 0; i < nranks; ++i) args.y[i] = y[i], args.flag[i] = flag[i];
    // a fixed CTA count per destination, so that the signals expected per step never depend on the size
    peer_gather_kernel<<<dim3(kPeerBlocks, nranks), 256, 0, s>>>(args, src, (uint32_t)m, (uint32_t)n_shard, (uint32_t)(n_shard * nranks),
                                                          (uint32_t)rank, (uint32_t)nranks, status);
}

}  // namespace gq
