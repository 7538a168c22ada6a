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
//  * gq_peer_gather — this library's own collective over peer-mapped memory
//    (CUDA IPC). Each value of y travels as ONE 64-bit word, step << 32 | the
//    float's bits, stored with a single plain store into every rank's receive
//    buffer; a receiver knows a word has arrived when its upper half is the
//    step it is waiting for. There is no fence, no counter and no signal: one
//    NVLink traversal per value, which for the <= 230 KB this path moves is
//    what matters. The receiver's wait is bounded and reports through the
//    context's status word. The buffer has two halves that alternate by step
//    parity (a rank can be at most one step ahead of the slowest). No TMA and
//    no multicast is involved. gq_int4_linear_gather speaks the same protocol
//    from the GEMV's own epilogue (gemv_ring.cu), so the two may be mixed on
//    one set of buffers.
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

__device__ __forceinline__ void st_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Every CTA sends a slice of this rank's block to every rank, then receives a slice of the whole y.
// slices > 0: src holds `slices` partial results of m x n_shard floats each (the tcgen05 decode kernel's K slices); what is
// sent is their sum in slice order, plus bias.
__global__ void __launch_bounds__(256) peer_gather_kernel(PeerOut peer, const float* __restrict__ src, uint32_t m, uint32_t n_shard,
                                                         uint32_t slices, const float* __restrict__ bias, uint32_t* status) {
    const uint32_t step = *reinterpret_cast<const volatile uint32_t*>(peer.state) + 1u;  // the last CTA to finish writes it: every CTA has read it by then
    const size_t half = ((size_t)(step & 1u) * peer.m_total + peer.row0) * peer.n_full;
    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x, nthreads = gridDim.x * blockDim.x;
    for (uint32_t i = tid; i < m * n_shard; i += nthreads) {
        const uint32_t r = i / n_shard, c = i - r * n_shard;
        float value;
        if (slices == 0) {
            value = src[i];
        } else {
            float part[16];  // every slice's value is requested before the first is used
#pragma unroll
            for (uint32_t sl = 0; sl < 16; ++sl) part[sl] = sl < slices ? __ldcg(src + (size_t)sl * m * n_shard + i) : 0.0f;
            value = part[0];
#pragma unroll
            for (uint32_t sl = 1; sl < 16; ++sl)
                if (sl < slices) value = __fadd_rn(value, part[sl]);
            if (bias) value = __fadd_rn(value, bias[c]);
        }
        const unsigned long long word = ((unsigned long long)step << 32) | __float_as_uint(value);
        const size_t at = half + (size_t)r * peer.n_full + (size_t)peer.rank * n_shard + c;
        for (uint32_t pr = 0; pr < peer.nranks; ++pr) st_sys_u64(peer.ll[pr] + at, word);
    }
    const unsigned long long* mine = peer.ll[peer.rank] + half;
    const long long start = clock64();
    for (uint32_t i = tid; i < m * peer.n_full; i += nthreads) {
        unsigned long long v;
        for (;;) {
            v = ld_sys_u64(mine + i);
            if ((uint32_t)(v >> 32) == step) break;
            if (clock64() - start > peer.wait_cycles) {  // give up, tell the host which rank's words never came
                atomicCAS(status, 0u, kStatusPeerWaitTimedOut + (i % peer.n_full) / n_shard);
                break;
            }
        }
        peer.y_full[(size_t)peer.row0 * peer.n_full + i] = __uint_as_float((uint32_t)v);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(peer.state + 1, 1u) == gridDim.x - 1) {
            peer.state[1] = 0;
            peer.state[0] = step;
        }
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

void launch_peer_gather(cudaStream_t s, int sm_count, const PeerOut& peer, const float* src, uint64_t m, uint64_t n_shard, uint32_t* status,
                        uint32_t slices, const float* bias) {
    // all CTAs must be resident at once (a CTA waits for words other CTAs of this very launch send): at most one per SM
    const uint64_t work = m * n_shard * peer.nranks;
    uint64_t grid = (work + 1023) / 1024;
    if (grid > (uint64_t)sm_count) grid = sm_count;
    if (grid < 1) grid = 1;
    peer_gather_kernel<<<(uint32_t)grid, 256, 0, s>>>(peer, src, (uint32_t)m, (uint32_t)n_shard, slices, bias, status);
}

}  // namespace gq
