// Internal declarations shared by the backend's translation units. Nothing
// here is part of the ABI; include/gq.h is.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "gq.h"

namespace gq {

// Thrown inside the library, turned into GQ_ERR + message at the boundary.
struct Failure : std::runtime_error {
    using std::runtime_error::runtime_error;
};

[[noreturn]] void fail(const char* fmt, ...) __attribute__((format(printf, 1, 2)));

#define GQ_CUDA(expr)                                                                         \
    do {                                                                                      \
        cudaError_t gq_e_ = (expr);                                                           \
        if (gq_e_ != cudaSuccess) ::gq::fail("%s: %s", #expr, cudaGetErrorString(gq_e_));     \
    } while (0)

struct Buffer {
    void* ptr = nullptr;
    uint64_t bytes = 0;     // what the caller asked for
    uint64_t capacity = 0;  // what the allocation holds (pool bucket) — 0 for wrapped memory
    uint32_t mem = GQ_MEM_DEVICE;
    bool owned = true;
    uint32_t refs = 1;  // the handle itself + one per graph that retains it
    bool released = false;
    bool ipc = false;  // opened from another process's export: closed, not freed, on release
};

bool launch_gemv_q8_dp4a(cudaStream_t s, int sm_count, const float* x, uint64_t m, uint64_t k, const uint32_t* q, const float* scale,
                         const float* bias, uint64_t n, float* y);
bool launch_gemv_q4_dp4a(cudaStream_t s, int sm_count, const float* x, uint64_t m, uint64_t k, const uint32_t* q, const float* scale,
                         const float* zero, const float* bias, uint64_t n, uint64_t group, float* y);

}  // namespace gq

struct gq_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint64_t nodes = 0;                // operator launches recorded
    std::vector<gq_buf> retained;      // buffers the recorded work names
};

struct gq_ctx {
    std::mutex mutex;
    int device = 0;
    cudaDeviceProp prop{};
    cudaStream_t stream = nullptr;
    uint64_t next_handle = 1;
    std::unordered_map<gq_buf, gq::Buffer> buffers;
    std::multimap<uint64_t, void*> pool;  // capacity -> free block (GQ_MEM_DEVICE only)
    gq_stats stats{};
    bool launch_blocking = false;  // GQ_LAUNCH_BLOCKING=1: wait after every launch
    // capture state
    bool capturing = false;
    uint64_t capture_nodes = 0;
    std::vector<gq_buf> capture_retained;
    // A word in mapped host memory that kernels with bounded waits write when a wait gives up; the
    // host checks it whenever it waits for the stream.
    uint32_t* status_host = nullptr;
    uint32_t* status_dev = nullptr;
    // What the last operation put on the stream wrote, when that operation was one of this library's kernels whose
    // outputs are known (prev_known): a GEMV that follows may then fetch its weights before that kernel has finished,
    // provided they are none of these buffers.
    bool prev_known = false;
    gq_buf prev_written[4] = {0, 0, 0, 0};
    void* argmax_state = nullptr;  // keys and counters of gq_argmax_rows, zero between calls
    void* sample_state = nullptr;  // gq_sample's arrival ticket, zero between calls
    // How long a kernel waits for another GPU's data before it gives up and reports through the status word, in SM
    // clock cycles (gq_set_wait_limit_us).
    long long peer_wait_cycles = 4000000000ll;
    // Scratch of kernels that split K over CTAs (partial sums, arrival counters). Grow-only: a block that a captured
    // graph may name is kept until the context is destroyed.
    void* scratch = nullptr;
    uint64_t scratch_bytes = 0;
    std::vector<void*> retired_scratch;
};

namespace gq {

// Entry-point plumbing shared by the files that define extern "C" functions.
void set_last_error(const char* msg);
template <class F>
int32_t guarded(F&& f) {  // any exception -> GQ_ERR + thread-local message (gc_shim.cpp:343-354)
    try {
        f();
        return GQ_OK;
    } catch (const std::exception& e) {
        set_last_error(e.what());
    } catch (...) {
        set_last_error("unknown error");
    }
    return GQ_ERR;
}
struct Locked {  // serialises calls on a context and makes its device current
    gq_ctx* ctx;
    std::lock_guard<std::mutex> lock;
    explicit Locked(gq_ctx* c) : ctx(c ? c : (fail("null context"), c)), lock(c->mutex) {
        cudaError_t e = cudaSetDevice(c->device);
        if (e != cudaSuccess) fail("cudaSetDevice: %s", cudaGetErrorString(e));
    }
};
Buffer& lookup(gq_ctx* ctx, gq_buf h, const char* what);
// Gives back one reference to a buffer (a released handle's memory is freed with its last reference).
void drop_ref(gq_ctx* ctx, gq_buf h);
void check_dims(const char* op, uint64_t a, uint64_t b, uint64_t c = 1);


// ── launches that hide the launch latency behind the previous kernel ─────
// A kernel whose FIRST statement is GQ_GRID_DEP_SYNC() may be launched with launch_after(): its CTAs are scheduled
// as soon as the kernel before it in the stream lets them (programmatic stream serialization) and then wait, in
// hardware, until that kernel has finished and its writes are visible. Stream-order semantics are unchanged (nothing
// is read or written before the wait); what is saved is the launch gap. A kernel lets the one behind it start only AFTER its
// own wait has returned, so whatever runs early in that next kernel knows that everything up to the kernel before this one is
// complete: the only writes in doubt are this kernel's own. Inside a capture the edge is recorded as such.
#ifdef __CUDACC__
#define GQ_GRID_DEP_SYNC()                                                  \
    do {                                                                    \
        asm volatile("griddepcontrol.wait;" ::: "memory");                  \
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");     \
    } while (0)

template <typename... KArgs, typename... Args>
void launch_after(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr, cfg.numAttrs = 1;
    GQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}
#endif

// A checked view of `count` elements of `elem` bytes at element offset `off`.
void* view(gq_ctx* ctx, gq_buf buf, uint64_t off, uint64_t count, uint64_t elem, const char* what);
// True when two device ranges share a byte. The linears read x from many CTAs while others already write y (and, in the
// fused forms, h_out), so an output that overlaps an input would be read half-updated: the entry points refuse it.
inline bool ranges_overlap(const void* a, uint64_t a_bytes, const void* b, uint64_t b_bytes) {
    if (!a || !b || !a_bytes || !b_bytes) return false;
    const char* pa = static_cast<const char*>(a);
    const char* pb = static_cast<const char*>(b);
    return pa < pb + b_bytes && pb < pa + a_bytes;
}
// Counts a launch, notes buffers for an open capture, honours launch_blocking.
void after_launch(gq_ctx* ctx, const char* kernel, std::initializer_list<gq_buf> used, std::initializer_list<gq_buf> written = {});
// True when none of `weights` was written by the operation before this one on the stream (and that operation is known).
bool weights_settled(const gq_ctx* ctx, std::initializer_list<gq_buf> weights);

// ── kernels (each file states which reference shader it replaces) ─────────
void launch_quantize_q8(cudaStream_t s, const float* w, uint64_t rows, uint64_t k, uint32_t* q, float* scale);
void launch_dequantize_q8(cudaStream_t s, const uint32_t* q, const float* scale, uint64_t rows, uint64_t k, float* w);
void launch_quantize_q4(cudaStream_t s, const float* w, uint64_t rows, uint64_t k, uint64_t group, uint32_t* q,
                        float* scale, float* zero);
// The frozen-weight backward (backward.cu): grad_x = grad . dequantize(W) with the weight dequantized on the fly in shared
// memory, and the column sums of grad for the bias.
void launch_linear_backward_q8(cudaStream_t s, const float* g, uint64_t m, const uint32_t* q, const float* scale, uint64_t n, uint64_t k, float* gx);
void launch_linear_backward_q4(cudaStream_t s, const float* g, uint64_t m, const uint32_t* q, const float* scale, const float* zero, uint64_t n,
                               uint64_t k, uint64_t group, float* gx);
void launch_column_sum(cudaStream_t s, const float* g, uint64_t m, uint64_t n, float* out);
void launch_dequantize_q4(cudaStream_t s, const uint32_t* q, const float* scale, const float* zero, uint64_t rows,
                          uint64_t k, uint64_t group, float* w);
void launch_fill_u32(cudaStream_t s, uint32_t* dst, uint64_t n, uint32_t word);
void launch_gemv_q8(cudaStream_t s, int sm_count, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                    const float* scale, const float* bias, uint64_t n, float* y);
void launch_gemv_q4(cudaStream_t s, int sm_count, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                    const float* scale, const float* zero, const float* bias, uint64_t n, uint64_t group, float* y);

bool launch_gemv_q8_dp4a(cudaStream_t s, int sm_count, const float* x, uint64_t m, uint64_t k, const uint32_t* q, const float* scale,
                         const float* bias, uint64_t n, float* y);
bool launch_gemv_q4_dp4a(cudaStream_t s, int sm_count, const float* x, uint64_t m, uint64_t k, const uint32_t* q, const float* scale,
                         const float* zero, const float* bias, uint64_t n, uint64_t group, float* y);

bool launch_gemv_q8_imma(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                         const float* scale, const float* bias, uint64_t n, float* y, bool weights_settled);
struct Prologue;
// A column-sharded layer's gather: every rank's receive buffer (peer-mapped, this rank's own included) of
// 2 x m_total x n_full 64-bit words (step << 32 | float bits; the halves alternate by step parity), this rank's plain
// y_full [m_total][n_full], and this rank's two state words (the step of the last finished call, the CTAs done).
// A call covers rows [row0, row0 + rows) of y.
struct PeerOut {
    unsigned long long* ll[8] = {};
    float* y_full = nullptr;
    uint32_t* state = nullptr;
    uint32_t nranks = 0, rank = 0, n_full = 0, m_total = 0, row0 = 0;
    long long wait_cycles = 0;
};
bool launch_gemv_q8_imma_fused(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t k, const uint32_t* q,
                               const float* scale, const float* bias, uint64_t n, float* y, int kind, const Prologue& pro, bool weights_settled);
bool launch_gemv_q4_ring(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                          const float* scale, const float* zero, const float* bias, uint64_t n, uint64_t group, float* y,
                         bool overlap_previous, bool x_settled, const PeerOut* peer = nullptr);
bool launch_gemv_q4_imma(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                         const float* scale, const float* zero, const float* bias, uint64_t n, uint64_t group, float* y,
                         bool weights_settled);

// int4 group-128 decode on tcgen05 for 1 to 16 rows of x in one pass (gemv_umma4.cu). The scratch holds the K slices'
// partial sums and the per-tile arrival counters (zero between launches).
uint64_t gemv_q4_umma_scratch_bytes(uint64_t m, uint64_t k, uint64_t n, int sm_count);
// `deferred`, when given: the sum over the K slices is left to the caller — *deferred receives the number of slices (their
// partial sums lie at gemv_q4_umma_partials(scratch, ...), bias NOT added), or 0 when K was not split and y (with bias) is complete.
bool launch_gemv_q4_lanes(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                          const float* scale, const float* zero, const float* bias, uint64_t n, uint64_t group, float* y, void* scratch,
                          uint32_t* deferred = nullptr);
void gemv_q4_lanes_shape(uint64_t n, uint64_t k, int sm_count, uint32_t* kslices, uint32_t* stages_per_cta);
bool launch_gemv_q4_umma(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                         const float* scale, const float* zero, const float* bias, uint64_t n, uint64_t group, float* y, void* scratch,
                         uint32_t* deferred = nullptr);
const float* gemv_q4_umma_partials(const void* scratch, uint64_t m, uint64_t k, uint64_t n, int sm_count);
// Zeroed device memory owned by the context, grown (never shrunk or moved while graphs may name it) on demand.
void* context_scratch(gq_ctx* ctx, uint64_t bytes);

bool launch_gemv_q8_tc(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                       const float* scale, const float* bias, uint64_t n, float* y);

bool launch_gemm_q8_tc(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                       const float* scale, const float* bias, uint64_t n, float* y);
// The same product in exact integer arithmetic (kind::i8 against three digit planes of x); `scratch` holds
// gemm_q8_i8_scratch_bytes(m, k) bytes.
uint64_t gemm_q8_i8_scratch_bytes(uint64_t m, uint64_t k);
bool launch_gemm_q8_i8(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                       const float* scale, const float* bias, uint64_t n, float* y, void* scratch);
// Rows of x from which AUTO takes the tf32 tensor-core GEMM when the integer one cannot run (its scratch would have to
// grow inside a capture).
constexpr uint64_t kTensorMinRows = 64;

// multi-GPU (sharded.cu)
void comm_unique_id(void* out128);
gq_comm* comm_create(int nranks, int rank, const void* id128);
void comm_destroy(gq_comm* c);
void comm_info(gq_comm* c, int* nranks, int* rank);
void all_gather_columns(cudaStream_t s, gq_comm* c, const float* src, float* dst, uint64_t m, uint64_t n_shard);
void launch_peer_gather(cudaStream_t s, int sm_count, const PeerOut& peer, const float* src, uint64_t m, uint64_t n_shard, uint32_t* status,
                        uint32_t slices = 0, const float* bias = nullptr);

// GPTQ (gptq.cu)
void launch_hessian_add(cudaStream_t s, const float* x, uint64_t rows, uint64_t k, float* h);
uint64_t gptq_error_floats(uint64_t n);
void launch_gptq(cudaStream_t s, float* w, const float* u, uint64_t n, uint64_t k, uint64_t group, float* err, uint32_t* q, float* scale, float* zero);

// decode-step operators (decode_ops.cu)
void launch_embedding(cudaStream_t s, const float* table, const int32_t* ids, uint64_t rows, uint64_t width, uint64_t vocab, float* out);
void launch_add_rms_norm(cudaStream_t s, const float* x, const float* res, const float* w, uint64_t rows, uint64_t n, float eps,
                         float* y, float* h);
void launch_rope_kv_append(cudaStream_t s, const float* qkv, const float* cosv, const float* sinv, const uint32_t* lens, uint32_t layer,
                           uint32_t heads, uint32_t kv_heads, uint32_t dim, uint32_t max_len, float* q_out, float* kc, float* vc);
void launch_kv_advance(cudaStream_t s, uint32_t* lens, uint32_t layers, uint32_t max_len);
uint32_t attn_splits(uint32_t heads, uint32_t max_len, int sm_count);
uint64_t attn_scratch_floats(uint32_t heads, uint32_t dim, uint32_t splits);
void launch_attn_decode(cudaStream_t s, const float* q, float* kc, float* vc, const uint32_t* lens, uint32_t layer, uint32_t heads,
                        uint32_t kv_heads, uint32_t dim, uint32_t max_len, float scale, uint32_t splits, float* scratch, float* out,
                        const float* cosv = nullptr, const float* sinv = nullptr, bool early = false);
void launch_rope_append_rows(cudaStream_t s, const float* qkv, const float* cosv, const float* sinv, const uint32_t* lens, uint32_t layer,
                             uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t dim, uint32_t max_len, float* q_out, void* kc, void* vc,
                             float* kscale, float* vscale, bool int8_cache);
void launch_attn_prefill(cudaStream_t s, const float* q, const void* kc, const void* vc, const float* kscale, const float* vscale,
                         const uint32_t* lens, uint32_t layer, uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t dim, uint32_t max_len,
                         float scale, float* out, bool int8_cache);
void launch_kv_advance_by(cudaStream_t s, uint32_t* lens, uint32_t layers, uint32_t max_len, uint32_t count);
void launch_swiglu(cudaStream_t s, const float* gate_up, uint64_t rows, uint64_t width, float* out);
uint64_t sample_state_bytes();
void launch_sample(cudaStream_t s, const float* logits, uint64_t rows, uint64_t v, int32_t* history, uint64_t hist_cap, uint32_t* hist_len,
                   bool do_sample, float temperature, uint64_t top_k, float one_minus_p, float penalty, const float* uniforms,
                   uint64_t uniform_rows, uint32_t* draws, float* scores, float* ex, int32_t* tokens, float* probs, bool append, void* state);
uint64_t argmax_state_bytes();
void launch_argmax_rows(cudaStream_t s, const float* v, uint64_t rows, uint64_t n, int32_t* out, void* state);

}  // namespace gq
