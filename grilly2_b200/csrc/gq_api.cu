// The C ABI of include/gq.h: context, buffers, transfers, statistics,
// capture/replay, and the operator entry points, which validate their
// operands and hand device pointers to the kernel launchers.
//
// Conventions follow the reference's Vulkan shim
// (crates/grilly-sys/shim/gc_shim.cpp:343-354 `guarded`, :36 thread-local
// error, :52-339 context bookkeeping): every entry point runs inside
// guarded(), which turns any exception into GQ_ERR plus a message.
#include <chrono>
#include <cstdarg>
#include <cstdlib>
#include <cstring>

#include "gq_internal.h"
#include "async_common.cuh"

namespace gq {

static thread_local std::string g_last_error;

void fail(const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    throw Failure(buf);
}

void set_last_error(const char* msg) { g_last_error = msg; }

Buffer& lookup(gq_ctx* ctx, gq_buf h, const char* what) {
    auto it = ctx->buffers.find(h);
    if (h == 0 || it == ctx->buffers.end() || it->second.released) fail("%s: invalid buffer handle %llu", what, (unsigned long long)h);
    return it->second;
}

void* view(gq_ctx* ctx, gq_buf h, uint64_t off, uint64_t count, uint64_t elem, const char* what) {
    Buffer& b = lookup(ctx, h, what);
    // overflow-safe: off and count are element counts
    if (off > b.bytes / elem || count > b.bytes / elem - off)
        fail("%s: needs %llu elements of %llu bytes at element offset %llu, but the buffer holds %llu bytes", what,
             (unsigned long long)count, (unsigned long long)elem, (unsigned long long)off, (unsigned long long)b.bytes);
    return static_cast<char*>(b.ptr) + off * elem;
}

void check_dims(const char* op, uint64_t a, uint64_t b, uint64_t c) {
    const uint64_t max_dim = 0x7fffffffull;  // kernels index with 32-bit row/column counts
    if (a > max_dim || b > max_dim || c > max_dim) fail("%s: a dimension exceeds 2^31 - 1", op);
}

static uint64_t bucket_of(uint64_t bytes) {
    // pooled blocks come in power-of-two sizes from 512 B, as the reference's
    // pool does (gc_shim.h:37-41): a decode step's activations recycle.
    uint64_t cap = 512;
    while (cap < bytes) cap <<= 1;
    return cap;
}

void drop_ref(gq_ctx* ctx, gq_buf h) {
    auto it = ctx->buffers.find(h);
    if (it == ctx->buffers.end()) return;
    Buffer& b = it->second;
    if (--b.refs > 0) return;
    if (b.ipc && b.ptr) cudaIpcCloseMemHandle(b.ptr);
    if (b.owned && b.ptr) {
        if (b.mem == GQ_MEM_DEVICE_PERSISTENT) {
            cudaFree(b.ptr);  // waits for the device: nothing recorded can still be using it
            ctx->stats.persistent_buffers--;
            ctx->stats.persistent_bytes -= b.bytes;
        } else {
            // stream order makes reuse safe: the next user runs on the same stream
            ctx->pool.emplace(b.capacity, b.ptr);
        }
    }
    ctx->buffers.erase(it);
}

void after_launch(gq_ctx* ctx, const char* kernel, std::initializer_list<gq_buf> used, std::initializer_list<gq_buf> written) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) fail("launching %s: %s", kernel, cudaGetErrorString(e));
    ctx->stats.launches++;
    ctx->prev_known = written.size() > 0 && written.size() <= 4;
    for (auto& w : ctx->prev_written) w = 0;
    if (ctx->prev_known) {
        int i = 0;
        for (gq_buf h : written) ctx->prev_written[i++] = h;
    }
    if (ctx->capturing) {
        ctx->capture_nodes++;
        for (gq_buf h : used) {
            if (h == 0) continue;
            auto it = ctx->buffers.find(h);
            if (it == ctx->buffers.end()) continue;
            it->second.refs++;
            ctx->capture_retained.push_back(h);
        }
    } else if (ctx->launch_blocking) {
        e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) fail("%s failed on the device: %s", kernel, cudaGetErrorString(e));
    }
}

bool weights_settled(const gq_ctx* ctx, std::initializer_list<gq_buf> weights) {
    if (!ctx->prev_known) return false;
    for (gq_buf w : weights)
        for (gq_buf p : ctx->prev_written)
            if (w != 0 && w == p) return false;
    return true;
}

void* context_scratch(gq_ctx* ctx, uint64_t bytes) {
    if (ctx->scratch_bytes >= bytes) return ctx->scratch;
    if (ctx->capturing)
        fail("the context's scratch would have to grow to %llu bytes inside a capture: run the step once eagerly first "
             "(the reference records on the second sighting of a shape for the same reason, python/grilly/_graph.py:100-163)",
             (unsigned long long)bytes);
    uint64_t cap = 1ull << 20;
    while (cap < bytes) cap <<= 1;
    void* p = nullptr;
    GQ_CUDA(cudaMalloc(&p, cap));
    GQ_CUDA(cudaMemsetAsync(p, 0, cap, ctx->stream));
    if (ctx->scratch) ctx->retired_scratch.push_back(ctx->scratch);  // launches already on the stream, and graphs, may still name it
    ctx->scratch = p, ctx->scratch_bytes = cap;
    ctx->stats.buffer_allocations++;
    ctx->prev_known = false;
    return p;
}

static void host_wait(gq_ctx* ctx) {
    auto t0 = std::chrono::steady_clock::now();
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    uint64_t ns = (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0).count();
    ctx->stats.syncs++;
    ctx->stats.wait_ns_total += ns;
    ctx->stats.wait_ns_last = ns;
    if (e != cudaSuccess) fail("the device reported an error while the host waited: %s", cudaGetErrorString(e));
    if (ctx->status_host && *ctx->status_host) {
        const uint32_t code = *ctx->status_host;
        *ctx->status_host = 0;
        if (code >= kStatusPeerWaitTimedOut)
            fail("a gather gave up waiting for rank %u's block of the output (code %u = 16 + the rank; the limit is set by "
                 "gq_set_wait_limit_us); its results are not valid", code - kStatusPeerWaitTimedOut, code);
        fail("a kernel gave up a bounded wait (code %u: 1 = a bulk copy never landed, 2 = a pipeline stage was never freed, "
             "3 = the tensor cores never signalled completion, 4 = a grid-wide barrier was never completed); its results are not valid", code);
    }
}

static const char* const kCaptureRead =
    "a capture read data back to the host. A replay re-issues the recorded work without running the host code "
    "again, so nothing the host decides from a value can be reproduced: keep the value on the device, or leave "
    "that step out of the capture.";
static const char* const kCaptureWrite =
    "a capture wrote host data into a buffer. A replay re-issues the recorded work, so it would write those same "
    "bytes every time: put the value in a buffer and update it between replays instead, which is what a captured "
    "step's inputs are for.";

}  // namespace gq

using namespace gq;

extern "C" {

const char* gq_last_error(void) { return g_last_error.c_str(); }

int32_t gq_create(int32_t device, gq_ctx** out) {
    return guarded([&] {
        if (!out) fail("gq_create: null out pointer");
        *out = nullptr;
        int count = 0;
        cudaError_t e = cudaGetDeviceCount(&count);
        if (e != cudaSuccess || count == 0)
            fail("gq_create: no CUDA device is visible (%s). This backend has no CPU path.", e == cudaSuccess ? "device count 0" : cudaGetErrorString(e));
        if (device < 0 || device >= count) fail("gq_create: device %d out of range (0..%d)", device, count - 1);
        GQ_CUDA(cudaSetDevice(device));
        auto ctx = new gq_ctx();
        try {
            ctx->device = device;
            GQ_CUDA(cudaGetDeviceProperties(&ctx->prop, device));
            if (ctx->prop.major != 10)
                fail("gq_create: device %d (%s) is compute capability %d.%d; the kernels are built for sm_100a (B200) only", device,
                     ctx->prop.name, ctx->prop.major, ctx->prop.minor);
            GQ_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
            GQ_CUDA(cudaHostAlloc((void**)&ctx->status_host, 64, cudaHostAllocMapped));
            *ctx->status_host = 0;
            GQ_CUDA(cudaHostGetDevicePointer((void**)&ctx->status_dev, ctx->status_host, 0));
            GQ_CUDA(cudaMalloc(&ctx->argmax_state, argmax_state_bytes()));
            GQ_CUDA(cudaMemset(ctx->argmax_state, 0, argmax_state_bytes()));
            GQ_CUDA(cudaMalloc(&ctx->sample_state, sample_state_bytes()));
            GQ_CUDA(cudaMemset(ctx->sample_state, 0, sample_state_bytes()));
            const char* lb = getenv("GQ_LAUNCH_BLOCKING");
            ctx->launch_blocking = lb && lb[0] == '1';
        } catch (...) {
            delete ctx;
            throw;
        }
        *out = ctx;
    });
}

void gq_destroy(gq_ctx* ctx) {
    if (!ctx) return;
    guarded([&] {
        {
            std::lock_guard<std::mutex> lock(ctx->mutex);
            cudaSetDevice(ctx->device);
            cudaStreamSynchronize(ctx->stream);
            for (auto& kv : ctx->buffers) {
                if (kv.second.ipc && kv.second.ptr) cudaIpcCloseMemHandle(kv.second.ptr);
                if (kv.second.owned && kv.second.ptr) cudaFree(kv.second.ptr);
            }
            for (auto& kv : ctx->pool) cudaFree(kv.second);
            if (ctx->argmax_state) cudaFree(ctx->argmax_state);
            if (ctx->sample_state) cudaFree(ctx->sample_state);
            if (ctx->scratch) cudaFree(ctx->scratch);
            for (void* p : ctx->retired_scratch) cudaFree(p);
            if (ctx->status_host) cudaFreeHost(ctx->status_host);
            cudaStreamDestroy(ctx->stream);
        }
        delete ctx;
    });
}

int32_t gq_caps_get(gq_ctx* ctx, gq_caps* out) {
    return guarded([&] {
        Locked l(ctx);
        if (!out) fail("gq_caps_get: null out pointer");
        memset(out, 0, sizeof *out);
        snprintf(out->device_name, sizeof out->device_name, "%s", ctx->prop.name);
        out->cc_major = ctx->prop.major;
        out->cc_minor = ctx->prop.minor;
        out->sm_count = ctx->prop.multiProcessorCount;
        out->max_shared_per_block = (uint32_t)ctx->prop.sharedMemPerBlockOptin;
        out->total_memory = ctx->prop.totalGlobalMem;
        out->l2_bytes = ctx->prop.l2CacheSize;
    });
}

int32_t gq_buffer_create(gq_ctx* ctx, uint64_t bytes, uint32_t mem, gq_buf* out) {
    return guarded([&] {
        Locked l(ctx);
        if (!out) fail("gq_buffer_create: null out pointer");
        *out = 0;
        if (mem != GQ_MEM_DEVICE && mem != GQ_MEM_DEVICE_PERSISTENT) fail("gq_buffer_create: unknown memory class %u", mem);
        Buffer b;
        b.bytes = bytes;
        b.mem = mem;
        if (mem == GQ_MEM_DEVICE_PERSISTENT) {
            b.capacity = bytes;
            if (bytes) GQ_CUDA(cudaMalloc(&b.ptr, bytes));
            ctx->stats.buffer_allocations++;
            ctx->stats.persistent_buffers++;
            ctx->stats.persistent_bytes += bytes;
            if (ctx->stats.persistent_bytes > ctx->stats.persistent_peak) ctx->stats.persistent_peak = ctx->stats.persistent_bytes;
        } else {
            b.capacity = bucket_of(bytes);
            auto it = ctx->pool.find(b.capacity);
            if (it != ctx->pool.end()) {
                b.ptr = it->second;
                ctx->pool.erase(it);
                ctx->stats.pool_reuses++;
            } else {
                GQ_CUDA(cudaMalloc(&b.ptr, b.capacity));
                ctx->stats.buffer_allocations++;
            }
        }
        gq_buf h = ctx->next_handle++;
        ctx->buffers.emplace(h, b);
        ctx->stats.buffers_outstanding++;
        *out = h;
    });
}

int32_t gq_buffer_wrap(gq_ctx* ctx, void* device_ptr, uint64_t bytes, gq_buf* out) {
    return guarded([&] {
        Locked l(ctx);
        if (!out) fail("gq_buffer_wrap: null out pointer");
        *out = 0;
        if (!device_ptr && bytes) fail("gq_buffer_wrap: null device pointer");
        if (bytes) {
            cudaPointerAttributes attr{};
            cudaError_t e = cudaPointerGetAttributes(&attr, device_ptr);
            if (e != cudaSuccess || (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged)) {
                cudaGetLastError();
                fail("gq_buffer_wrap: %p is not device memory", device_ptr);
            }
        }
        Buffer b;
        b.ptr = device_ptr;
        b.bytes = bytes;
        b.owned = false;
        gq_buf h = ctx->next_handle++;
        ctx->buffers.emplace(h, b);
        ctx->stats.buffers_outstanding++;
        *out = h;
    });
}

int32_t gq_buffer_release(gq_ctx* ctx, gq_buf buf) {
    return guarded([&] {
        Locked l(ctx);
        Buffer& b = lookup(ctx, buf, "gq_buffer_release");
        b.released = true;  // the handle dies now; the memory when no graph names it
        ctx->stats.buffers_outstanding--;
        drop_ref(ctx, buf);
    });
}

int32_t gq_buffer_size(gq_ctx* ctx, gq_buf buf, uint64_t* out) {
    return guarded([&] {
        Locked l(ctx);
        if (!out) fail("gq_buffer_size: null out pointer");
        *out = lookup(ctx, buf, "gq_buffer_size").bytes;
    });
}

int32_t gq_buffer_ptr(gq_ctx* ctx, gq_buf buf, void** out) {
    return guarded([&] {
        Locked l(ctx);
        if (!out) fail("gq_buffer_ptr: null out pointer");
        *out = lookup(ctx, buf, "gq_buffer_ptr").ptr;
    });
}

int32_t gq_stream(gq_ctx* ctx, void** out) {
    return guarded([&] {
        Locked l(ctx);
        if (!out) fail("gq_stream: null out pointer");
        *out = (void*)ctx->stream;
    });
}

int32_t gq_upload(gq_ctx* ctx, gq_buf dst, uint64_t offset, const void* src, uint64_t bytes) {
    return guarded([&] {
        Locked l(ctx);
        if (ctx->capturing) fail("%s", kCaptureWrite);
        void* d = view(ctx, dst, offset, bytes, 1, "gq_upload");
        if (!bytes) return;
        if (!src) fail("gq_upload: null source");
        ctx->prev_known = false;
        GQ_CUDA(cudaMemcpyAsync(d, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
        GQ_CUDA(cudaStreamSynchronize(ctx->stream));
        ctx->stats.uploads++;
    });
}

int32_t gq_download(gq_ctx* ctx, gq_buf src, uint64_t offset, void* dst, uint64_t bytes) {
    return guarded([&] {
        Locked l(ctx);
        if (ctx->capturing) fail("%s", kCaptureRead);
        void* s = view(ctx, src, offset, bytes, 1, "gq_download");
        if (bytes) {
            if (!dst) fail("gq_download: null destination");
            ctx->prev_known = false;
            GQ_CUDA(cudaMemcpyAsync(dst, s, bytes, cudaMemcpyDeviceToHost, ctx->stream));
        }
        host_wait(ctx);
        ctx->stats.downloads++;
    });
}

int32_t gq_upload_async(gq_ctx* ctx, gq_buf dst, uint64_t offset, const void* src, uint64_t bytes) {
    return guarded([&] {
        Locked l(ctx);
        void* d = view(ctx, dst, offset, bytes, 1, "gq_upload_async");
        if (!bytes) return;
        if (!src) fail("gq_upload_async: null source");
        ctx->prev_known = false;
        GQ_CUDA(cudaMemcpyAsync(d, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
        ctx->stats.uploads++;
        if (ctx->capturing) {
            lookup(ctx, dst, "gq_upload_async").refs++;
            ctx->capture_retained.push_back(dst);
            ctx->capture_nodes++;
        }
    });
}

int32_t gq_download_async(gq_ctx* ctx, gq_buf src, uint64_t offset, void* dst, uint64_t bytes) {
    return guarded([&] {
        Locked l(ctx);
        void* s = view(ctx, src, offset, bytes, 1, "gq_download_async");
        if (!bytes) return;
        if (!dst) fail("gq_download_async: null destination");
        ctx->prev_known = false;
        GQ_CUDA(cudaMemcpyAsync(dst, s, bytes, cudaMemcpyDeviceToHost, ctx->stream));
        ctx->stats.downloads++;
        if (ctx->capturing) {
            lookup(ctx, src, "gq_download_async").refs++;
            ctx->capture_retained.push_back(src);
            ctx->capture_nodes++;
        }
    });
}

int32_t gq_host_alloc(gq_ctx* ctx, uint64_t bytes, void** out) {
    return guarded([&] {
        Locked l(ctx);
        if (!out) fail("gq_host_alloc: null out pointer");
        *out = nullptr;
        GQ_CUDA(cudaMallocHost(out, bytes ? bytes : 1));
    });
}

int32_t gq_host_free(gq_ctx* ctx, void* ptr) {
    return guarded([&] {
        Locked l(ctx);
        if (ptr) GQ_CUDA(cudaFreeHost(ptr));
    });
}

int32_t gq_copy(gq_ctx* ctx, gq_buf src, uint64_t src_offset, gq_buf dst, uint64_t dst_offset, uint64_t bytes) {
    return guarded([&] {
        Locked l(ctx);
        if ((src_offset | dst_offset | bytes) & 3) fail("gq_copy: offsets and size must be multiples of 4");
        void* s = view(ctx, src, src_offset, bytes, 1, "gq_copy source");
        void* d = view(ctx, dst, dst_offset, bytes, 1, "gq_copy destination");
        if (!bytes) return;
        ctx->prev_known = false;
        GQ_CUDA(cudaMemcpyAsync(d, s, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
        after_launch(ctx, "copy", {src, dst});
    });
}

int32_t gq_fill(gq_ctx* ctx, gq_buf dst, uint64_t offset, uint64_t bytes, uint32_t word) {
    return guarded([&] {
        Locked l(ctx);
        if ((offset | bytes) & 3) fail("gq_fill: offset and size must be multiples of 4");
        void* d = view(ctx, dst, offset, bytes, 1, "gq_fill");
        if (!bytes) return;
        launch_fill_u32(ctx->stream, (uint32_t*)d, bytes / 4, word);
        after_launch(ctx, "fill", {dst});
    });
}

int32_t gq_synchronize(gq_ctx* ctx) {
    return guarded([&] {
        Locked l(ctx);
        if (ctx->capturing) fail("%s", kCaptureRead);
        host_wait(ctx);
    });
}

int32_t gq_set_wait_limit_us(gq_ctx* ctx, uint64_t microseconds) {
    return guarded([&] {
        Locked l(ctx);
        // prop.clockRate is the SM clock in kHz: cycles = us * kHz / 1000
        const uint64_t us = microseconds ? microseconds : 2000000ull;
        if (us > 3600ull * 1000000ull) fail("gq_set_wait_limit_us: at most one hour");
        ctx->peer_wait_cycles = (long long)(us * (uint64_t)(ctx->prop.clockRate > 0 ? ctx->prop.clockRate : 1965000) / 1000ull);
    });
}

int32_t gq_stats_get(gq_ctx* ctx, gq_stats* out) {
    return guarded([&] {
        Locked l(ctx);
        if (!out) fail("gq_stats_get: null out pointer");
        *out = ctx->stats;
    });
}

int32_t gq_persistent_peak_reset(gq_ctx* ctx) {
    return guarded([&] {
        Locked l(ctx);
        ctx->stats.persistent_peak = ctx->stats.persistent_bytes;
    });
}

// ── operators ────────────────────────────────────────────────────────────

static uint64_t words8(uint64_t k) { return (k + 15) / 16 * 4; }
static uint64_t words4(uint64_t k) { return (k + 31) / 32 * 4; }
static const uint64_t kMaxDim = 0x7fffffffull;

static void check_group(uint64_t group) {
    // crates/grilly-infer/src/quant4.rs:99-103
    if (group == 0 || group % 32 != 0) fail("int4 group_size must be a positive multiple of 32, got %llu", (unsigned long long)group);
    if (group > kMaxDim) fail("int4 group_size exceeds 2^31 - 1");
}

int32_t gq_int8_quantize(gq_ctx* ctx, gq_buf w, uint64_t w_off, uint64_t rows, uint64_t k, gq_buf q, gq_buf scale) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_int8_quantize", rows, k);
        if (k == 0) fail("cannot quantize a weight with no input features");  // quant.rs:106-110
        auto wp = (const float*)view(ctx, w, w_off, rows * k, 4, "gq_int8_quantize weight");
        auto qp = (uint32_t*)view(ctx, q, 0, rows * words8(k), 4, "gq_int8_quantize q");
        auto sp = (float*)view(ctx, scale, 0, rows, 4, "gq_int8_quantize scale");
        if (rows == 0) return;
        launch_quantize_q8(ctx->stream, wp, rows, k, qp, sp);
        after_launch(ctx, "quantize_q8", {w, q, scale});
    });
}

int32_t gq_int8_quantize_rows(gq_ctx* ctx, gq_buf w, uint64_t w_off, uint64_t rows, uint64_t k, gq_buf q, gq_buf scale, uint64_t row0,
                              uint64_t total_rows) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_int8_quantize_rows", rows, k, total_rows);
        if (k == 0) fail("cannot quantize a weight with no input features");
        if (row0 > total_rows || rows > total_rows - row0)
            fail("gq_int8_quantize_rows: rows %llu..%llu do not fit a weight of %llu rows", (unsigned long long)row0,
                 (unsigned long long)(row0 + rows), (unsigned long long)total_rows);
        auto wp = (const float*)view(ctx, w, w_off, rows * k, 4, "gq_int8_quantize_rows weight");
        auto qp = (uint32_t*)view(ctx, q, 0, total_rows * words8(k), 4, "gq_int8_quantize_rows q");
        auto sp = (float*)view(ctx, scale, 0, total_rows, 4, "gq_int8_quantize_rows scale");
        if (rows == 0) return;
        launch_quantize_q8(ctx->stream, wp, rows, k, qp + row0 * words8(k), sp + row0);
        after_launch(ctx, "quantize_q8", {w, q, scale});
    });
}

int32_t gq_int4_quantize_rows(gq_ctx* ctx, gq_buf w, uint64_t w_off, uint64_t rows, uint64_t k, uint64_t group, gq_buf q, gq_buf scale, gq_buf zero,
                              uint64_t row0, uint64_t total_rows) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_int4_quantize_rows", rows, k, total_rows);
        if (k == 0) fail("cannot quantize a weight with no input features");
        check_group(group);
        if (row0 > total_rows || rows > total_rows - row0)
            fail("gq_int4_quantize_rows: rows %llu..%llu do not fit a weight of %llu rows", (unsigned long long)row0,
                 (unsigned long long)(row0 + rows), (unsigned long long)total_rows);
        const uint64_t groups = (k + group - 1) / group;
        auto wp = (const float*)view(ctx, w, w_off, rows * k, 4, "gq_int4_quantize_rows weight");
        auto qp = (uint32_t*)view(ctx, q, 0, total_rows * words4(k), 4, "gq_int4_quantize_rows q");
        auto sp = (float*)view(ctx, scale, 0, total_rows * groups, 4, "gq_int4_quantize_rows scale");
        auto zp = (float*)view(ctx, zero, 0, total_rows * groups, 4, "gq_int4_quantize_rows zero");
        if (rows == 0) return;
        launch_quantize_q4(ctx->stream, wp, rows, k, group, qp + row0 * words4(k), sp + row0 * groups, zp + row0 * groups);
        after_launch(ctx, "quantize_q4", {w, q, scale, zero});
    });
}

int32_t gq_int8_dequantize(gq_ctx* ctx, gq_buf q, gq_buf scale, uint64_t rows, uint64_t k, gq_buf w) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_int8_dequantize", rows, k);
        auto qp = (const uint32_t*)view(ctx, q, 0, rows * words8(k), 4, "gq_int8_dequantize q");
        auto sp = (const float*)view(ctx, scale, 0, rows, 4, "gq_int8_dequantize scale");
        auto wp = (float*)view(ctx, w, 0, rows * k, 4, "gq_int8_dequantize weight");
        if (rows == 0 || k == 0) return;
        launch_dequantize_q8(ctx->stream, qp, sp, rows, k, wp);
        after_launch(ctx, "dequantize_q8", {q, scale, w});
    });
}

int32_t gq_int8_linear_backward(gq_ctx* ctx, gq_buf grad, uint64_t g_off, uint64_t m, gq_buf q, gq_buf scale, uint64_t n, uint64_t k, gq_buf grad_x,
                                gq_buf grad_bias) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_int8_linear_backward", m, k, n);
        auto gp = (const float*)view(ctx, grad, g_off, m * n, 4, "gq_int8_linear_backward grad");
        auto qp = (const uint32_t*)view(ctx, q, 0, n * words8(k), 4, "gq_int8_linear_backward q");
        auto sp = (const float*)view(ctx, scale, 0, n, 4, "gq_int8_linear_backward scale");
        auto xp = grad_x ? (float*)view(ctx, grad_x, 0, m * k, 4, "gq_int8_linear_backward grad_x") : nullptr;
        auto bp = grad_bias ? (float*)view(ctx, grad_bias, 0, n, 4, "gq_int8_linear_backward grad_bias") : nullptr;
        if ((xp && ranges_overlap(xp, m * k * 4, gp, m * n * 4)) || (bp && ranges_overlap(bp, n * 4, gp, m * n * 4)))
            fail("gq_int8_linear_backward: the outputs must not overlap grad");
        if (xp && m && k) launch_linear_backward_q8(ctx->stream, gp, m, qp, sp, n, k, xp);
        if (bp && n) launch_column_sum(ctx->stream, gp, m, n, bp);
        after_launch(ctx, "linear_backward_q8", {grad, q, scale, grad_x, grad_bias});
    });
}

int32_t gq_int4_linear_backward(gq_ctx* ctx, gq_buf grad, uint64_t g_off, uint64_t m, gq_buf q, gq_buf scale, gq_buf zero, uint64_t n, uint64_t k,
                                uint64_t group, gq_buf grad_x, gq_buf grad_bias) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_int4_linear_backward", m, k, n);
        check_group(group);
        const uint64_t groups = (k + group - 1) / group;
        auto gp = (const float*)view(ctx, grad, g_off, m * n, 4, "gq_int4_linear_backward grad");
        auto qp = (const uint32_t*)view(ctx, q, 0, n * words4(k), 4, "gq_int4_linear_backward q");
        auto sp = (const float*)view(ctx, scale, 0, n * groups, 4, "gq_int4_linear_backward scale");
        auto zp = (const float*)view(ctx, zero, 0, n * groups, 4, "gq_int4_linear_backward zero");
        auto xp = grad_x ? (float*)view(ctx, grad_x, 0, m * k, 4, "gq_int4_linear_backward grad_x") : nullptr;
        auto bp = grad_bias ? (float*)view(ctx, grad_bias, 0, n, 4, "gq_int4_linear_backward grad_bias") : nullptr;
        if ((xp && ranges_overlap(xp, m * k * 4, gp, m * n * 4)) || (bp && ranges_overlap(bp, n * 4, gp, m * n * 4)))
            fail("gq_int4_linear_backward: the outputs must not overlap grad");
        if (xp && m && k) launch_linear_backward_q4(ctx->stream, gp, m, qp, sp, zp, n, k, group, xp);
        if (bp && n) launch_column_sum(ctx->stream, gp, m, n, bp);
        after_launch(ctx, "linear_backward_q4", {grad, q, scale, zero, grad_x, grad_bias});
    });
}

int32_t gq_int8_linear(gq_ctx* ctx, gq_buf x, uint64_t x_off, uint64_t m, uint64_t k, gq_buf q, gq_buf scale,
                       gq_buf bias, uint64_t b_off, uint64_t n, gq_buf y, int32_t kernel) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_int8_linear", m, k, n);
        if (kernel < GQ_KERNEL_AUTO || (kernel > GQ_KERNEL_UMMA && kernel != GQ_KERNEL_TENSOR_I8)) fail("gq_int8_linear: unknown kernel selector %d", kernel);
        auto xp = (const float*)view(ctx, x, x_off, m * k, 4, "gq_int8_linear input");
        auto qp = (const uint32_t*)view(ctx, q, 0, n * words8(k), 4, "gq_int8_linear q");
        auto sp = (const float*)view(ctx, scale, 0, n, 4, "gq_int8_linear scale");
        auto bp = bias ? (const float*)view(ctx, bias, b_off, n, 4, "gq_int8_linear bias") : nullptr;
        auto yp = (float*)view(ctx, y, 0, m * n, 4, "gq_int8_linear output");
        if (ranges_overlap(yp, m * n * 4, xp, m * k * 4)) fail("gq_int8_linear: the output must not overlap the input (CTAs read x while others write y)");
        if (m == 0 || n == 0) return;  // quant.rs:267-269
        bool done = false;
        const char* name = "gemv_q8";
        // AUTO: the integer tensor-core kernel from three rows of x on (at three rows only where the weight is 8 MB and more:
        // measured, dp4a still wins on the small projections there); one or two rows stay with the streaming IMMA kernel
        const bool auto_i8 = kernel == GQ_KERNEL_AUTO && (m >= 4 || (m == 3 && n * k >= (8ull << 20)));
        if (kernel == GQ_KERNEL_TENSOR_I8 || auto_i8) {
            // (a scratch that would have to grow inside a capture leaves AUTO to the tf32 kernel, which needs none)
            const uint64_t need = gemm_q8_i8_scratch_bytes(m, k);
            if (kernel == GQ_KERNEL_TENSOR_I8 || !(ctx->capturing && ctx->scratch_bytes < need))
                done = launch_gemm_q8_i8(ctx->stream, ctx->prop.multiProcessorCount, ctx->status_dev, xp, m, k, qp, sp, bp, n, yp, context_scratch(ctx, need));
            if (done) name = "gemm_i8_q8", ctx->stats.launches += 1;  // the digit planes of x ahead of it
            if (!done && kernel == GQ_KERNEL_TENSOR_I8)
                fail("gq_int8_linear: the integer tensor-core GEMM takes in_features up to 131072 (k = %llu)", (unsigned long long)k);
        }
        if (!done && (kernel == GQ_KERNEL_TENSOR || (kernel == GQ_KERNEL_AUTO && m >= kTensorMinRows))) {
            done = launch_gemm_q8_tc(ctx->stream, ctx->prop.multiProcessorCount, ctx->status_dev, xp, m, k, qp, sp, bp, n, yp);
            if (done) name = "gemm_tf32_q8";
            if (!done && kernel == GQ_KERNEL_TENSOR)
                fail("gq_int8_linear: the tensor-core GEMM needs in_features %% 4 == 0 and x on a 16-byte boundary (k = %llu, x_off = %llu)",
                     (unsigned long long)k, (unsigned long long)x_off);
        }
        if (!done && kernel == GQ_KERNEL_UMMA) {
            done = launch_gemv_q8_tc(ctx->stream, ctx->prop.multiProcessorCount, ctx->status_dev, xp, m, k, qp, sp, bp, n, yp);
            if (done) name = "gemv_q8_tc";
            if (!done && kernel == GQ_KERNEL_UMMA) fail("gq_int8_linear: the tcgen05 decode kernel takes one or two rows of x (m = %llu, k = %llu)", (unsigned long long)m, (unsigned long long)k);
        }
        if (!done && (kernel == GQ_KERNEL_AUTO || kernel == GQ_KERNEL_IMMA)) {
            done = launch_gemv_q8_imma(ctx->stream, ctx->prop.multiProcessorCount, ctx->status_dev, xp, m, k, qp, sp, bp, n, yp, weights_settled(ctx, {q, scale}));
            if (done) name = "gemv_q8_imma";
            if (!done && kernel == GQ_KERNEL_IMMA) fail("gq_int8_linear: the IMMA kernel takes one or two rows of x and rows that fit shared memory (m = %llu, k = %llu)", (unsigned long long)m, (unsigned long long)k);
        }
        if (!done && kernel != GQ_KERNEL_GEMV) {
            done = launch_gemv_q8_dp4a(ctx->stream, ctx->prop.multiProcessorCount, xp, m, k, qp, sp, bp, n, yp);
            if (!done && kernel == GQ_KERNEL_DP4A) fail("gq_int8_linear: in_features = %llu is too long for the dp4a kernel's shared-memory digit planes", (unsigned long long)k);
        }
        if (!done) launch_gemv_q8(ctx->stream, ctx->prop.multiProcessorCount, xp, m, k, qp, sp, bp, n, yp);
        after_launch(ctx, name, {x, q, scale, bias, y}, {y});
    });
}

int32_t gq_int4_quantize(gq_ctx* ctx, gq_buf w, uint64_t w_off, uint64_t rows, uint64_t k, uint64_t group, gq_buf q,
                         gq_buf scale, gq_buf zero) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_int4_quantize", rows, k);
        if (k == 0) fail("cannot quantize a weight with no input features");  // quant4.rs:93-97
        check_group(group);
        uint64_t groups = (k + group - 1) / group;
        auto wp = (const float*)view(ctx, w, w_off, rows * k, 4, "gq_int4_quantize weight");
        auto qp = (uint32_t*)view(ctx, q, 0, rows * words4(k), 4, "gq_int4_quantize q");
        auto sp = (float*)view(ctx, scale, 0, rows * groups, 4, "gq_int4_quantize scale");
        auto zp = (float*)view(ctx, zero, 0, rows * groups, 4, "gq_int4_quantize zero");
        if (rows == 0) return;
        launch_quantize_q4(ctx->stream, wp, rows, k, group, qp, sp, zp);
        after_launch(ctx, "quantize_q4", {w, q, scale, zero});
    });
}

int32_t gq_int4_dequantize(gq_ctx* ctx, gq_buf q, gq_buf scale, gq_buf zero, uint64_t rows, uint64_t k,
                           uint64_t group, gq_buf w) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_int4_dequantize", rows, k);
        check_group(group);
        uint64_t groups = (k + group - 1) / group;
        auto qp = (const uint32_t*)view(ctx, q, 0, rows * words4(k), 4, "gq_int4_dequantize q");
        auto sp = (const float*)view(ctx, scale, 0, rows * groups, 4, "gq_int4_dequantize scale");
        auto zp = (const float*)view(ctx, zero, 0, rows * groups, 4, "gq_int4_dequantize zero");
        auto wp = (float*)view(ctx, w, 0, rows * k, 4, "gq_int4_dequantize weight");
        if (rows == 0 || k == 0) return;
        launch_dequantize_q4(ctx->stream, qp, sp, zp, rows, k, group, wp);
        after_launch(ctx, "dequantize_q4", {q, scale, zero, w});
    });
}

// Which kernel GQ_KERNEL_AUTO gives an int4 group-128 linear of m rows: 0 = the single-launch kernels (ring passes, dp4a),
// 1 = the tcgen05 decode kernel with K cut in slices (gemv_q4_umma), 2 = the one with the features on the lanes
// (gemv_q4_lanes). Both tcgen05 kernels read the weight once whatever m is. The sliced one runs at about 2.2 bytes per ns
// after ~9 us of launches and start-up. The lanes one takes ~0.78 us per stage of two groups, whatever the stage's width,
// after ~4.5 us; a CTA owns tiles of up to 128 features over all of K (14336 x 4096: 16-18 us against 24-25; 28672 x 8192:
// 52-57 against 61-70) or, where the features alone do not fill the SMs, over a slice of K (+ ~3 us for the sum). The warp-level ring kernel (K = 4096 or 8192) takes a pass at ~4.5 bytes per ns
// (one row) per four rows of x, a pass with three or four rows running ~1.7 times as long as a one-row pass (its IMMA issue
// rate); the dp4a kernel elsewhere grows with every row. Measured on B200; weights under 4 MB stay with the single-launch
// kernels.
static int int4_tensor_route(uint64_t m, uint64_t n, uint64_t k, uint64_t group, int sm_count) {
    if (m < 3 || m > 16 || group != 128 || k % 128) return 0;
    const double mb = (double)n * (double)k / 2e6;
    if (mb < 4.0) return 0;
    const double umma_us = 9.0 + mb / 2.2;
    double lanes_us = 1e30;
    if (k / 128 <= 128) {
        uint32_t kslices, stages;
        gemv_q4_lanes_shape(n, k, sm_count, &kslices, &stages);
        lanes_us = 4.5 + 0.78 * (double)stages + (kslices > 1 ? 3.0 : 0.0);  // (the sum over its K slices, where it cuts K)
    }
    double other_us = mb * (0.26 * (double)m + 0.27);
    if (k == 4096 || k == 8192) {
        other_us = 0.0;
        for (uint64_t r = 0; r < m; r += 4) other_us += (2.5 + mb / 4.5) * (m - r >= 3 ? 1.7 : m - r == 2 ? 1.1 : 1.0);
    }
    if (lanes_us <= umma_us) return lanes_us < other_us ? 2 : 0;
    return umma_us < other_us ? 1 : 0;
}
int32_t gq_int4_linear(gq_ctx* ctx, gq_buf x, uint64_t x_off, uint64_t m, uint64_t k, gq_buf q, gq_buf scale,
                       gq_buf zero, gq_buf bias, uint64_t b_off, uint64_t n, uint64_t group, gq_buf y,
                       int32_t kernel) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_int4_linear", m, k, n);
        check_group(group);
        if (kernel < GQ_KERNEL_AUTO || (kernel > GQ_KERNEL_RING && kernel != GQ_KERNEL_UMMA_LANES)) fail("gq_int4_linear: unknown kernel selector %d", kernel);
        uint64_t groups = (k + group - 1) / group;
        auto xp = (const float*)view(ctx, x, x_off, m * k, 4, "gq_int4_linear input");
        auto qp = (const uint32_t*)view(ctx, q, 0, n * words4(k), 4, "gq_int4_linear q");
        auto sp = (const float*)view(ctx, scale, 0, n * groups, 4, "gq_int4_linear scale");
        auto zp = (const float*)view(ctx, zero, 0, n * groups, 4, "gq_int4_linear zero");
        auto bp = bias ? (const float*)view(ctx, bias, b_off, n, 4, "gq_int4_linear bias") : nullptr;
        auto yp = (float*)view(ctx, y, 0, m * n, 4, "gq_int4_linear output");
        if (ranges_overlap(yp, m * n * 4, xp, m * k * 4)) fail("gq_int4_linear: the output must not overlap the input (CTAs read x while others write y)");
        if (m == 0 || n == 0) return;
        const int route = kernel == GQ_KERNEL_AUTO ? int4_tensor_route(m, n, k, group, ctx->prop.multiProcessorCount) : 0;
        if (route == 2) {
            const uint64_t need = gemv_q4_umma_scratch_bytes(m, k, n, ctx->prop.multiProcessorCount);
            if (need && !(ctx->capturing && ctx->scratch_bytes < need) &&
                launch_gemv_q4_lanes(ctx->stream, ctx->prop.multiProcessorCount, ctx->status_dev, xp, m, k, qp, sp, zp, bp, n, group, yp, context_scratch(ctx, need))) {
                after_launch(ctx, "gemv_q4_lanes", {x, q, scale, zero, bias, y}, {y});
                ctx->stats.launches += 1;  // the digit conversion ahead of it
                return;
            }
        }
        if (route != 0) {
            const uint64_t need = gemv_q4_umma_scratch_bytes(m, k, n, ctx->prop.multiProcessorCount);
            // (a scratch that would have to grow inside a capture leaves the choice to the kernels that need none)
            if (need && !(ctx->capturing && ctx->scratch_bytes < need) &&
                launch_gemv_q4_umma(ctx->stream, ctx->prop.multiProcessorCount, ctx->status_dev, xp, m, k, qp, sp, zp, bp, n, group, yp, context_scratch(ctx, need))) {
                after_launch(ctx, "gemv_q4_umma", {x, q, scale, zero, bias, y}, {y});
                ctx->stats.launches += 2;  // the digit conversion ahead of it and the sum over the K slices behind it
                return;
            }
        }
        // More than sixteen rows (a prompt through an int4 layer): passes of sixteen through the same kernel, each reading the
        // weight once (the reference's tiled path does not exist for int4 either; dp4a would read it once per row).
        if (kernel == GQ_KERNEL_AUTO && m > 16 && group == 128 && k % 128 == 0 && n * k >= (8ull << 20)) {
            const uint64_t need = gemv_q4_umma_scratch_bytes(16, k, n, ctx->prop.multiProcessorCount);
            if (need && !(ctx->capturing && ctx->scratch_bytes < need)) {
                void* scratch = context_scratch(ctx, need);
                bool all = true;
                uint64_t passes = 0;
                for (uint64_t r = 0; r < m && all; r += 16, ++passes)
                    all = launch_gemv_q4_lanes(ctx->stream, ctx->prop.multiProcessorCount, ctx->status_dev, xp + r * k, m - r < 16 ? m - r : 16, k, qp, sp, zp, bp, n, group,
                                               yp + r * n, scratch);
                if (all) {
                    after_launch(ctx, "gemv_q4_lanes", {x, q, scale, zero, bias, y}, {y});
                    ctx->stats.launches += 2 * passes - 1;
                    return;
                }
                if (passes > 1) fail("gq_int4_linear: a pass of the tcgen05 kernel was refused after an earlier one had been launched");
            }
        }
        if (kernel == GQ_KERNEL_UMMA_LANES) {
            const uint64_t need = gemv_q4_umma_scratch_bytes(m, k, n, ctx->prop.multiProcessorCount);
            if (!need || !launch_gemv_q4_lanes(ctx->stream, ctx->prop.multiProcessorCount, ctx->status_dev, xp, m, k, qp, sp, zp, bp, n, group, yp,
                                               context_scratch(ctx, need)))
                fail("gq_int4_linear: the features-on-the-lanes tcgen05 kernel takes group_size 128, in_features a multiple of 128 up to 16384, 1 to 16 "
                     "rows of x and 16-byte aligned x (m = %llu, k = %llu, group_size = %llu, x_off = %llu)",
                     (unsigned long long)m, (unsigned long long)k, (unsigned long long)group, (unsigned long long)x_off);
            after_launch(ctx, "gemv_q4_lanes", {x, q, scale, zero, bias, y}, {y});
            ctx->stats.launches += 1;  // the digit conversion ahead of it
            return;
        }
        if (kernel == GQ_KERNEL_UMMA) {
            const uint64_t need = gemv_q4_umma_scratch_bytes(m, k, n, ctx->prop.multiProcessorCount);
            if (!need || !launch_gemv_q4_umma(ctx->stream, ctx->prop.multiProcessorCount, ctx->status_dev, xp, m, k, qp, sp, zp, bp, n, group, yp,
                                              context_scratch(ctx, need)))
                fail("gq_int4_linear: the tcgen05 decode kernel takes group_size 128, in_features a multiple of 128, 1 to 16 rows of x and "
                     "16-byte aligned x (m = %llu, k = %llu, group_size = %llu, x_off = %llu)",
                     (unsigned long long)m, (unsigned long long)k, (unsigned long long)group, (unsigned long long)x_off);
            after_launch(ctx, "gemv_q4_umma", {x, q, scale, zero, bias, y}, {y});
            return;
        }
        if (kernel == GQ_KERNEL_TENSOR) fail("gq_int4_linear: there is no tensor-core int4 kernel (the reference has none either, crates/grilly-infer/src/quant4.rs:412-413)");
        bool done = false;
        const char* name = "gemv_q4";
        if (kernel == GQ_KERNEL_AUTO || kernel == GQ_KERNEL_RING) {
            // Straight after another kernel of this library whose outputs are known, the launch may begin while that one
            // drains (its weight copies only; it waits for it to finish before it reads x or writes y), provided its
            // weights are not what that kernel wrote.
            // More rows of x than one launch takes (4) go in passes of that many, up to 16
            // rows: the packed weight (a few tens of MB) stays in L2 between the passes.
            const bool overlap = weights_settled(ctx, {q, scale, zero});
            const uint64_t per_pass = 4;
            if (m <= 16) {
                for (uint64_t r = 0; r < m; r += per_pass) {
                    const uint64_t rows = m - r < per_pass ? m - r : per_pass;
                    const bool first = r == 0;
                    done = launch_gemv_q4_ring(ctx->stream, ctx->prop.multiProcessorCount, ctx->status_dev, xp + r * k, rows, k, qp, sp, zp, bp, n, group,
                                               yp + r * n, first ? overlap : (y != q && y != scale && y != zero),
                                               first ? weights_settled(ctx, {x}) : x != y);
                    if (!done) break;  // refused on the first pass: nothing was launched
                    if (!first) ctx->stats.launches++;
                }
            }
            if (done) name = "gemv_q4_ring";
            if (!done && kernel == GQ_KERNEL_RING) fail("gq_int4_linear: the ring kernel takes up to 16 rows of x, group_size 128 and in_features 4096 or 8192 (m = %llu, k = %llu, group_size = %llu)", (unsigned long long)m, (unsigned long long)k, (unsigned long long)group);
        }
        if (!done && (kernel == GQ_KERNEL_AUTO || kernel == GQ_KERNEL_IMMA)) {
            done = launch_gemv_q4_imma(ctx->stream, ctx->prop.multiProcessorCount, ctx->status_dev, xp, m, k, qp, sp, zp, bp, n, group, yp, weights_settled(ctx, {q, scale, zero}));
            if (done) name = "gemv_q4_imma";
            if (!done && kernel == GQ_KERNEL_IMMA) fail("gq_int4_linear: the IMMA kernel takes one or two rows of x, a group_size that is a multiple of 128 and rows that fit shared memory (m = %llu, k = %llu, group_size = %llu)", (unsigned long long)m, (unsigned long long)k, (unsigned long long)group);
        }
        if (!done && kernel != GQ_KERNEL_GEMV) {
            done = launch_gemv_q4_dp4a(ctx->stream, ctx->prop.multiProcessorCount, xp, m, k, qp, sp, zp, bp, n, group, yp);
            if (!done && kernel == GQ_KERNEL_DP4A) fail("gq_int4_linear: in_features = %llu is too long for the dp4a kernel's shared-memory digit planes", (unsigned long long)k);
        }
        if (!done) launch_gemv_q4(ctx->stream, ctx->prop.multiProcessorCount, xp, m, k, qp, sp, zp, bp, n, group, yp);
        after_launch(ctx, name, {x, q, scale, zero, bias, y}, {y});
    });
}

// ── GPTQ ─────────────────────────────────────────────────────────────────

int32_t gq_gptq_hessian_add(gq_ctx* ctx, gq_buf x, uint64_t x_off, uint64_t rows, uint64_t k, gq_buf hessian) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_gptq_hessian_add", rows, k);
        if (k == 0) fail("gq_gptq_hessian_add: no input features");
        auto xp = (const float*)view(ctx, x, x_off, rows * k, 4, "gq_gptq_hessian_add inputs");
        auto hp = (float*)view(ctx, hessian, 0, k * k, 4, "gq_gptq_hessian_add hessian");
        if (rows == 0) return;
        launch_hessian_add(ctx->stream, xp, rows, k, hp);
        after_launch(ctx, "gptq_hessian_add", {x, hessian});
    });
}

int32_t gq_gptq_quantize(gq_ctx* ctx, gq_buf work, uint64_t rows, uint64_t k, uint64_t group, gq_buf upper, gq_buf errors, gq_buf q, gq_buf scale,
                         gq_buf zero) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_gptq_quantize", rows, k);
        check_group(group);
        // python/grilly/infer/gptq.py:128-129
        if (k == 0 || k % group) fail("in_features %llu must be a whole number of groups of %llu", (unsigned long long)k, (unsigned long long)group);
        if (128 % group) fail("gq_gptq_quantize: group_size %llu is not implemented yet (32, 64 or 128: a group must lie inside a block of 128 columns)", (unsigned long long)group);
        const uint64_t groups = k / group;
        auto wp = (float*)view(ctx, work, 0, rows * k, 4, "gq_gptq_quantize working weight");
        auto up = (const float*)view(ctx, upper, 0, k * k, 4, "gq_gptq_quantize inverse Cholesky factor");
        auto ep = (float*)view(ctx, errors, 0, gptq_error_floats(rows), 4, "gq_gptq_quantize errors");
        auto qp = (uint32_t*)view(ctx, q, 0, rows * words4(k), 4, "gq_gptq_quantize q");
        auto sp = (float*)view(ctx, scale, 0, rows * groups, 4, "gq_gptq_quantize scale");
        auto zp = (float*)view(ctx, zero, 0, rows * groups, 4, "gq_gptq_quantize zero");
        if (rows == 0) return;
        GQ_CUDA(cudaMemsetAsync(qp, 0, rows * words4(k) * 4, ctx->stream));  // padding words stay zero
        launch_gptq(ctx->stream, wp, up, rows, k, group, ep, qp, sp, zp);
        ctx->stats.launches += 2 * ((k + 127) / 128) - 1;
        after_launch(ctx, "gptq", {work, upper, errors, q, scale, zero});
    });
}

// ── capture / replay ─────────────────────────────────────────────────────

int32_t gq_begin_capture(gq_ctx* ctx) {
    return guarded([&] {
        Locked l(ctx);
        if (ctx->capturing) fail("a capture is already running on this context");
        // Relaxed: buffer allocation (cudaMalloc on a pool miss) stays legal while recording.
        ctx->prev_known = false;
        GQ_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
        ctx->capturing = true;
        ctx->capture_nodes = 0;
        ctx->capture_retained.clear();
    });
}

int32_t gq_end_capture(gq_ctx* ctx, gq_graph** out) {
    return guarded([&] {
        Locked l(ctx);
        if (out) *out = nullptr;
        if (!ctx->capturing) fail("no capture is running on this context");
        ctx->capturing = false;
        cudaGraph_t graph = nullptr;
        ctx->prev_known = false;
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
        auto retained = std::move(ctx->capture_retained);
        ctx->capture_retained.clear();
        auto release_all = [&] {
            for (gq_buf h : retained) drop_ref(ctx, h);
        };
        if (e != cudaSuccess) {
            release_all();
            cudaGetLastError();
            fail("ending the capture: %s", cudaGetErrorString(e));
        }
        if (!out) {  // the caller only wanted the capture closed (an exception path)
            if (graph) cudaGraphDestroy(graph);
            release_all();
            return;
        }
        if (ctx->capture_nodes == 0) {
            if (graph) cudaGraphDestroy(graph);
            release_all();
            // crates/grilly-core/src/graph.rs:157-161
            fail("nothing was captured: the callable recorded no GPU work, so there is nothing to replay");
        }
        auto g = new gq_graph();
        g->graph = graph;
        g->nodes = ctx->capture_nodes;
        g->retained = std::move(retained);
        e = cudaGraphInstantiate(&g->exec, graph, 0);
        if (e != cudaSuccess) {
            cudaGraphDestroy(graph);
            for (gq_buf h : g->retained) drop_ref(ctx, h);
            delete g;
            fail("instantiating the captured graph: %s", cudaGetErrorString(e));
        }
        ctx->stats.captures++;
        // The reference records while it runs, so the step has happened by the
        // time its capture ends. A CUDA stream capture only records: run it once.
        ctx->prev_known = false;
        e = cudaGraphLaunch(g->exec, ctx->stream);
        if (e != cudaSuccess) {
            cudaGraphExecDestroy(g->exec);
            cudaGraphDestroy(graph);
            for (gq_buf h : g->retained) drop_ref(ctx, h);
            delete g;
            fail("running the captured graph: %s", cudaGetErrorString(e));
        }
        *out = g;
    });
}

int32_t gq_capturing(gq_ctx* ctx, uint32_t* out) {
    return guarded([&] {
        Locked l(ctx);
        if (!out) fail("gq_capturing: null out pointer");
        *out = ctx->capturing ? 1u : 0u;
    });
}

int32_t gq_graph_replay(gq_ctx* ctx, gq_graph* graph) {
    return guarded([&] {
        Locked l(ctx);
        if (!graph || !graph->exec) fail("gq_graph_replay: null graph");
        if (ctx->capturing) fail("gq_graph_replay: a capture is running on this context");
        ctx->prev_known = false;
        GQ_CUDA(cudaGraphLaunch(graph->exec, ctx->stream));
        ctx->stats.graph_launches++;
        ctx->stats.graph_nodes_replayed += graph->nodes;
        if (ctx->launch_blocking) GQ_CUDA(cudaStreamSynchronize(ctx->stream));
    });
}

int32_t gq_graph_nodes(gq_graph* graph, uint64_t* out) {
    return guarded([&] {
        if (!graph || !out) fail("gq_graph_nodes: null argument");
        *out = graph->nodes;
    });
}

void gq_graph_destroy(gq_ctx* ctx, gq_graph* graph) {
    if (!ctx || !graph) return;
    guarded([&] {
        Locked l(ctx);
        cudaStreamSynchronize(ctx->stream);  // a replay may still be running
        if (graph->exec) cudaGraphExecDestroy(graph->exec);
        if (graph->graph) cudaGraphDestroy(graph->graph);
        for (gq_buf h : graph->retained) drop_ref(ctx, h);
        delete graph;
    });
}

// ── multi-GPU ────────────────────────────────────────────────────────────

int32_t gq_comm_unique_id(void* out, uint64_t bytes) {
    return guarded([&] {
        if (!out || bytes < GQ_COMM_ID_BYTES) fail("gq_comm_unique_id: the id needs %d bytes", GQ_COMM_ID_BYTES);
        comm_unique_id(out);
    });
}

int32_t gq_comm_create(gq_ctx* ctx, int32_t nranks, int32_t rank, const void* unique_id, gq_comm** out) {
    return guarded([&] {
        Locked l(ctx);
        if (!out || !unique_id) fail("gq_comm_create: null argument");
        *out = nullptr;
        *out = comm_create(nranks, rank, unique_id);
    });
}

void gq_comm_destroy(gq_ctx* ctx, gq_comm* comm) {
    if (!ctx || !comm) return;
    guarded([&] {
        Locked l(ctx);
        cudaStreamSynchronize(ctx->stream);
        comm_destroy(comm);
    });
}

int32_t gq_all_gather_columns(gq_ctx* ctx, gq_comm* comm, gq_buf src, gq_buf dst, uint64_t m, uint64_t n_shard) {
    return guarded([&] {
        Locked l(ctx);
        if (!comm) fail("gq_all_gather_columns: null communicator");
        int nranks, rank;
        comm_info(comm, &nranks, &rank);
        check_dims("gq_all_gather_columns", m, n_shard * nranks);
        auto sp = (const float*)view(ctx, src, 0, m * n_shard, 4, "gq_all_gather_columns source");
        auto dp = (float*)view(ctx, dst, 0, m * n_shard * nranks, 4, "gq_all_gather_columns destination");
        if (m == 0 || n_shard == 0) return;
        all_gather_columns(ctx->stream, comm, sp, dp, m, n_shard);
        after_launch(ctx, "nccl_all_gather", {src, dst});
    });
}

int32_t gq_buffer_ipc_export(gq_ctx* ctx, gq_buf buf, void* out, uint64_t bytes) {
    return guarded([&] {
        Locked l(ctx);
        static_assert(sizeof(cudaIpcMemHandle_t) <= GQ_IPC_HANDLE_BYTES, "ipc handle size");
        if (!out || bytes < GQ_IPC_HANDLE_BYTES) fail("gq_buffer_ipc_export: the handle needs %d bytes", GQ_IPC_HANDLE_BYTES);
        Buffer& b = lookup(ctx, buf, "gq_buffer_ipc_export");
        if (!b.owned || b.ipc || !b.ptr) fail("gq_buffer_ipc_export: only non-empty buffers made by gq_buffer_create can be exported");
        cudaIpcMemHandle_t h;
        GQ_CUDA(cudaIpcGetMemHandle(&h, b.ptr));
        memset(out, 0, GQ_IPC_HANDLE_BYTES);
        memcpy(out, &h, sizeof h);
    });
}

int32_t gq_buffer_ipc_open(gq_ctx* ctx, const void* handle, uint64_t buffer_bytes, gq_buf* out) {
    return guarded([&] {
        Locked l(ctx);
        if (!out || !handle) fail("gq_buffer_ipc_open: null argument");
        *out = 0;
        cudaIpcMemHandle_t h;
        memcpy(&h, handle, sizeof h);
        void* p = nullptr;
        GQ_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        Buffer b;
        b.ptr = p;
        b.bytes = buffer_bytes;
        b.owned = false;
        b.ipc = true;
        gq_buf hnd = ctx->next_handle++;
        ctx->buffers.emplace(hnd, b);
        ctx->stats.buffers_outstanding++;
        *out = hnd;
    });
}

static PeerOut peer_views(gq_ctx* ctx, const char* op, uint64_t m, uint64_t n_shard, int32_t rank, int32_t nranks, const gq_buf* peer_recv,
                           gq_buf state, gq_buf y_full) {
    if (nranks < 1 || nranks > 8 || rank < 0 || rank >= nranks) fail("%s: rank %d of %d is out of range (at most 8 ranks)", op, rank, nranks);
    if (!peer_recv) fail("%s: null handle array", op);
    PeerOut peer;
    peer.nranks = (uint32_t)nranks, peer.rank = (uint32_t)rank, peer.n_full = (uint32_t)(n_shard * nranks), peer.m_total = (uint32_t)m;
    peer.wait_cycles = ctx->peer_wait_cycles;
    for (int i = 0; i < nranks; ++i) peer.ll[i] = (unsigned long long*)view(ctx, peer_recv[i], 0, 2 * m * n_shard * nranks, 8, "gather receive buffer");
    peer.state = (uint32_t*)view(ctx, state, 0, 2, 4, "gather state words");
    peer.y_full = (float*)view(ctx, y_full, 0, m * n_shard * nranks, 4, "gather y_full");
    return peer;
}

int32_t gq_peer_gather(gq_ctx* ctx, gq_buf src, uint64_t m, uint64_t n_shard, int32_t rank, int32_t nranks, const gq_buf* peer_recv,
                       gq_buf state, gq_buf y_full) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_peer_gather", m, n_shard * (nranks > 0 ? nranks : 1));
        if (m * n_shard * (uint64_t)(nranks > 0 ? nranks : 1) > 0x7fffffffull) fail("gq_peer_gather: more than 2^31 - 1 values");
        auto sp = (const float*)view(ctx, src, 0, m * n_shard, 4, "gq_peer_gather source");
        PeerOut peer = peer_views(ctx, "gq_peer_gather", m, n_shard, rank, nranks, peer_recv, state, y_full);
        if (src == y_full) fail("gq_peer_gather: the source block and y_full must be different buffers");
        if (m == 0 || n_shard == 0) return;
        launch_peer_gather(ctx->stream, ctx->prop.multiProcessorCount, peer, sp, m, n_shard, ctx->status_dev);
        after_launch(ctx, "peer_gather", {src, peer_recv[rank], state, y_full}, {peer_recv[rank], state, y_full});
    });
}

int32_t gq_int4_linear_gather(gq_ctx* ctx, gq_buf x, uint64_t x_off, uint64_t m, uint64_t k, gq_buf q, gq_buf scale, gq_buf zero, gq_buf bias,
                              uint64_t b_off, uint64_t n_shard, uint64_t group, int32_t rank, int32_t nranks, const gq_buf* peer_recv,
                              gq_buf state, gq_buf y_full) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_int4_linear_gather", m, k, n_shard * (nranks > 0 ? nranks : 1));
        check_group(group);
        if (m == 0 || n_shard == 0) fail("gq_int4_linear_gather: an empty layer");
        if (m > 16) fail("gq_int4_linear_gather: at most 16 rows of x (m = %llu)", (unsigned long long)m);
        const uint64_t groups = (k + group - 1) / group;
        auto xp = (const float*)view(ctx, x, x_off, m * k, 4, "gq_int4_linear_gather input");
        auto qp = (const uint32_t*)view(ctx, q, 0, n_shard * words4(k), 4, "gq_int4_linear_gather q");
        auto sp = (const float*)view(ctx, scale, 0, n_shard * groups, 4, "gq_int4_linear_gather scale");
        auto zp = (const float*)view(ctx, zero, 0, n_shard * groups, 4, "gq_int4_linear_gather zero");
        auto bp = bias ? (const float*)view(ctx, bias, b_off, n_shard, 4, "gq_int4_linear_gather bias") : nullptr;
        PeerOut peer = peer_views(ctx, "gq_int4_linear_gather", m, n_shard, rank, nranks, peer_recv, state, y_full);
        if (y_full == x) fail("gq_int4_linear_gather: y_full must not be the input buffer");
        // Many rows on a large shard: the tcgen05 decode kernel (one pass over the weight), and the gather adds up its K
        // slices' partial sums as it sends them.
        const int route = int4_tensor_route(m, n_shard, k, group, ctx->prop.multiProcessorCount);
        if (route != 0) {
            const int sms = ctx->prop.multiProcessorCount;
            const uint64_t need = gemv_q4_umma_scratch_bytes(m, k, n_shard, sms);
            if (need && !(ctx->capturing && ctx->scratch_bytes < need)) {
                void* scratch = context_scratch(ctx, need);
                const float* part = gemv_q4_umma_partials(scratch, m, k, n_shard, sms);  // the slices' sums, or (K not split) the shard's y
                uint32_t slices = 0;
                // (the kernel with the features on the lanes writes the shard's y, bias included, where the other leaves its sums)
                if ((route == 2 && launch_gemv_q4_lanes(ctx->stream, sms, ctx->status_dev, xp, m, k, qp, sp, zp, bp, n_shard, group, const_cast<float*>(part), scratch, &slices)) ||
                    launch_gemv_q4_umma(ctx->stream, sms, ctx->status_dev, xp, m, k, qp, sp, zp, bp, n_shard, group, const_cast<float*>(part), scratch, &slices)) {
                    peer.row0 = 0;
                    launch_peer_gather(ctx->stream, sms, peer, part, m, n_shard, ctx->status_dev, slices, slices ? bp : nullptr);
                    after_launch(ctx, "gemv_q4_umma_gather", {x, q, scale, zero, bias, peer_recv[rank], state, y_full}, {peer_recv[rank], state, y_full});
                    ctx->stats.launches += 2;
                    return;
                }
            }
        }
        // more rows of x than one launch takes go in passes, each a gather of its own rows (and a step of its own)
        const uint64_t per_pass = 4;
        for (uint64_t r = 0; r < m; r += per_pass) {
            const uint64_t rows = m - r < per_pass ? m - r : per_pass;
            peer.row0 = (uint32_t)r;
            if (!launch_gemv_q4_ring(ctx->stream, ctx->prop.multiProcessorCount, ctx->status_dev, xp + r * k, rows, k, qp, sp, zp, bp, n_shard, group, nullptr,
                                     r == 0 ? weights_settled(ctx, {q, scale, zero}) : true, r == 0 ? weights_settled(ctx, {x}) : x != y_full, &peer))
                fail("gq_int4_linear_gather: the fused kernel takes group_size 128 and in_features 4096 or 8192 (m = %llu, k = %llu, group_size = %llu)",
                     (unsigned long long)m, (unsigned long long)k, (unsigned long long)group);
            if (r) ctx->stats.launches++;
        }
        after_launch(ctx, "gemv_q4_ring_gather", {x, q, scale, zero, bias, peer_recv[rank], state, y_full}, {peer_recv[rank], state, y_full});
    });
}

}  // extern "C"
