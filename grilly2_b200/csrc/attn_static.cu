// gq_attn_decode_static: the split-and-merge decode attention of decode_ops.cu
// with its scratch (the splits' partial results and the per-head arrival
// counters) in a fixed array of this module's device memory instead of a
// caller's buffer, so that the call needs no scratch buffer and allocates
// nothing: no device, host or pool allocation happens on this path, on the
// first call or any later one.
//
// The first call on a device looks the array's address up (set-up: one
// cudaGetSymbolAddress, remembered per device); make that call before any
// stream capture begins. The array is zero when the module loads and every
// launch leaves the counters at zero again, which is all the kernel needs; the
// counters lie at the start of the array whatever the shape, so calls of
// different shapes may follow one another.
// Every call on a device shares the one array: calls that overlap on the GPU
// (two contexts, hence two streams, on one device) race on it; calls on one
// context are ordered by its stream and do not.
#include <mutex>

#include "gq_internal.h"

namespace {

// 2 MiB: room for 1024 counters + heads * splits * (head_dim + 2) floats, e.g. 32 heads x 64 splits x head_dim 128.
constexpr uint64_t kStaticScratchFloats = 512ull * 1024ull;
static __device__ __align__(256) float g_attn_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
float* g_scratch_ptr[kMaxDevices] = {};

float* static_scratch(int device) {
    if (device < 0 || device >= kMaxDevices) gq::fail("gq_attn_decode_static: device ordinal %d is out of range", device);
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ptr[device]) {
        float* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_attn_scratch);
        if (e != cudaSuccess || !ptr) gq::fail("gq_attn_decode_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_scratch_ptr[device] = ptr;
    }
    return g_scratch_ptr[device];
}

}  // namespace

using namespace gq;

extern "C" int32_t gq_attn_decode_static(gq_ctx* ctx, gq_buf q, gq_buf kcache, uint64_t k_off, gq_buf vcache, uint64_t v_off, gq_buf lens,
                                         uint64_t layer, uint64_t layers, uint64_t heads, uint64_t kv_heads, uint64_t dim,
                                         uint64_t max_len, float scale, gq_buf out) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_attn_decode_static", heads, kv_heads, dim);
        check_dims("gq_attn_decode_static", max_len, layers);
        if (heads == 0 || kv_heads == 0 || heads % kv_heads)
            fail("gq_attn_decode_static: %llu heads do not group over %llu kv heads", (unsigned long long)heads, (unsigned long long)kv_heads);
        if (dim != 32 && dim != 64 && dim != 128) fail("gq_attn_decode_static: head_dim must be 32, 64 or 128, got %llu", (unsigned long long)dim);
        if (max_len == 0) fail("gq_attn_decode_static: a cache of no positions");
        if (layer >= layers) fail("gq_attn_decode_static: layer %llu of %llu", (unsigned long long)layer, (unsigned long long)layers);
        const uint32_t splits = attn_splits((uint32_t)heads, (uint32_t)max_len, ctx->prop.multiProcessorCount);
        const uint64_t need = attn_scratch_floats((uint32_t)heads, (uint32_t)dim, splits);
        if (need > kStaticScratchFloats)
            fail("gq_attn_decode_static: %llu heads x %u splits x head_dim %llu needs %llu bytes of scratch, beyond the fixed %llu "
                 "bytes of this entry point: use gq_attn_decode with a scratch buffer",
                 (unsigned long long)heads, splits, (unsigned long long)dim, (unsigned long long)(need * 4),
                 (unsigned long long)(kStaticScratchFloats * 4));
        auto qp = (const float*)view(ctx, q, 0, heads * dim, 4, "gq_attn_decode_static q");
        auto kp = (float*)view(ctx, kcache, k_off, kv_heads * max_len * dim, 4, "gq_attn_decode_static key cache");
        auto vp = (float*)view(ctx, vcache, v_off, kv_heads * max_len * dim, 4, "gq_attn_decode_static value cache");
        auto lp = (const uint32_t*)view(ctx, lens, 0, layers, 4, "gq_attn_decode_static cursor");
        auto op = (float*)view(ctx, out, 0, heads * dim, 4, "gq_attn_decode_static output");
        float* sp = static_scratch(ctx->device);
        launch_attn_decode(ctx->stream, qp, kp, vp, lp, (uint32_t)layer, (uint32_t)heads, (uint32_t)kv_heads, (uint32_t)dim,
                           (uint32_t)max_len, scale, splits, sp, op);
        after_launch(ctx, "attn_decode_static", {q, kcache, vcache, lens, out}, {out});
    });
}
