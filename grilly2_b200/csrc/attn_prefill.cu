// Prompt processing: rotary + cache append for T new tokens at once, and causal
// grouped-query attention of those tokens over the cache — what the
// reference's prefill branch does with rope, scaled_dot_product_attention
// (is_causal, enable_gqa) and cache.append
// (python/grilly/infer/models/llama.py:168-179; crates/grilly-torch/src/attention.rs
// for the tiled kernel behind it). Here the T tokens continue from the DEVICE
// cursor (positions lens[layer] + t), so chunked prefill over a non-empty cache
// is the same call, and the whole prompt step can be captured.
//
// rope_append_rows: one thread per element of the T x (q | k | v) rows; q goes
// out rotated, k (rotated) and v go into the cache at their positions.
//
// attn_prefill: one warp per (query, head). A lane owns dim / 32 components of
// the output; keys are taken 32 at a time, lane j computing key j's whole dot
// product (q is broadcast from shared memory), then one warp-wide max / sum for
// the online softmax and 32 broadcasts of p_j against V's rows. fp32
// throughout; the exp is the accurate expf. The cache (1 MB per layer at 1024
// positions) stays in L2 across the queries that share it.
// Bound: L2 bandwidth and the FP32 pipes; it is the O(T^2) term of a prompt.
//
// The int8 KV cache (no counterpart in the reference, whose cache is exact
// float32, kv_cache.rs:1-19): each cached key / value row of one head is
// stored as dim int8 codes and one float32 scale, scale = max|v| / 127,
// code = rint(v / scale) — 4 x fewer bytes to read per decoded token. The
// same kernels take it (template parameter): rows are dequantized as they are
// read.
#include "gq_internal.h"

namespace gq {

namespace {

template <bool Q8>
__global__ void __launch_bounds__(256) rope_append_rows_kernel(const float* __restrict__ qkv, const float* __restrict__ cosv,
                                                              const float* __restrict__ sinv, const uint32_t* __restrict__ lens,
                                                              uint32_t layer, uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t dim,
                                                              uint32_t max_len, float* __restrict__ q_out, void* kc, void* vc,
                                                              float* __restrict__ kscale, float* __restrict__ vscale) {
    GQ_GRID_DEP_SYNC();
    // one warp per (row, head-slot): dim <= 128 values, dim / 32 per lane (dim is 32, 64 or 128)
    const uint32_t per = dim / 32, slots = heads + 2 * kv_heads, half = dim / 2;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows * slots) return;
    const uint32_t t = warp / slots, hd = warp - t * slots;
    const uint32_t pos = lens[layer] + t;
    const float* src = qkv + (size_t)t * slots * dim + (size_t)hd * dim;
    float v[4];
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
        if (i < per) {
            const uint32_t d = lane * per + i;
            const float xv = src[d];
            if (hd < heads + kv_heads) {
                const uint32_t p = min(pos, max_len - 1);
                const float rv = d < half ? -src[d + half] : src[d - half];
                v[i] = __fadd_rn(__fmul_rn(xv, cosv[(size_t)p * dim + d]), __fmul_rn(rv, sinv[(size_t)p * dim + d]));
            } else {
                v[i] = xv;
            }
        } else {
            v[i] = 0.0f;
        }
    }
    if (hd < heads) {
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i)
            if (i < per) q_out[(size_t)t * heads * dim + (size_t)hd * dim + lane * per + i] = v[i];
        return;
    }
    if (pos >= max_len) return;  // a full cache takes nothing more
    const bool is_k = hd < heads + kv_heads;
    const uint32_t g = is_k ? hd - heads : hd - heads - kv_heads;
    const size_t row = (size_t)g * max_len + pos;
    if (!Q8) {
        float* dst = reinterpret_cast<float*>(is_k ? kc : vc) + row * dim;
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i)
            if (i < per) dst[lane * per + i] = v[i];
    } else {
        float amax = 0.0f;
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float sc = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
        int8_t* dst = reinterpret_cast<int8_t*>(is_k ? kc : vc) + row * dim;
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i)
            if (i < per) dst[lane * per + i] = (int8_t)max(-127, min(127, __float2int_rn(__fdiv_rn(v[i], sc))));
        if (lane == 0) (is_k ? kscale : vscale)[row] = sc;
    }
}

// A cached row's component d, dequantized when the cache is int8.
template <bool Q8>
__device__ __forceinline__ float cache_at(const void* base, const float* scales, size_t row, uint32_t dim, uint32_t d) {
    if (!Q8) return reinterpret_cast<const float*>(base)[row * dim + d];
    return (float)reinterpret_cast<const int8_t*>(base)[row * dim + d] * scales[row];
}

constexpr int kPrefillWarps = 8;

template <bool Q8>
__global__ void __launch_bounds__(kPrefillWarps * 32) attn_prefill_kernel(const float* __restrict__ q, const void* __restrict__ kc,
                                                                         const void* __restrict__ vc, const float* __restrict__ kscale,
                                                                         const float* __restrict__ vscale, const uint32_t* __restrict__ lens,
                                                                         uint32_t layer, uint32_t rows, uint32_t heads, uint32_t kv_heads,
                                                                         uint32_t dim, uint32_t max_len, float scale, float* __restrict__ out) {
    GQ_GRID_DEP_SYNC();
    __shared__ float s_q[kPrefillWarps][128];
    const uint32_t w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t item = blockIdx.x * kPrefillWarps + w;  // (query row, head)
    if (item >= rows * heads) return;
    const uint32_t t = item / heads, h = item - t * heads, g = h / (heads / kv_heads), per = dim / 32;
    const uint32_t pos0 = lens[layer];
    const uint32_t qpos = min(pos0 + t, max_len - 1);  // the query attends to cache positions 0 .. qpos
    for (uint32_t d = lane; d < dim; d += 32) s_q[w][d] = q[(size_t)t * heads * dim + (size_t)h * dim + d] * scale;
    __syncwarp();
    float m = __uint_as_float(0xff800000u), l = 0.0f, acc[4] = {0.f, 0.f, 0.f, 0.f};
    const size_t base = (size_t)g * max_len;
    for (uint32_t j0 = 0; j0 <= qpos; j0 += 32) {
        const uint32_t j = j0 + lane;
        float s = __uint_as_float(0xff800000u);
        if (j <= qpos) {
            s = 0.0f;
            if (!Q8) {
                const float4* kr = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(kc) + (base + j) * dim);
                for (uint32_t d4 = 0; d4 < dim / 4; ++d4) {
                    const float4 kv = kr[d4];
                    s = __fmaf_rn(s_q[w][4 * d4], kv.x, s), s = __fmaf_rn(s_q[w][4 * d4 + 1], kv.y, s);
                    s = __fmaf_rn(s_q[w][4 * d4 + 2], kv.z, s), s = __fmaf_rn(s_q[w][4 * d4 + 3], kv.w, s);
                }
            } else {
                const char4* kr = reinterpret_cast<const char4*>(reinterpret_cast<const int8_t*>(kc) + (base + j) * dim);
                for (uint32_t d4 = 0; d4 < dim / 4; ++d4) {
                    const char4 kv = kr[d4];
                    s = __fmaf_rn(s_q[w][4 * d4], (float)kv.x, s), s = __fmaf_rn(s_q[w][4 * d4 + 1], (float)kv.y, s);
                    s = __fmaf_rn(s_q[w][4 * d4 + 2], (float)kv.z, s), s = __fmaf_rn(s_q[w][4 * d4 + 3], (float)kv.w, s);
                }
                s *= kscale[base + j];
            }
        }
        float cm = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
        const float mn = fmaxf(m, cm);
        const float corr = m == mn ? 1.0f : expf(m - mn);  // m = -inf only before the first chunk, where l and acc are zero
        const float p = j <= qpos ? expf(s - mn) : 0.0f;
        float ps = p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l = __fmaf_rn(l, corr, ps);
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) acc[i] *= corr;
        const uint32_t cnt = min(32u, qpos + 1 - j0);
        for (uint32_t jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i)
                if (i < per) acc[i] = __fmaf_rn(pj, cache_at<Q8>(vc, vscale, base + j0 + jj, dim, lane * per + i), acc[i]);
        }
        m = mn;
    }
    const float inv = l > 0.0f ? __fdiv_rn(1.0f, l) : 0.0f;
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i)
        if (i < per) out[(size_t)t * heads * dim + (size_t)h * dim + lane * per + i] = acc[i] * inv;
}

__global__ void kv_advance_by_kernel(uint32_t* lens, uint32_t layers, uint32_t max_len, uint32_t count) {
    GQ_GRID_DEP_SYNC();
    const uint32_t l = blockIdx.x * blockDim.x + threadIdx.x;
    if (l < layers) lens[l] = min(lens[l] + count, max_len);
}

}  // namespace

void launch_rope_append_rows(cudaStream_t s, const float* qkv, const float* cosv, const float* sinv, const uint32_t* lens, uint32_t layer,
                             uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t dim, uint32_t max_len, float* q_out, void* kc, void* vc,
                             float* kscale, float* vscale, bool int8_cache) {
    const uint64_t warps = (uint64_t)rows * (heads + 2 * kv_heads);
    const dim3 grid((uint32_t)((warps * 32 + 255) / 256)), block(256);
    if (int8_cache)
        launch_after(rope_append_rows_kernel<true>, grid, block, 0, s, qkv, cosv, sinv, lens, layer, rows, heads, kv_heads, dim, max_len, q_out, kc, vc,
                     kscale, vscale);
    else
        launch_after(rope_append_rows_kernel<false>, grid, block, 0, s, qkv, cosv, sinv, lens, layer, rows, heads, kv_heads, dim, max_len, q_out, kc, vc,
                     kscale, vscale);
}

void launch_attn_prefill(cudaStream_t s, const float* q, const void* kc, const void* vc, const float* kscale, const float* vscale,
                         const uint32_t* lens, uint32_t layer, uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t dim, uint32_t max_len,
                         float scale, float* out, bool int8_cache) {
    const uint64_t items = (uint64_t)rows * heads;
    const dim3 grid((uint32_t)((items + kPrefillWarps - 1) / kPrefillWarps)), block(kPrefillWarps * 32);
    if (int8_cache)
        launch_after(attn_prefill_kernel<true>, grid, block, 0, s, q, kc, vc, kscale, vscale, lens, layer, rows, heads, kv_heads, dim, max_len, scale, out);
    else
        launch_after(attn_prefill_kernel<false>, grid, block, 0, s, q, kc, vc, kscale, vscale, lens, layer, rows, heads, kv_heads, dim, max_len, scale, out);
}

void launch_kv_advance_by(cudaStream_t s, uint32_t* lens, uint32_t layers, uint32_t max_len, uint32_t count) {
    launch_after(kv_advance_by_kernel, dim3((layers + 127) / 128), dim3(128), 0, s, lens, layers, max_len, count);
}

}  // namespace gq
