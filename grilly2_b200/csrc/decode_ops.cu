// The non-linear tenth of a decode step of a Llama/Qwen2-shaped model, for
// the int8 weight-only full-step configuration: embedding lookup, add +
// RMSNorm, rotary embedding into the KV cache, grouped-query decode attention
// (split over the cache length), SwiGLU, greedy argmax. They replace the
// reference's shaders
//   g2-index.glsl:22-38, g2-rms-norm.glsl:54-74, g2-rope.glsl:24-40,
//   g2-kv-write.glsl:43-72, g2-kv-advance.glsl:18-21,
//   g2-attn-decode{,-split,-merge}.glsl, g2-swiglu.glsl:21-29,
//   g2-argreduce-rows.glsl:42-77   (all under crates/grilly-core/shaders/).
//
// Everything a step needs to know about *where it is* comes from device
// memory — the token id, the cache cursor (which is also the rotary position
// of q AND k) — never from a kernel argument, so a captured step replays
// correctly: the reference pushes q's position from the host
// (python/grilly/infer/models/llama.py:168-173), which a replay would bake in.
//
// All kernels here are small and latency-bound; the step's time is the
// quantized linears' (97 of them, ~494 of ~522 MB per token).
#include "gq_internal.h"
#include "math_common.cuh"

namespace gq {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// out[r][:] = table[ids[r]][:]; an id outside the table yields a row of NaN
// (the reference raises a deferred IndexError from a fault buffer).
__global__ void __launch_bounds__(256) embedding_kernel(const float* __restrict__ table, const int32_t* __restrict__ ids,
                                                       uint32_t rows, uint32_t width, uint32_t vocab, float* __restrict__ out) {
    GQ_GRID_DEP_SYNC();
    for (uint32_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const int32_t id = ids[r];
        const bool ok = id >= 0 && (uint32_t)id < vocab;
        for (uint32_t c = threadIdx.x; c < width; c += blockDim.x)
            out[(size_t)r * width + c] = ok ? table[(size_t)id * width + c] : __uint_as_float(0x7fc00000u);
    }
}

// h = x (+ residual); y = h * (1 / sqrt(mean(h^2) + eps)) * w, torch's order
// of operations (g2-rms-norm.glsl:54-74). The sum of squares is taken in
// float64, which rounds to float32 where the shader's compensated sum does.
__global__ void __launch_bounds__(256) add_rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ res,
                                                          const float* __restrict__ w, uint32_t rows, uint32_t n, float eps,
                                                          float* __restrict__ y, float* __restrict__ h) {
    GQ_GRID_DEP_SYNC();
    __shared__ double s_part[8];
    __shared__ float s_r;
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* xr = x + (size_t)row * n;
        const float* rr = res ? res + (size_t)row * n : nullptr;
        double ss = 0.0;
        for (uint32_t k = threadIdx.x; k < n; k += 256) {
            const float v = rr ? __fadd_rn(xr[k], rr[k]) : xr[k];
            ss += (double)__fmul_rn(v, v);
        }
        ss = warp_sum(ss);
        if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x == 0) {
            double t = 0.0;
            for (int i = 0; i < 8; ++i) t += s_part[i];
            const float mean = __fdiv_rn((float)t, (float)n);
            s_r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
        }
        __syncthreads();
        const float r = s_r;
        for (uint32_t k = threadIdx.x; k < n; k += 256) {
            const float v = rr ? __fadd_rn(xr[k], rr[k]) : xr[k];
            if (h) h[(size_t)row * n + k] = v;
            float yv = __fmul_rn(v, r);
            if (w) yv = __fmul_rn(yv, w[k]);
            y[(size_t)row * n + k] = yv;
        }
        __syncthreads();
    }
}

// One decode token's q, k, v (the fused projection's output row, q | k | v):
// rotate q and k at the cursor's position (y = x cos + rotate_half(x) sin, two
// multiplies and an add as g2-rope.glsl:33-39), write q out, append k and v to
// the cache at the cursor. A full cache takes nothing more (g2-kv-write.glsl:46-50).
__global__ void __launch_bounds__(256) rope_kv_append_kernel(const float* __restrict__ qkv, const float* __restrict__ cosv,
                                                            const float* __restrict__ sinv, const uint32_t* __restrict__ lens,
                                                            uint32_t layer, uint32_t heads, uint32_t kv_heads, uint32_t dim,
                                                            uint32_t max_len, float* __restrict__ q_out, float* __restrict__ kc,
                                                            float* __restrict__ vc) {
    GQ_GRID_DEP_SYNC();
    const uint32_t pos = lens[layer];
    const uint32_t total = (heads + 2 * kv_heads) * dim, half = dim / 2;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const uint32_t hd = i / dim, d = i % dim;
        const float xv = qkv[i];
        if (hd < heads + kv_heads) {  // q or k: rotary
            const uint32_t p = min(pos, max_len - 1);
            const float rv = d < half ? -qkv[i + half] : qkv[i - half];
            const float y = __fadd_rn(__fmul_rn(xv, cosv[(size_t)p * dim + d]), __fmul_rn(rv, sinv[(size_t)p * dim + d]));
            if (hd < heads)
                q_out[i] = y;
            else if (pos < max_len)
                kc[((size_t)(hd - heads) * max_len + pos) * dim + d] = y;
        } else if (pos < max_len) {
            vc[((size_t)(hd - heads - kv_heads) * max_len + pos) * dim + d] = xv;
        }
    }
}

// lens[l] = min(lens[l] + 1, max_len) for every layer: once per step, after the last layer has attended.
__global__ void kv_advance_kernel(uint32_t* lens, uint32_t layers, uint32_t max_len) {
    GQ_GRID_DEP_SYNC();
    const uint32_t l = blockIdx.x * blockDim.x + threadIdx.x;
    if (l < layers) lens[l] = min(lens[l] + 1, max_len);
}

// out[r][j] = (g * sigmoid(g)) * u with g = gate_up[r][j], u = gate_up[r][width + j] (g2-swiglu.glsl:21-29;
// sigmoid as g2-common.glsl:163-166).
__global__ void __launch_bounds__(256) swiglu_kernel(const float* __restrict__ gate_up, uint32_t rows, uint32_t width,
                                                    float* __restrict__ out) {
    GQ_GRID_DEP_SYNC();
    const size_t total = (size_t)rows * width;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
        const size_t r = i / width, j = i % width;
        const float g = gate_up[r * 2 * width + j], u = gate_up[r * 2 * width + width + j];
        out[i] = silu_mul(g, u);
    }
}

// Greedy next token: the index of each row's maximum (the first one on ties; NaN ranks below every number).
// CTAs (b, row) each reduce a slice to one 64-bit key — the value's bits made monotone in the upper word, the
// complemented index in the lower — and atomicMax it into state[row]; the last CTA of a row to arrive (a counter
// after the 1024 keys of `state`) decodes the winner and puts both words back to zero for the next call.
constexpr uint32_t kArgmaxRows = 1024;  // rows one launch handles (and the size of the state)
__global__ void __launch_bounds__(256) argmax_rows_kernel(const float* __restrict__ v, uint32_t n, int32_t* __restrict__ out,
                                                         unsigned long long* state) {
    GQ_GRID_DEP_SYNC();
    __shared__ unsigned long long s_key[8];
    const uint32_t row = blockIdx.y;
    const float* vr = v + (size_t)row * n;
    unsigned long long best = 0;
    for (uint32_t i = blockIdx.x * 256 + threadIdx.x; i < n; i += gridDim.x * 256) {
        const float x = vr[i];
        const uint32_t bits = __float_as_uint(x);
        const uint32_t ord = x != x ? 1u : (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
        const unsigned long long key = ((unsigned long long)ord << 32) | (0xffffffffu - i);
        best = key > best ? key : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((threadIdx.x & 31) == 0) s_key[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) best = s_key[w] > best ? s_key[w] : best;
        atomicMax(state + row, best);
        __threadfence();
        uint32_t* counters = reinterpret_cast<uint32_t*>(state + kArgmaxRows);
        if (atomicAdd(counters + row, 1u) == gridDim.x - 1) {
            __threadfence();
            const unsigned long long win = atomicExch(state + row, 0ull);
            out[row] = (int32_t)(0xffffffffu - (uint32_t)win);
            counters[row] = 0;
        }
    }
}

// Grouped-query attention of one new token against the cache ("flash decoding"):
// CTA (split s, head h) scores keys [s * chunk, (s + 1) * chunk) of the head's
// KV group, keeps (max, sum of exp, weighted sum of values) and writes them to
// scratch; the last CTA of a head to finish — found with a counter in scratch,
// which it then resets — merges the splits:
//   out = sum_s acc_s exp(m_s - M) / sum_s z_s exp(m_s - M),  M = max_s m_s.
// The length is the cache cursor plus the token just appended, read from
// device memory. scratch: kAttnCounterWords counters (one per head) that must be
// zero before the first call and are left at zero by every call, then heads *
// splits * (dim + 2) floats. The counters come FIRST, at the same place whatever
// the shape, so that calls of different shapes may share one scratch: behind the
// partial results they would land inside what a call of another shape left there.
constexpr int kAttnThreads = 128;
constexpr uint32_t kAttnMaxChunk = 512;  // keys per split (scores live in shared memory)
constexpr uint32_t kAttnChunk = 32;      // keys per split aimed at: short dependent chains, many CTAs
constexpr uint32_t kAttnMaxSplits = 64;
constexpr uint32_t kAttnCounterWords = 1024;  // heads at most

// L = dim / 4 lanes share a key (one float4 of the row each), so a CTA takes 128 / L keys per pass with every
// load of the pass independent of the others.
//
// ROPE: `q` is the fused projection's raw row q | k | v instead. The CTA rotates its head of q itself at the cursor's
// position, the new token's key (rotated) and value are taken from that row wherever the cursor's position is needed —
// the cache row is stale there — and the first head of each KV group, in the split that holds the position, appends
// them to the cache: rope_kv_append_kernel's arithmetic and attn_decode_kernel's in one launch.
template <uint32_t L, bool ROPE>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(const float* __restrict__ q, float* kc, float* vc,
                                                                  const uint32_t* __restrict__ lens, uint32_t layer, uint32_t heads,
                                                                  uint32_t kv_heads, uint32_t max_len, float scale, uint32_t chunk,
                                                                  float* scratch, float* __restrict__ out, const float* __restrict__ cosv,
                                                                  const float* __restrict__ sinv, bool early) {
    // `early`: the kernel ahead in the stream wrote none of the cache, the cursor and the rotary tables, so they are read while
    // it still runs; the query row (and every write) waits for it.
    if (!early) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    constexpr uint32_t dim = 4 * L, KP = kAttnThreads / L;
    __shared__ float s_sc[kAttnMaxChunk];
    __shared__ float s_red[kAttnThreads / 32];
    __shared__ float4 s_acc[kAttnThreads];
    __shared__ bool s_last;
    const uint32_t split = blockIdx.x, splits = gridDim.x, h = blockIdx.y;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t sub = tid % L, grp = tid / L;
    const uint32_t g = h / (heads / kv_heads);
    const uint32_t j0 = split * chunk, jcap = min(j0 + chunk, max_len);  // where this split's keys lie, whatever the cursor says
    const float4* kb = reinterpret_cast<const float4*>(kc + (size_t)g * max_len * dim);
    const float4* vb = reinterpret_cast<const float4*>(vc + (size_t)g * max_len * dim);
    float* part = scratch + kAttnCounterWords + ((size_t)h * splits + split) * (dim + 2);
    uint32_t* counters = reinterpret_cast<uint32_t*>(scratch);

    // The first passes' keys AND values are requested at once, before the cursor is known (rows past it are valid
    // memory and are masked below): q, the cursor, K and V then cost one memory latency instead of four in a row.
    constexpr int kPre = 4;
    float4 kpre[kPre], vpre[kPre];
#pragma unroll
    for (int p = 0; p < kPre; ++p) {
        const uint32_t j = j0 + p * KP + grp;
        const bool in = j < jcap;
        kpre[p] = in ? kb[(size_t)j * L + sub] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        vpre[p] = in ? vb[(size_t)j * L + sub] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    const uint32_t pos = lens[layer];
    const uint32_t len = min(pos + 1, max_len);
    const uint32_t j1 = min(len, j0 + chunk);
    float4 knew = make_float4(0.0f, 0.0f, 0.0f, 0.0f), vnew = knew;
    float4 c4 = knew, s4 = knew;
    if (ROPE) {
        const uint32_t p = min(pos, max_len - 1);
        c4 = reinterpret_cast<const float4*>(cosv + (size_t)p * dim)[sub], s4 = reinterpret_cast<const float4*>(sinv + (size_t)p * dim)[sub];
    }
    if (early) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    float4 q4 = reinterpret_cast<const float4*>(q + (size_t)h * dim)[sub];
    if (ROPE) {
        // y = x cos + rotate_half(x) sin; rotate_half(x)[d] = -x[d + dim/2] below dim/2, x[d - dim/2] above
        const uint32_t partner = (sub + L / 2) % L;
        const float sign = sub < L / 2 ? -1.0f : 1.0f;
        auto rotate = [&](const float4& xv, const float4& pv) {
            float4 r;
            r.x = __fadd_rn(__fmul_rn(xv.x, c4.x), __fmul_rn(sign * pv.x, s4.x)), r.y = __fadd_rn(__fmul_rn(xv.y, c4.y), __fmul_rn(sign * pv.y, s4.y));
            r.z = __fadd_rn(__fmul_rn(xv.z, c4.z), __fmul_rn(sign * pv.z, s4.z)), r.w = __fadd_rn(__fmul_rn(xv.w, c4.w), __fmul_rn(sign * pv.w, s4.w));
            return r;
        };
        q4 = rotate(q4, reinterpret_cast<const float4*>(q + (size_t)h * dim)[partner]);
        if (pos < max_len && pos >= j0 && pos < j0 + chunk) {  // this split holds the new token (uniform over the CTA)
            const float4* kraw = reinterpret_cast<const float4*>(q + (size_t)(heads + g) * dim);
            knew = rotate(kraw[sub], kraw[partner]);
            vnew = reinterpret_cast<const float4*>(q + (size_t)(heads + kv_heads + g) * dim)[sub];
            if (h % (heads / kv_heads) == 0 && grp == 0) {
                reinterpret_cast<float4*>(kc + ((size_t)g * max_len + pos) * dim)[sub] = knew;
                reinterpret_cast<float4*>(vc + ((size_t)g * max_len + pos) * dim)[sub] = vnew;
            }
        }
    }
    const uint32_t jnew = ROPE && pos < max_len ? pos : 0xffffffffu;  // the key whose cache row must not be used

    // Every lane of a warp runs the same number of passes (the shuffles below name the whole warp): a lane
    // whose key lies past the end computes on zeros and keeps nothing.
    float m = -INFINITY;
    const uint32_t passes = j1 > j0 ? (j1 - j0 + KP - 1) / KP : 0;
    auto score = [&](uint32_t j, bool live, const float4& k4) {
        float sdot = __fmaf_rn(q4.w, k4.w, __fmaf_rn(q4.z, k4.z, __fmaf_rn(q4.y, k4.y, __fmul_rn(q4.x, k4.x))));
#pragma unroll
        for (uint32_t o = L / 2; o > 0; o >>= 1) sdot += __shfl_xor_sync(0xffffffffu, sdot, o);
        sdot *= scale;
        if (live) {
            if (sub == 0) s_sc[j - j0] = sdot;
            m = fmaxf(m, sdot);
        }
    };
#pragma unroll
    for (int p = 0; p < kPre; ++p) {
        if ((uint32_t)p < passes) {  // uniform over the CTA
            const uint32_t j = j0 + p * KP + grp;
            const bool live = j < j1;
            score(j, live, !live ? make_float4(0.0f, 0.0f, 0.0f, 0.0f) : j == jnew ? knew : kpre[p]);
        }
    }
#pragma unroll 4
    for (uint32_t pass = kPre; pass < passes; ++pass) {
        const uint32_t j = j0 + pass * KP + grp;
        const bool live = j < j1;
        score(j, live, !live ? make_float4(0.0f, 0.0f, 0.0f, 0.0f) : j == jnew ? knew : kb[(size_t)j * L + sub]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    m = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
    __syncthreads();

    float z = 0.0f;
    for (uint32_t j = j0 + tid; j < j1; j += kAttnThreads) {
        const float e = exp_cephes(s_sc[j - j0] - m);
        s_sc[j - j0] = e;
        z += e;
    }
    z = warp_sum(z);
    if (lane == 0) s_red[warp] = z;
    __syncthreads();
    z = (s_red[0] + s_red[1]) + (s_red[2] + s_red[3]);

    // weighted values: group `grp` strides over the keys, lane `sub` owns one float4 of the output
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    auto weigh = [&](uint32_t j, const float4& v4) {
        const float p = s_sc[j - j0];
        acc.x = __fmaf_rn(p, v4.x, acc.x), acc.y = __fmaf_rn(p, v4.y, acc.y);
        acc.z = __fmaf_rn(p, v4.z, acc.z), acc.w = __fmaf_rn(p, v4.w, acc.w);
    };
#pragma unroll
    for (int p = 0; p < kPre; ++p) {
        const uint32_t j = j0 + p * KP + grp;
        if (j < j1) weigh(j, j == jnew ? vnew : vpre[p]);
    }
#pragma unroll 4
    for (uint32_t j = j0 + kPre * KP + grp; j < j1; j += KP) weigh(j, j == jnew ? vnew : vb[(size_t)j * L + sub]);
    s_acc[tid] = acc;
    __syncthreads();
    if (tid < L) {
        float4 t = s_acc[tid];
        for (uint32_t k = 1; k < KP; ++k) {
            const float4 o = s_acc[k * L + tid];
            t.x += o.x, t.y += o.y, t.z += o.z, t.w += o.w;
        }
        part[2 + 4 * tid] = t.x, part[3 + 4 * tid] = t.y, part[4 + 4 * tid] = t.z, part[5 + 4 * tid] = t.w;
    }
    if (tid == 0) part[0] = m, part[1] = z;

    // the last split of this head to arrive merges
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const uint32_t seen = atomicAdd(counters + h, 1u);
        s_last = seen == splits - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* hp = scratch + kAttnCounterWords + (size_t)h * splits * (dim + 2);
    // the weights exp(m_s - M) once, in shared memory (the scores are no longer needed)
    float M = -INFINITY;
    for (uint32_t s = 0; s < splits; ++s) M = fmaxf(M, __ldcg(hp + s * (dim + 2)));
    for (uint32_t s = tid; s < splits; s += kAttnThreads) {
        const float ms = __ldcg(hp + s * (dim + 2));
        s_sc[s] = ms == -INFINITY ? 0.0f : exp_cephes(ms - M);  // an empty split contributes nothing
    }
    __syncthreads();
    if (tid < dim) {
        float Z = 0.0f, o = 0.0f;
#pragma unroll 4
        for (uint32_t s = 0; s < splits; ++s) {
            const float wgt = s_sc[s];
            Z = __fmaf_rn(__ldcg(hp + s * (dim + 2) + 1), wgt, Z);
            o = __fmaf_rn(__ldcg(hp + s * (dim + 2) + 2 + tid), wgt, o);
        }
        out[(size_t)h * dim + tid] = __fdiv_rn(o, Z);
    }
    if (tid == 0) counters[h] = 0;  // ready for the next call
}

}  // namespace

static inline uint32_t blocks_for(size_t items, uint32_t per, uint32_t cap) {
    size_t b = (items + per - 1) / per;
    return (uint32_t)(b < 1 ? 1 : b > cap ? cap : b);
}

void launch_embedding(cudaStream_t s, const float* table, const int32_t* ids, uint64_t rows, uint64_t width, uint64_t vocab, float* out) {
    launch_after(embedding_kernel, dim3(blocks_for(rows, 1, 1024)), dim3(256), 0, s, table, ids, (uint32_t)rows, (uint32_t)width, (uint32_t)vocab, out);
}
void launch_add_rms_norm(cudaStream_t s, const float* x, const float* res, const float* w, uint64_t rows, uint64_t n, float eps,
                         float* y, float* h) {
    launch_after(add_rms_norm_kernel, dim3(blocks_for(rows, 1, 1024)), dim3(256), 0, s, x, res, w, (uint32_t)rows, (uint32_t)n, eps, y, h);
}
void launch_rope_kv_append(cudaStream_t s, const float* qkv, const float* cosv, const float* sinv, const uint32_t* lens, uint32_t layer,
                           uint32_t heads, uint32_t kv_heads, uint32_t dim, uint32_t max_len, float* q_out, float* kc, float* vc) {
    const uint32_t total = (heads + 2 * kv_heads) * dim;
    launch_after(rope_kv_append_kernel, dim3(blocks_for(total, 256, 64)), dim3(256), 0, s, qkv, cosv, sinv, lens, layer, heads, kv_heads, dim, max_len,
                 q_out, kc, vc);
}
void launch_kv_advance(cudaStream_t s, uint32_t* lens, uint32_t layers, uint32_t max_len) {
    launch_after(kv_advance_kernel, dim3((layers + 127) / 128), dim3(128), 0, s, lens, layers, max_len);
}
// Splits of the cache length: about kAttnChunk keys each, at most kAttnMaxSplits (more only where a split would
// otherwise exceed the kAttnMaxChunk scores that fit in shared memory).
uint32_t attn_splits(uint32_t heads, uint32_t max_len, int sm_count) {
    (void)heads, (void)sm_count;
    uint32_t splits = (max_len + kAttnChunk - 1) / kAttnChunk;
    if (splits > kAttnMaxSplits) splits = kAttnMaxSplits;
    const uint32_t need = (max_len + kAttnMaxChunk - 1) / kAttnMaxChunk;
    if (splits < need) splits = need;
    return splits < 1 ? 1 : splits;
}
uint64_t attn_scratch_floats(uint32_t heads, uint32_t dim, uint32_t splits) { return (uint64_t)kAttnCounterWords + (uint64_t)heads * splits * (dim + 2); }
// cosv == nullptr: q is the rotated query and the cache already holds the new token (after rope_kv_append). Otherwise q is the raw
// q | k | v row, rotated and appended here.
void launch_attn_decode(cudaStream_t s, const float* q, float* kc, float* vc, const uint32_t* lens, uint32_t layer, uint32_t heads,
                        uint32_t kv_heads, uint32_t dim, uint32_t max_len, float scale, uint32_t splits, float* scratch, float* out,
                        const float* cosv, const float* sinv, bool early) {
    const uint32_t chunk = (max_len + splits - 1) / splits;
    if (heads > kAttnCounterWords) fail("attention: at most %u heads (got %u)", kAttnCounterWords, heads);
    if (splits > kAttnMaxChunk || chunk > kAttnMaxChunk)
        fail("attention: a cache of %u positions is beyond this kernel (%u splits of %u keys)", max_len, splits, chunk);
    const dim3 grid(splits, heads);
#define GQ_ATTN(LV)                                                                                                                   \
    do {                                                                                                                              \
        if (cosv)                                                                                                                     \
            launch_after(attn_decode_kernel<LV, true>, grid, dim3(kAttnThreads), 0, s, q, kc, vc, lens, layer, heads, kv_heads, max_len, \
                         scale, chunk, scratch, out, cosv, sinv, early);                                                              \
        else                                                                                                                          \
            launch_after(attn_decode_kernel<LV, false>, grid, dim3(kAttnThreads), 0, s, q, kc, vc, lens, layer, heads, kv_heads, max_len, \
                         scale, chunk, scratch, out, cosv, sinv, early);                                                              \
    } while (0)
    if (dim == 32)
        GQ_ATTN(8);
    else if (dim == 64)
        GQ_ATTN(16);
    else if (dim == 128)
        GQ_ATTN(32);
    else
        fail("attention: head_dim must be 32, 64 or 128, got %u", dim);
#undef GQ_ATTN
}
void launch_swiglu(cudaStream_t s, const float* gate_up, uint64_t rows, uint64_t width, float* out) {
    launch_after(swiglu_kernel, dim3(blocks_for(rows * width, 256, 148 * 8)), dim3(256), 0, s, gate_up, (uint32_t)rows, (uint32_t)width, out);
}
uint64_t argmax_state_bytes() { return kArgmaxRows * 12ull; }
void launch_argmax_rows(cudaStream_t s, const float* v, uint64_t rows, uint64_t n, int32_t* out, void* state) {
    const uint32_t per_row = blocks_for(n, 1024, rows >= 64 ? 4 : 148);
    for (uint64_t r0 = 0; r0 < rows; r0 += kArgmaxRows) {
        const uint32_t now = (uint32_t)(rows - r0 < kArgmaxRows ? rows - r0 : kArgmaxRows);
        launch_after(argmax_rows_kernel, dim3(per_row, now), dim3(256), 0, s, v + r0 * n, (uint32_t)n, out + r0, (unsigned long long*)state);
    }
}

}  // namespace gq
