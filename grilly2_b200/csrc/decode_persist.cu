// One decode token of the int8 weight-only Llama / Qwen2 decoder as ONE
// persistent kernel: every SM keeps a CTA resident for the whole step, the
// operators of the step are phases separated by grid-wide barriers, and each
// CTA's share of every weight matrix is prefetched into shared memory phases
// ahead, so that what a phase waits for is the barrier, not HBM.
//
// Why: as separate launches the step is 125 dependent kernels of ~5 us each
// (0.66 ms per token) although its 520 MB could stream in 80 us; the reference
// has the same structure, one dispatch per operator
// (python/grilly/infer/models/llama.py:353-366, 273 dispatches, 5.9 ms). Here a
// layer is five phases:
//   1  h += delta; x = rms_norm(h) w_in;  q|k|v rows of this CTA = Wqkv x + b
//   2  rotary, cache append, grouped-query attention over the cache: kv_heads x 32 CTAs take 1/32 of the positions
//      each, the last to finish a kv head merges its splits (the other CTAs go straight to the barrier)
//   3  o rows = Wo attn
//   4  h += o; x = rms_norm(h) w_post;  act rows = silu(Wgate x) * (Wup x)
//   5  delta rows = Wdown act
// then the final norm, the tied head (every CTA streams its 1/148 of the 136 MB
// through the same ring) and the arg-max. The residual stream h lives in every
// CTA's shared memory (each CTA applies the same updates), so it never travels.
//
// Arithmetic is the fast GEMV's (gemv_dp4a.cu): the phase's input vector is
// held as an exact fixed-point integer, X = rint(x 2^(30-e)), 2^e > max|x|,
// split in four signed base-256 digits; dp4a multiplies them by the int8
// codes exactly; the four sums are recombined in float64 and scaled once.
// Norm, SiLU, rotary and softmax are the separate operators' (decode_ops.cu).
//
// Measured on the int8 full-step configuration (24 layers, hidden 896, cache 1024): 0.93 ms per token against 0.66 ms
// for the launch-per-operator step, so the decoder does NOT select it by default. Stamps of %globaltimer around
// every barrier show why: a grid-wide barrier costs 2.1-2.5 us here (one release-add and acquire-polls through L2) and
// a phase another 3-8 us of which the arithmetic is a fraction — after a barrier every CTA re-reads the phase's input
// vector from L2, reduces its maximum, converts it, computes its few rows and publishes them — so 121 phases cost what
// 125 dependent launches with programmatic dependent launch cost (~5.3 us each). The step is bound by the number of
// grid-wide dependencies, five per layer, not by how they are expressed.
//
// Weight ring: a producer warp walks the CTA's fixed sequence of slices (its
// rows of each matrix, with their scales and bias, as bulk copies), three
// slices in flight in 192 KB. Barriers: one counter in global memory, bounded
// spins; a wait that gives up sets the status word and an abort flag that every
// CTA sees at its next barrier, so nothing hangs.
#include <algorithm>
#include <memory>

#include "async_common.cuh"
#include "gq_internal.h"
#include "math_common.cuh"

namespace gq {

namespace {

constexpr int kWarps = 16;
constexpr int kThreads = (kWarps + 1) * 32;  // + the producer warp
constexpr uint32_t kSlots = 3;               // slices in flight
constexpr uint32_t kRingBytes = 192 * 1024;
constexpr uint32_t kSplits = 32;             // attention: splits of the cache length per kv head
constexpr uint32_t kHeadRows = 32;           // rows of the head per slice

struct LayerPtrs {
    const float* in_norm;
    const uint8_t* qkv_q;
    const float* qkv_scale;
    const float* qkv_bias;  // may be null
    const uint8_t* o_q;
    const float* o_scale;
    const float* post_norm;
    const uint8_t* gu_q;
    const float* gu_scale;
    const uint8_t* down_q;
    const float* down_scale;
};

struct StepArgs {
    const LayerPtrs* layers;
    const float* embed;
    const int32_t* token;
    const float* final_norm;
    const uint8_t* head_q;
    const float* head_scale;
    const float* cosv;
    const float* sinv;
    float* kcache;
    float* vcache;
    uint32_t* lens;
    // activations that cross CTAs (global memory)
    float* qkv;     // [q_size + 2 kv_size]
    float* attn;    // [q_size]
    float* o;       // [hidden]
    float* act;     // [inter]
    float* delta;   // [hidden]
    float* logits;  // [vocab]
    int32_t* next_token;
    float* attn_part;          // [heads][kSplits][dim + 2]
    uint32_t* sync;            // [0] barrier counter, [1] exit ticket, [2] abort, [4 .. 4 + kv_heads) attention arrivals
    unsigned long long* best;  // arg-max key
    uint32_t* status;
    uint32_t hidden, heads, kv_heads, dim, inter, vocab, nlayers, max_len;
    float eps, attn_scale;
    long long wait_cycles;
};

// A slice of the CTA's weight sequence: up to two runs of matrix rows, their scales, one bias.
struct Slice {
    const uint8_t* w[2];
    const float* sc[2];
    const float* bias;
    uint32_t r0[2], rows[2], kbytes;
};

__device__ __forceinline__ uint32_t lo_of(uint32_t n, uint32_t c, uint32_t g) { return (uint32_t)((uint64_t)n * c / g); }
__device__ __forceinline__ uint32_t span_lo(uint32_t r0) { return r0 & ~3u; }                       // scales travel in whole 16-byte pieces
__device__ __forceinline__ uint32_t span_floats(uint32_t r0, uint32_t rows) { return ((r0 + rows + 3u) & ~3u) - (r0 & ~3u); }

// Slice number `i` of CTA `c`: layer slices first (four per layer), then the head in chunks of kHeadRows rows.
__device__ Slice slice_of(const StepArgs& a, uint32_t i, uint32_t c, uint32_t g) {
    Slice s{};
    const uint32_t q_size = a.heads * a.dim, kv_size = a.kv_heads * a.dim;
    if (i < 4 * a.nlayers) {
        const LayerPtrs& L = a.layers[i >> 2];
        switch (i & 3u) {
            case 0: {
                const uint32_t n = q_size + 2 * kv_size;
                s.w[0] = L.qkv_q, s.sc[0] = L.qkv_scale, s.bias = L.qkv_bias, s.kbytes = a.hidden;
                s.r0[0] = lo_of(n, c, g), s.rows[0] = lo_of(n, c + 1, g) - s.r0[0];
                break;
            }
            case 1:
                s.w[0] = L.o_q, s.sc[0] = L.o_scale, s.kbytes = q_size;
                s.r0[0] = lo_of(a.hidden, c, g), s.rows[0] = lo_of(a.hidden, c + 1, g) - s.r0[0];
                break;
            case 2:
                s.w[0] = s.w[1] = L.gu_q, s.sc[0] = s.sc[1] = L.gu_scale, s.kbytes = a.hidden;
                s.r0[0] = lo_of(a.inter, c, g), s.rows[0] = lo_of(a.inter, c + 1, g) - s.r0[0];
                s.r0[1] = a.inter + s.r0[0], s.rows[1] = s.rows[0];
                break;
            default:
                s.w[0] = L.down_q, s.sc[0] = L.down_scale, s.kbytes = a.inter;
                s.r0[0] = lo_of(a.hidden, c, g), s.rows[0] = lo_of(a.hidden, c + 1, g) - s.r0[0];
                break;
        }
    } else {
        const uint32_t j = i - 4 * a.nlayers, v0 = lo_of(a.vocab, c, g), v1 = lo_of(a.vocab, c + 1, g);
        s.w[0] = a.head_q, s.sc[0] = a.head_scale, s.kbytes = a.hidden;
        s.r0[0] = v0 + j * kHeadRows;
        s.rows[0] = s.r0[0] < v1 ? min(kHeadRows, v1 - s.r0[0]) : 0u;
    }
    return s;
}
__device__ __forceinline__ uint32_t head_slices(const StepArgs& a, uint32_t c, uint32_t g) {
    const uint32_t rows = lo_of(a.vocab, c + 1, g) - lo_of(a.vocab, c, g);
    return (rows + kHeadRows - 1) / kHeadRows;
}
// Byte layout of a slice in the ring: [rows0 | rows1 | scale span 0 | scale span 1 | bias span], each a multiple of 16 bytes.
__device__ __forceinline__ uint32_t slice_bytes(const Slice& s) {
    uint32_t b = (s.rows[0] + s.rows[1]) * s.kbytes;
    b += 4 * span_floats(s.r0[0], s.rows[0]);
    if (s.rows[1]) b += 4 * span_floats(s.r0[1], s.rows[1]);
    if (s.bias) b += 4 * span_floats(s.r0[0], s.rows[0]);
    return (b + 127u) & ~127u;
}
__device__ __forceinline__ uint32_t ring_place(uint32_t& off, uint32_t bytes) {  // the same walk on the producer's and the consumers' side
    if (off + bytes > kRingBytes) off = 0;
    const uint32_t at = off;
    off += bytes;
    return at;
}

__device__ __forceinline__ uint32_t fkey(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b >> 31) ? ~b : (b | 0x80000000u);
}

struct Shared {
    uint64_t full[kSlots], empty[kSlots];
    double red_d[kWarps];
    float red_f[kWarps];
    float inv;         // 2^(e-30) of the current input vector
    float rnorm;       // 1 / sqrt(mean(h^2) + eps)
    uint32_t abort;
    uint32_t last;
    volatile uint32_t failed;
};

__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(StepArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    Shared& sh = *reinterpret_cast<Shared*>(smem);
    float* hres = reinterpret_cast<float*>(smem + 512);                       // [hidden]
    const uint32_t kmax = max(a.hidden, a.inter);
    uint4* xdig = reinterpret_cast<uint4*>(smem + 512 + ((a.hidden * 4 + 127) & ~127u));  // [kmax / 4]: four digit words per four values
    float* qrot = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(xdig) + ((kmax * 4 + 127) & ~127u));   // attention: [heads / kv_heads][dim] + k[dim] + v[dim]
    const uint32_t rep = a.heads / a.kv_heads;
    uint8_t* ring = reinterpret_cast<uint8_t*>(qrot) + (((rep + 2) * a.dim * 4 + 127) & ~127u);

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, c = blockIdx.x, g = gridDim.x;
    const uint32_t nslices = 4 * a.nlayers + head_slices(a, c, g);
    if (tid == 0) {
        for (uint32_t s = 0; s < kSlots; ++s) mbar_init(sh.full + s, 1), mbar_init(sh.empty + s, 1);
        sh.abort = 0, sh.failed = 0;
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == kWarps) {
        // ── producer: the CTA's slices in order, at most kSlots in flight ──
        if (lane == 0) {
            uint32_t off = 0;
            for (uint32_t i = 0; i < nslices; ++i) {
                const uint32_t q = i % kSlots;
                if (i >= kSlots && !mbar_wait(sh.empty + q, (i / kSlots - 1) & 1, &sh.failed, a.status, kStatusEmptyWaitTimedOut)) break;
                const Slice s = slice_of(a, i, c, g);
                if (s.rows[0] == 0) {  // nothing of this matrix for this CTA: the consumers skip the slice as well
                    mbar_arrive(sh.full + q);
                    continue;
                }
                const uint32_t bytes = slice_bytes(s);
                uint8_t* dst = ring + ring_place(off, bytes);
                uint32_t tx = (s.rows[0] + s.rows[1]) * s.kbytes + 4 * span_floats(s.r0[0], s.rows[0]);
                if (s.rows[1]) tx += 4 * span_floats(s.r0[1], s.rows[1]);
                if (s.bias) tx += 4 * span_floats(s.r0[0], s.rows[0]);
                mbar_arrive_expect_tx(sh.full + q, tx);
                for (int p = 0; p < 2; ++p) {
                    if (!s.rows[p]) continue;
                    const uint32_t wb = s.rows[p] * s.kbytes;
                    for (uint32_t o = 0; o < wb; o += 32768u) bulk_load(dst + o, s.w[p] + (size_t)s.r0[p] * s.kbytes + o, min(32768u, wb - o), sh.full + q);
                    dst += wb;
                }
                for (int p = 0; p < 2; ++p) {
                    if (!s.rows[p]) continue;
                    const uint32_t sb = 4 * span_floats(s.r0[p], s.rows[p]);
                    bulk_load(dst, s.sc[p] + span_lo(s.r0[p]), sb, sh.full + q);
                    dst += sb;
                }
                if (s.bias) bulk_load(dst, s.bias + span_lo(s.r0[0]), 4 * span_floats(s.r0[0], s.rows[0]), sh.full + q);
            }
        }
        return;
    }

    // ── consumers (512 threads) ──
    auto csync = [&]() { named_barrier_sync(1, kWarps * 32); };
    uint32_t epoch = 0;
    // grid-wide barrier over the consumers of every CTA; false once any CTA gave up
    auto grid_barrier = [&]() -> bool {
        csync();
        if (tid == 0) {
            ++epoch;
            // the CTA's writes were ordered before this thread by the barrier above; the release makes them visible device-wide
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(a.sync) : "memory");
            const uint32_t want = epoch * g;
            const long long start = clock64();
            volatile uint32_t* ab = a.sync + 2;
            for (;;) {
                uint32_t seen;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(a.sync) : "memory");
                if ((int32_t)(seen - want) >= 0) break;
                if (*ab) break;
                if (clock64() - start > a.wait_cycles) {
                    atomicCAS(a.status, 0u, 4u);  // a grid-wide barrier was never completed
                    atomicExch(a.sync + 2, 1u);
                    break;
                }
            }
            sh.abort = *ab;
        }
        csync();
        return sh.abort == 0;
    };
    uint32_t slice_i = 0, ring_off = 0;
    // waits for the next slice of the CTA's sequence; returns its place in the ring (nullptr: no rows here, or gave up)
    auto take_slice = [&](Slice& s) -> const uint8_t* {
        s = slice_of(a, slice_i, c, g);
        const uint32_t q = slice_i % kSlots;
        bool ok = true;
        if (lane == 0) ok = mbar_wait(sh.full + q, (slice_i / kSlots) & 1, &sh.failed, a.status, kStatusFullWaitTimedOut);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok || s.rows[0] == 0) return nullptr;
        return ring + ring_place(ring_off, slice_bytes(s));
    };
    auto release_slice = [&]() {  // every consumer has finished with it
        csync();
        if (tid == 0) mbar_arrive(sh.empty + slice_i % kSlots);
        ++slice_i;
    };
    // The phase's input vector v[0 .. n) (each thread its groups of four: group gi = tid + 512 j) -> digit words in xdig, 2^(e-30) in sh.inv.
    // `vals` holds the thread's groups; n % 4 == 0.
    auto to_digits = [&](const float4* vals, uint32_t n) {
        float amax = 0.0f;
        bool bad = false;
        uint32_t j = 0;
        for (uint32_t gi = tid; gi < n / 4; gi += kWarps * 32, ++j) {
            const float4 v = vals[j];
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            bad |= !(fabsf(v.x) <= 3.402823466e+38f) | !(fabsf(v.y) <= 3.402823466e+38f) | !(fabsf(v.z) <= 3.402823466e+38f) | !(fabsf(v.w) <= 3.402823466e+38f);
        }
        if (bad) amax = __uint_as_float(0x7f800000u);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (lane == 0) sh.red_f[warp] = amax;
        csync();
        amax = sh.red_f[0];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) amax = fmaxf(amax, sh.red_f[w]);
        uint32_t e = __float_as_uint(amax) >> 23;
        float mult, inv;
        if (e == 255) mult = 0.0f, inv = __uint_as_float(0x7fc00000u);
        else if (amax == 0.0f) mult = inv = 0.0f;
        else {
            e = max(e, 32u);
            mult = __uint_as_float((283u - e) << 23), inv = __uint_as_float((e - 29u) << 23);
        }
        if (tid == 0) sh.inv = inv;
        j = 0;
        for (uint32_t gi = tid; gi < n / 4; gi += kWarps * 32, ++j) {
            const float v[4] = {vals[j].x, vals[j].y, vals[j].z, vals[j].w};
            uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                int X = __float2int_rn(v[b] * mult);
                const int d0 = (int)(int8_t)X;
                X = (X - d0) >> 8;
                const int d1 = (int)(int8_t)X;
                X = (X - d1) >> 8;
                const int d2 = (int)(int8_t)X;
                const int d3 = (X - d2) >> 8;
                w[0] |= ((uint32_t)d0 & 0xFFu) << (8 * b), w[1] |= ((uint32_t)d1 & 0xFFu) << (8 * b);
                w[2] |= ((uint32_t)d2 & 0xFFu) << (8 * b), w[3] |= ((uint32_t)d3 & 0xFFu) << (8 * b);
            }
            xdig[gi] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        csync();
    };
    // sum_k x[k] q[row][k] for one row of the slice (the whole warp): exact digit sums, recombined in float64
    auto row_dot = [&](const uint8_t* rowp, uint32_t kbytes) -> float {
        int a0 = 0, a1 = 0, a2 = 0, a3 = 0;
        const uint32_t* wp = reinterpret_cast<const uint32_t*>(rowp);
        for (uint32_t i = lane; i < kbytes / 4; i += 32) {
            const int w = (int)wp[i];
            const uint4 d = xdig[i];
            a0 = __dp4a(w, (int)d.x, a0), a1 = __dp4a(w, (int)d.y, a1), a2 = __dp4a(w, (int)d.z, a2), a3 = __dp4a(w, (int)d.w, a3);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            a0 += __shfl_xor_sync(0xffffffffu, a0, o), a1 += __shfl_xor_sync(0xffffffffu, a1, o);
            a2 += __shfl_xor_sync(0xffffffffu, a2, o), a3 += __shfl_xor_sync(0xffffffffu, a3, o);
        }
        const double t = (double)a0 + 256.0 * (double)a1 + 65536.0 * (double)a2 + 16777216.0 * (double)a3;
        return (float)(t * (double)sh.inv);
    };
    // h (+= add) ; x = h / sqrt(mean(h^2) + eps) * w  -> digits (add_rms_norm_kernel's arithmetic, the sum of squares in float64)
    auto norm_to_digits = [&](const float* add, const float* w) {
        float4 vals[2];  // hidden <= 4096: at most two groups of four per thread
        double ss = 0.0;
        uint32_t j = 0;
        for (uint32_t gi = tid; gi < a.hidden / 4; gi += kWarps * 32, ++j) {
            float4 h = reinterpret_cast<const float4*>(hres)[gi];
            if (add) {
                const float4 d = __ldcg(reinterpret_cast<const float4*>(add) + gi);
                h.x = __fadd_rn(h.x, d.x), h.y = __fadd_rn(h.y, d.y), h.z = __fadd_rn(h.z, d.z), h.w = __fadd_rn(h.w, d.w);
                reinterpret_cast<float4*>(hres)[gi] = h;
            }
            vals[j] = h;
            ss += (double)__fmul_rn(h.x, h.x) + (double)__fmul_rn(h.y, h.y) + (double)__fmul_rn(h.z, h.z) + (double)__fmul_rn(h.w, h.w);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) sh.red_d[warp] = ss;
        csync();
        if (tid == 0) {
            double t = 0.0;
            for (int i = 0; i < kWarps; ++i) t += sh.red_d[i];
            sh.rnorm = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn((float)t, (float)a.hidden), a.eps)));
        }
        csync();
        const float r = sh.rnorm;
        j = 0;
        for (uint32_t gi = tid; gi < a.hidden / 4; gi += kWarps * 32, ++j) {
            const float4 wv = __ldg(reinterpret_cast<const float4*>(w) + gi);
            vals[j].x = __fmul_rn(__fmul_rn(vals[j].x, r), wv.x), vals[j].y = __fmul_rn(__fmul_rn(vals[j].y, r), wv.y);
            vals[j].z = __fmul_rn(__fmul_rn(vals[j].z, r), wv.z), vals[j].w = __fmul_rn(__fmul_rn(vals[j].w, r), wv.w);
        }
        to_digits(vals, a.hidden);
    };
    // a vector another phase left in global memory -> digits
    auto global_to_digits = [&](const float* v, uint32_t n) {
        float4 vals[4];  // n <= 8192
        uint32_t j = 0;
        for (uint32_t gi = tid; gi < n / 4; gi += kWarps * 32, ++j) vals[j] = __ldcg(reinterpret_cast<const float4*>(v) + gi);
        to_digits(vals, n);
    };
    // y[r] = dot * scale[r] (+ bias[r]) for the slice's first run of rows, a warp per row
    auto gemv_rows = [&](const uint8_t* base, const Slice& s, float* out) {
        const float* sc = reinterpret_cast<const float*>(base + s.rows[0] * s.kbytes) + (s.r0[0] - span_lo(s.r0[0]));
        const float* bs = s.bias ? reinterpret_cast<const float*>(base + s.rows[0] * s.kbytes + 4 * span_floats(s.r0[0], s.rows[0])) + (s.r0[0] - span_lo(s.r0[0])) : nullptr;
        for (uint32_t r = warp; r < s.rows[0]; r += kWarps) {
            const float d = row_dot(base + (size_t)r * s.kbytes, s.kbytes);
            if (lane == 0) {
                float y = __fmul_rn(d, sc[r]);
                if (bs) y = __fadd_rn(y, bs[r]);
                out[s.r0[0] + r] = y;
            }
        }
    };

    const uint32_t q_size = a.heads * a.dim, kv_size = a.kv_heads * a.dim;
    const uint32_t pos = a.lens[0];  // the cursor, the same for every layer
    {  // h = embedding of the token
        const int32_t tok = *a.token;
        const bool ok = tok >= 0 && (uint32_t)tok < a.vocab;
        for (uint32_t i = tid; i < a.hidden; i += kWarps * 32) hres[i] = ok ? a.embed[(size_t)tok * a.hidden + i] : __uint_as_float(0x7fc00000u);
        csync();
    }
    bool alive = true;
    Slice s;
    for (uint32_t l = 0; l < a.nlayers && alive; ++l) {
        const LayerPtrs& L = a.layers[l];
        // ── phase 1: norm, q | k | v ──
        norm_to_digits(l ? a.delta : nullptr, L.in_norm);
        if (const uint8_t* base = take_slice(s)) gemv_rows(base, s, a.qkv);
        release_slice();
        if (!(alive = grid_barrier())) break;
        // ── phase 2: attention ──
        if (c < a.kv_heads * kSplits) {
            const uint32_t kvh = c / kSplits, split = c % kSplits, dim = a.dim, half = dim / 2;
            const uint32_t p = min(pos, a.max_len - 1);
            const uint32_t n_att = min(pos + 1, a.max_len);  // positions attended to
            const uint32_t chunk = (a.max_len + kSplits - 1) / kSplits, j0 = split * chunk, j1 = min(j0 + chunk, n_att);
            float* knew = qrot + rep * dim;
            float* vnew = knew + dim;
            // rotary on this group's queries and on the new key (rope_kv_append_kernel's arithmetic)
            for (uint32_t i = tid; i < (rep + 2) * dim; i += kWarps * 32) {
                const uint32_t hd = i / dim, d = i % dim;
                const float* src = hd < rep ? a.qkv + (size_t)(kvh * rep + hd) * dim : hd == rep ? a.qkv + q_size + (size_t)kvh * dim : a.qkv + q_size + kv_size + (size_t)kvh * dim;
                const float xv = __ldcg(src + d);
                float y = xv;
                if (hd <= rep) {
                    const float rv = d < half ? -__ldcg(src + d + half) : __ldcg(src + d - half);
                    y = __fadd_rn(__fmul_rn(xv, a.cosv[(size_t)p * dim + d]), __fmul_rn(rv, a.sinv[(size_t)p * dim + d]));
                }
                qrot[i] = y;
            }
            csync();
            float* kc = a.kcache + ((size_t)l * a.kv_heads + kvh) * a.max_len * dim;
            float* vc = a.vcache + ((size_t)l * a.kv_heads + kvh) * a.max_len * dim;
            if (pos < a.max_len && pos >= j0 && pos < j0 + chunk)  // the split that holds the cursor appends
                for (uint32_t d = tid; d < dim; d += kWarps * 32) kc[(size_t)pos * dim + d] = knew[d], vc[(size_t)pos * dim + d] = vnew[d];
            // The split's keys and values go to shared memory once (all loads in flight together: one memory latency), rows
            // padded by one float so that a lane per position reads without bank conflicts; the seven query heads of the group
            // then work from there. The next layer's rows are asked into L2 meanwhile.
            const uint32_t pitch = dim + 1, npos = j1 > j0 ? j1 - j0 : 0u;
            float* ks = reinterpret_cast<float*>(xdig);  // the digit area is free during this phase
            float* vs = ks + chunk * pitch;
            if (l + 1 < a.nlayers) {
                const size_t next = (size_t)a.kv_heads * a.max_len * dim;
                for (uint32_t i = tid; i < 2 * ((npos * dim * 4 + 127) / 128); i += kWarps * 32) {
                    const uint32_t half_n = (npos * dim * 4 + 127) / 128, line = i % half_n;
                    const float* base = (i < half_n ? kc : vc) + next + (size_t)j0 * dim;
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint8_t*>(base) + (size_t)line * 128));
                }
            }
            for (uint32_t i = tid; i < npos * dim / 4; i += kWarps * 32) {
                const uint32_t jj = i / (dim / 4), d4 = i % (dim / 4), j = j0 + jj;
                const float4 kv = j == pos ? reinterpret_cast<const float4*>(knew)[d4] : reinterpret_cast<const float4*>(kc + (size_t)j * dim)[d4];
                const float4 vv = j == pos ? reinterpret_cast<const float4*>(vnew)[d4] : reinterpret_cast<const float4*>(vc + (size_t)j * dim)[d4];
                float* kd = ks + jj * pitch + 4 * d4;
                float* vd = vs + jj * pitch + 4 * d4;
                kd[0] = kv.x, kd[1] = kv.y, kd[2] = kv.z, kd[3] = kv.w;
                vd[0] = vv.x, vd[1] = vv.y, vd[2] = vv.z, vd[3] = vv.w;
            }
            csync();
            // a warp per query head: lane j scores position j0 + j (chunk <= 32), lane d owns output components d, d + 32, ...
            for (uint32_t hh = warp; hh < rep; hh += kWarps) {
                const float* qv = qrot + hh * dim;
                const uint32_t per = dim / 32;
                float sc = __uint_as_float(0xff800000u);
                if (lane < npos) {
                    float dot = 0.0f;
                    const float* kr = ks + lane * pitch;
                    for (uint32_t d = 0; d < dim; ++d) dot = __fmaf_rn(qv[d], kr[d], dot);
                    sc = __fmul_rn(dot, a.attn_scale);
                }
                float m = sc;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                const float pj = lane < npos ? exp_cephes(sc - m) : 0.0f;
                float lsum = pj;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                for (uint32_t jj = 0; jj < npos; ++jj) {
                    const float pw = __shfl_sync(0xffffffffu, pj, jj);
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i)
                        if (i < per) acc[i] = __fmaf_rn(pw, vs[jj * pitch + i * 32 + lane], acc[i]);
                }
                float* part = a.attn_part + ((size_t)(kvh * rep + hh) * kSplits + split) * (dim + 2);
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i)
                    if (i < per) __stcg(part + i * 32 + lane, acc[i]);
                if (lane == 0) __stcg(part + dim, m), __stcg(part + dim + 1, lsum);
            }
            __threadfence();
            csync();
            if (tid == 0) {
                const uint32_t old = atomicAdd(a.sync + 4 + kvh, 1u);
                sh.last = old == kSplits - 1;
                if (sh.last) a.sync[4 + kvh] = 0;
            }
            csync();
            if (sh.last) {  // this CTA merges the kv head's splits: a warp per head
                __threadfence();
                const uint32_t per = dim / 32;
                for (uint32_t hh = warp; hh < rep; hh += kWarps) {
                    const float* base = a.attn_part + (size_t)(kvh * rep + hh) * kSplits * (dim + 2);
                    // lane = split for the weights (kSplits == 32) ...
                    const float ms = __ldcg(base + lane * (dim + 2) + dim), ls = __ldcg(base + lane * (dim + 2) + dim + 1);
                    float M = ms;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
                    const float wgt = ls == 0.0f ? 0.0f : exp_cephes(ms - M);  // an empty split weighs nothing
                    float Lsum = __fmul_rn(ls, wgt);
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) Lsum += __shfl_xor_sync(0xffffffffu, Lsum, o);
                    // ... lane = component for the sums: all 32 splits' values are requested before the first is used
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        if (i >= per) break;
                        float vals[kSplits];
#pragma unroll
                        for (uint32_t sp = 0; sp < kSplits; ++sp) vals[sp] = __ldcg(base + sp * (dim + 2) + i * 32 + lane);
                        float acc = 0.0f;
#pragma unroll
                        for (uint32_t sp = 0; sp < kSplits; ++sp) acc = __fmaf_rn(vals[sp], __shfl_sync(0xffffffffu, wgt, sp), acc);
                        a.attn[(size_t)(kvh * rep + hh) * dim + i * 32 + lane] = __fdiv_rn(acc, Lsum);
                    }
                }
            }
        }
        if (!(alive = grid_barrier())) break;
        // ── phase 3: o projection ──
        global_to_digits(a.attn, q_size);
        if (const uint8_t* base = take_slice(s)) gemv_rows(base, s, a.o);
        release_slice();
        if (!(alive = grid_barrier())) break;
        // ── phase 4: h += o, norm, gate | up, SwiGLU ──
        norm_to_digits(a.o, L.post_norm);
        if (const uint8_t* base = take_slice(s)) {
            const uint8_t* up = base + s.rows[0] * s.kbytes;
            const float* sc0 = reinterpret_cast<const float*>(up + s.rows[1] * s.kbytes) + (s.r0[0] - span_lo(s.r0[0]));
            const float* sc1 = reinterpret_cast<const float*>(up + s.rows[1] * s.kbytes + 4 * span_floats(s.r0[0], s.rows[0])) + (s.r0[1] - span_lo(s.r0[1]));
            for (uint32_t r = warp; r < s.rows[0]; r += kWarps) {
                const float gd = row_dot(base + (size_t)r * s.kbytes, s.kbytes), ud = row_dot(up + (size_t)r * s.kbytes, s.kbytes);
                if (lane == 0) a.act[s.r0[0] + r] = silu_mul(__fmul_rn(gd, sc0[r]), __fmul_rn(ud, sc1[r]));
            }
        }
        release_slice();
        if (!(alive = grid_barrier())) break;
        // ── phase 5: down projection ──
        global_to_digits(a.act, a.inter);
        if (const uint8_t* base = take_slice(s)) gemv_rows(base, s, a.delta);
        release_slice();
        if (!(alive = grid_barrier())) break;
    }
    if (alive) {
        // ── final norm, the head, the arg-max ──
        norm_to_digits(a.delta, a.final_norm);
        unsigned long long best = 0ull;
        const uint32_t hs = head_slices(a, c, g);
        for (uint32_t j = 0; j < hs; ++j) {
            if (const uint8_t* base = take_slice(s)) {
                const float* sc = reinterpret_cast<const float*>(base + s.rows[0] * s.kbytes) + (s.r0[0] - span_lo(s.r0[0]));
                for (uint32_t r = warp; r < s.rows[0]; r += kWarps) {
                    const float y = __fmul_rn(row_dot(base + (size_t)r * s.kbytes, s.kbytes), sc[r]);
                    if (lane == 0) {
                        a.logits[s.r0[0] + r] = y;
                        const unsigned long long key = ((unsigned long long)(y == y ? fkey(y) : 0u) << 32) | (0xFFFFFFFFu - (s.r0[0] + r));
                        best = key > best ? key : best;
                    }
                }
            }
            release_slice();
        }
        if (lane == 0) reinterpret_cast<unsigned long long*>(sh.red_d)[warp] = best;
        csync();
        if (tid == 0) {
            for (int w = 1; w < kWarps; ++w) {
                const unsigned long long o = reinterpret_cast<unsigned long long*>(sh.red_d)[w];
                best = o > best ? o : best;
            }
            atomicMax(a.best, best);
        }
        alive = grid_barrier();
        if (alive && c == 0) {
            if (tid == 0) {
                *a.next_token = (int32_t)(0xFFFFFFFFu - (uint32_t)(*reinterpret_cast<volatile unsigned long long*>(a.best)));
                *a.best = 0ull;
            }
            for (uint32_t i = tid; i < a.nlayers; i += kWarps * 32) a.lens[i] = min(a.lens[i] + 1, a.max_len);  // g2-kv-advance
        }
    }
    // the last CTA out leaves the counters at zero for the next launch
    csync();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(a.sync + 1, 1u) == g - 1) a.sync[0] = 0, a.sync[1] = 0, a.sync[2] = 0;
    }
}

}  // namespace

struct DecodePlanDevice {
    StepArgs args;
    size_t smem;
    uint32_t grid;
};

}  // namespace gq

using namespace gq;

struct gq_decode_plan {
    DecodePlanDevice d;
    void* layers_dev = nullptr;  // LayerPtrs[nlayers]
    void* work = nullptr;        // activations, partial attention, counters
    std::vector<gq_buf> held;    // every buffer the plan names (retained while the plan lives)
};

extern "C" {

int32_t gq_decode_plan_create(gq_ctx* ctx, const gq_decode_desc* desc, gq_decode_plan** out) {
    return guarded([&] {
        Locked l(ctx);
        if (!desc || !out) fail("gq_decode_plan_create: null argument");
        *out = nullptr;
        const uint64_t H = desc->hidden, Hq = desc->heads, Hkv = desc->kv_heads, D = desc->dim, I = desc->inter, V = desc->vocab, L = desc->layers, ML = desc->max_len;
        check_dims("gq_decode_plan_create", H, I, V);
        if (!L || !H || !Hq || !Hkv || !I || !V || !ML) fail("gq_decode_plan_create: a dimension is zero");
        if (Hq % Hkv) fail("gq_decode_plan_create: %llu heads do not group over %llu kv heads", (unsigned long long)Hq, (unsigned long long)Hkv);
        if (D != 32 && D != 64 && D != 128) fail("gq_decode_plan_create: head_dim must be 32, 64 or 128, got %llu", (unsigned long long)D);
        const uint64_t qs = Hq * D, kvs = Hkv * D;
        if (H % 16 || I % 16 || qs % 16 || H > 4096 || I > 8192 || qs > 8192)
            fail("gq_decode_plan_create: hidden, q_size and intermediate sizes must be multiples of 16, hidden <= 4096, the others <= 8192 "
                 "(hidden %llu, q_size %llu, intermediate %llu): use the operator-by-operator step", (unsigned long long)H, (unsigned long long)qs, (unsigned long long)I);
        if (V % 4) fail("gq_decode_plan_create: the vocabulary size must be a multiple of 4 (scales travel in 16-byte pieces), got %llu", (unsigned long long)V);
        const int sms = ctx->prop.multiProcessorCount;
        if (Hkv * kSplits > (uint64_t)sms) fail("gq_decode_plan_create: %llu kv heads need more CTAs than the device has SMs", (unsigned long long)Hkv);
        if (!desc->layer) fail("gq_decode_plan_create: null layer table");
        {
            const uint64_t chunk = (ML + kSplits - 1) / kSplits, kmax_ = H > I ? H : I;
            if (chunk > 32 || 2 * chunk * (D + 1) * 4 > kmax_ * 4)
                fail("gq_decode_plan_create: a cache of %llu positions is beyond this kernel (at most %u, and 1/32 of it times head_dim must fit "
                     "the digit area): use the operator-by-operator step", (unsigned long long)ML, 32 * kSplits);
        }
        auto plan = std::unique_ptr<gq_decode_plan>(new gq_decode_plan());
        auto hold = [&](gq_buf h) {
            if (h) lookup(ctx, h, "gq_decode_plan_create").refs++, plan->held.push_back(h);
        };
        auto ptr = [&](gq_buf h, uint64_t count, uint64_t elem, const char* what) -> void* {
            void* p = view(ctx, h, 0, count, elem, what);
            if (reinterpret_cast<uintptr_t>(p) & 15) fail("gq_decode_plan_create: %s must be 16-byte aligned", what);
            hold(h);
            return p;
        };
        std::vector<LayerPtrs> lp(L);
        try {
            for (uint64_t i = 0; i < L; ++i) {
                const gq_decode_layer& s = desc->layer[i];
                lp[i].in_norm = (const float*)ptr(s.input_norm, H, 4, "input norm weight");
                lp[i].qkv_q = (const uint8_t*)ptr(s.qkv_q, (qs + 2 * kvs) * H, 1, "q|k|v codes");
                lp[i].qkv_scale = (const float*)ptr(s.qkv_scale, qs + 2 * kvs, 4, "q|k|v scales");
                lp[i].qkv_bias = s.qkv_bias ? (const float*)ptr(s.qkv_bias, qs + 2 * kvs, 4, "q|k|v bias") : nullptr;
                lp[i].o_q = (const uint8_t*)ptr(s.o_q, H * qs, 1, "o codes");
                lp[i].o_scale = (const float*)ptr(s.o_scale, H, 4, "o scales");
                lp[i].post_norm = (const float*)ptr(s.post_norm, H, 4, "post-attention norm weight");
                lp[i].gu_q = (const uint8_t*)ptr(s.gate_up_q, 2 * I * H, 1, "gate|up codes");
                lp[i].gu_scale = (const float*)ptr(s.gate_up_scale, 2 * I, 4, "gate|up scales");
                lp[i].down_q = (const uint8_t*)ptr(s.down_q, H * I, 1, "down codes");
                lp[i].down_scale = (const float*)ptr(s.down_scale, H, 4, "down scales");
            }
            StepArgs& a = plan->d.args;
            a.embed = (const float*)ptr(desc->embed, V * H, 4, "embedding table");
            a.final_norm = (const float*)ptr(desc->final_norm, H, 4, "final norm weight");
            a.head_q = (const uint8_t*)ptr(desc->head_q, V * H, 1, "head codes");
            a.head_scale = (const float*)ptr(desc->head_scale, V, 4, "head scales");
            a.cosv = (const float*)ptr(desc->cos, ML * D, 4, "cos table");
            a.sinv = (const float*)ptr(desc->sin, ML * D, 4, "sin table");
            a.kcache = (float*)ptr(desc->kcache, L * Hkv * ML * D, 4, "key cache");
            a.vcache = (float*)ptr(desc->vcache, L * Hkv * ML * D, 4, "value cache");
            a.lens = (uint32_t*)ptr(desc->lens, L, 4, "cursor");
            // work area: qkv | attn | o | act | delta | partial attention | counters | arg-max key
            auto up16 = [](uint64_t v) { return (v + 15) / 16 * 16; };
            const uint64_t f_qkv = up16(qs + 2 * kvs), f_attn = up16(qs), f_h = up16(H), f_act = up16(I), f_part = up16(Hq * kSplits * (D + 2));
            const uint64_t floats = f_qkv + f_attn + 2 * f_h + f_act + f_part;
            const uint64_t bytes = floats * 4 + 256 + 64;
            GQ_CUDA(cudaMalloc(&plan->work, bytes));
            GQ_CUDA(cudaMemsetAsync(plan->work, 0, bytes, ctx->stream));
            ctx->stats.buffer_allocations++;
            float* w = (float*)plan->work;
            a.qkv = w, w += f_qkv, a.attn = w, w += f_attn, a.o = w, w += f_h, a.delta = w, w += f_h, a.act = w, w += f_act, a.attn_part = w, w += f_part;
            a.sync = (uint32_t*)w;
            a.best = (unsigned long long*)((uint8_t*)w + 256);
            GQ_CUDA(cudaMalloc(&plan->layers_dev, L * sizeof(LayerPtrs)));
            GQ_CUDA(cudaMemcpyAsync(plan->layers_dev, lp.data(), L * sizeof(LayerPtrs), cudaMemcpyHostToDevice, ctx->stream));
            GQ_CUDA(cudaStreamSynchronize(ctx->stream));  // lp goes out of scope
            a.layers = (const LayerPtrs*)plan->layers_dev;
            a.status = ctx->status_dev;
            a.hidden = (uint32_t)H, a.heads = (uint32_t)Hq, a.kv_heads = (uint32_t)Hkv, a.dim = (uint32_t)D, a.inter = (uint32_t)I, a.vocab = (uint32_t)V;
            a.nlayers = (uint32_t)L, a.max_len = (uint32_t)ML, a.eps = desc->eps, a.attn_scale = desc->attn_scale;
            const uint64_t kmax = H > I ? H : I, rep = Hq / Hkv;
            plan->d.smem = 512 + ((H * 4 + 127) & ~127ull) + ((kmax * 4 + 127) & ~127ull) + (((rep + 2) * D * 4 + 127) & ~127ull) + kRingBytes + 128;
            if (plan->d.smem > (size_t)ctx->prop.sharedMemPerBlockOptin) fail("gq_decode_plan_create: the step needs %zu bytes of shared memory per CTA", plan->d.smem);
            // The ring is walked the same way by the producer and the consumers (ring_place); a slice may be overwritten once
            // the slice three before it has been released, so no slice may overlap the two placed before it. Checked here for
            // every CTA's sequence of shares.
            {
                auto lo = [&](uint64_t n, uint64_t c) { return n * c / (uint64_t)sms; };
                auto span = [](uint64_t r0, uint64_t rows) { return ((r0 + rows + 3) & ~3ull) - (r0 & ~3ull); };
                auto bytes_of = [&](uint64_t r0, uint64_t rows, uint64_t kb, bool two, uint64_t r0b, bool bias) {
                    uint64_t b = (two ? 2 : 1) * rows * kb + 4 * span(r0, rows) + (two ? 4 * span(r0b, rows) : 0) + (bias ? 4 * span(r0, rows) : 0);
                    return (b + 127) & ~127ull;
                };
                for (uint64_t c = 0; c < (uint64_t)sms; ++c) {
                    std::vector<uint64_t> sizes;
                    const uint64_t nq = qs + 2 * kvs;
                    const uint64_t per_layer[4] = {
                        bytes_of(lo(nq, c), lo(nq, c + 1) - lo(nq, c), H, false, 0, desc->layer[0].qkv_bias != 0),
                        bytes_of(lo(H, c), lo(H, c + 1) - lo(H, c), qs, false, 0, false),
                        bytes_of(lo(I, c), lo(I, c + 1) - lo(I, c), H, true, I + lo(I, c), false),
                        bytes_of(lo(H, c), lo(H, c + 1) - lo(H, c), I, false, 0, false)};
                    const bool has[4] = {lo(nq, c + 1) > lo(nq, c), lo(H, c + 1) > lo(H, c), lo(I, c + 1) > lo(I, c), lo(H, c + 1) > lo(H, c)};
                    for (int rep2 = 0; rep2 < 2; ++rep2)
                        for (int i = 0; i < 4; ++i)
                            if (has[i]) sizes.push_back(per_layer[i]);
                    const uint64_t v0 = lo(V, c), v1 = lo(V, c + 1);
                    for (uint64_t r = v0; r < v1; r += kHeadRows) sizes.push_back(bytes_of(r, std::min<uint64_t>(kHeadRows, v1 - r), H, false, 0, false));
                    uint64_t off = 0, prev[2][2] = {{0, 0}, {0, 0}};
                    for (uint64_t b : sizes) {
                        if (b > kRingBytes) fail("gq_decode_plan_create: a CTA's share of a layer (%llu bytes) does not fit the weight ring", (unsigned long long)b);
                        if (off + b > kRingBytes) off = 0;
                        for (auto& p : prev)
                            if (p[1] > p[0] && off < p[1] && p[0] < off + b)
                                fail("gq_decode_plan_create: the weight ring (%u bytes) cannot hold three consecutive shares of this model", kRingBytes);
                        prev[0][0] = prev[1][0], prev[0][1] = prev[1][1], prev[1][0] = off, prev[1][1] = off + b;
                        off += b;
                    }
                }
            }
            GQ_CUDA(cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan->d.smem));
            int per_sm = 0;
            GQ_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel, kThreads, plan->d.smem));
            if (per_sm < 1) fail("gq_decode_plan_create: the step kernel does not fit an SM");
            plan->d.grid = (uint32_t)sms;  // one CTA per SM, all resident: the barriers need that (cooperative launch)
        } catch (...) {
            for (gq_buf h : plan->held) drop_ref(ctx, h);
            if (plan->work) cudaFree(plan->work);
            if (plan->layers_dev) cudaFree(plan->layers_dev);
            throw;
        }
        *out = plan.release();
    });
}

int32_t gq_decode_plan_step(gq_ctx* ctx, gq_decode_plan* plan, gq_buf token, gq_buf logits, gq_buf next_token) {
    return guarded([&] {
        Locked l(ctx);
        if (!plan) fail("gq_decode_plan_step: null plan");
        StepArgs a = plan->d.args;
        a.token = (const int32_t*)view(ctx, token, 0, 1, 4, "gq_decode_plan_step token");
        a.logits = (float*)view(ctx, logits, 0, a.vocab, 4, "gq_decode_plan_step logits");
        a.next_token = (int32_t*)view(ctx, next_token, 0, 1, 4, "gq_decode_plan_step next token");
        a.wait_cycles = ctx->peer_wait_cycles;
        void* params[] = {&a};
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(plan->d.grid), cfg.blockDim = dim3(kThreads), cfg.dynamicSmemBytes = plan->d.smem, cfg.stream = ctx->stream;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeCooperative;
        attr.val.cooperative = 1;
        cfg.attrs = &attr, cfg.numAttrs = 1;
        GQ_CUDA(cudaLaunchKernelExC(&cfg, (const void*)decode_step_kernel, params));
        after_launch(ctx, "decode_step", {token, logits, next_token}, {});
    });
}

void gq_decode_plan_destroy(gq_ctx* ctx, gq_decode_plan* plan) {
    if (!ctx || !plan) return;
    guarded([&] {
        Locked l(ctx);
        cudaStreamSynchronize(ctx->stream);
        if (plan->work) cudaFree(plan->work);
        if (plan->layers_dev) cudaFree(plan->layers_dev);
        for (gq_buf h : plan->held) drop_ref(ctx, h);
        delete plan;
    });
}

}  // extern "C"
