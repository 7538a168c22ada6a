// Dequant-fused GEMV for decode (few rows of x): y = x @ dequant(W)^T + bias
// with W int8 per-row or int4 group-wise, read once from HBM in its packed
// form. Replaces the reference's GLSL decode kernels
//   crates/grilly-core/shaders/g2-linear-q8.glsl:33-95
//   crates/grilly-core/shaders/g2-linear-q4.glsl:43-111
// and reproduces their float32 summation ORDER, so the result equals the CPU
// restatement of those shaders bit for bit, not merely within a tolerance:
//
//   reference: 64 lanes per output feature; lane l chains the FMAs of the
//   16-byte vectors l, l+64, l+128, … in order; then the fixed tree
//   partial[t] += partial[t + s], s = 32, 16, …, 1.
//
//   here: one 32-thread warp per output feature. Thread t plays lanes t and
//   t+32: it reads vectors t, t+32, t+64, … (so a warp's loads are 512
//   contiguous bytes), feeding them alternately to two accumulators. The
//   tree's first step (s = 32) is then the sum of a thread's own two
//   accumulators, and steps 16 … 1 are shuffles.
//
// A warp owns C output features at a time so that one register copy of an x
// vector serves C weight vectors: without that, re-reading x from L1 would
// cost more than reading the weights from HBM (an int4 vector is 16 bytes of
// weights against 128 bytes of x). The kernel is bounded by HBM bandwidth for
// a single row of x; by the FP32 pipes as rows are added (each weight costs
// one FMA per row, and 16 rows of int4 would need five times the FP32 peak
// to keep up with HBM), which is what the tensor-core decode path is for.
//
// Algorithmic bytes per call: packed weights + scales (+ zero points) + x + y
// (+ bias), each counted once.
#include "gq_internal.h"

namespace gq {

// 16-byte streaming load: weights are read exactly once, so they should not
// displace x (which every warp re-reads) from L1.
__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float warp_tree(float v) {
    // partial[t] += partial[t + s] for t < s, s = 16 … 1; lane 0 ends with the tree's root
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, s));
    return v;
}

// x[k0 .. k0 + N) of one row into registers, zero beyond `count`. FMAs against
// the zeros leave an accumulator unchanged, so padded tails need no branches
// in the arithmetic.
template <int N, bool XVEC>
__device__ __forceinline__ void load_x(const float* __restrict__ xr, uint32_t k0, uint32_t count, float (&xv)[N]) {
    if (XVEC) {
#pragma unroll
        for (int j = 0; j < N / 4; ++j) {
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            if (4u * j < count) t = __ldg(reinterpret_cast<const float4*>(xr + k0) + j);
            xv[4 * j] = t.x, xv[4 * j + 1] = t.y, xv[4 * j + 2] = t.z, xv[4 * j + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < N; ++j) xv[j] = (uint32_t)j < count ? __ldg(xr + k0 + j) : 0.0f;
    }
}

static constexpr int kWarps = 8;  // warps per CTA

// ── int8 ────────────────────────────────────────────────────────────────
template <int MR, int C, bool XVEC>
__global__ void __launch_bounds__(kWarps * 32) gemv_q8_kernel(const float* __restrict__ x, const uint4* __restrict__ q,
                                                               const float* __restrict__ scale, const float* __restrict__ bias,
                                                               float* __restrict__ y, uint32_t m, uint32_t k, uint32_t n,
                                                               uint32_t vecs) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t col0 = (blockIdx.x * kWarps + warp) * C;
    const uint32_t row0 = blockIdx.y * MR;
    if (col0 >= n) return;

    float acc[C][MR][2];
#pragma unroll
    for (int c = 0; c < C; ++c)
#pragma unroll
        for (int r = 0; r < MR; ++r) acc[c][r][0] = acc[c][r][1] = 0.0f;

    for (uint32_t v0 = lane; v0 < vecs; v0 += 64) {
        uint4 wq[2][C];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const uint32_t v = v0 + 32 * h, col = col0 + c;
                wq[h][c] = (v < vecs && col < n) ? ldg_stream(q + (size_t)col * vecs + v) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t v = v0 + 32 * h;
            if (v >= vecs) continue;
            const uint32_t k0 = v * 16, count = min(16u, k - k0);
#pragma unroll
            for (int r = 0; r < MR; ++r) {
                if (row0 + r >= m) continue;
                float xv[16];
                load_x<16, XVEC>(x + (size_t)(row0 + r) * k, k0, count, xv);
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    const uint32_t w[4] = {wq[h][c].x, wq[h][c].y, wq[h][c].z, wq[h][c].w};
                    float a = acc[c][r][h];
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        a = __fmaf_rn(xv[j], (float)(int)(int8_t)(w[j >> 2] >> (8 * (j & 3))), a);
                    acc[c][r][h] = a;
                }
            }
        }
    }

#pragma unroll
    for (int c = 0; c < C; ++c) {
        const uint32_t col = col0 + c;
#pragma unroll
        for (int r = 0; r < MR; ++r) {
            float p = warp_tree(__fadd_rn(acc[c][r][0], acc[c][r][1]));
            if (lane == 0 && col < n && row0 + r < m) {
                float out = __fmul_rn(p, scale[col]);  // the scale multiplies the finished dot product
                if (bias) out = __fadd_rn(out, bias[col]);
                y[(size_t)(row0 + r) * n + col] = out;
            }
        }
    }
}

// ── int4 ────────────────────────────────────────────────────────────────
// Per vector (32 levels, one group): dot = sum level * x (an FMA chain from
// 0), sum = sum x — four at a time as (x0+x1)+(x2+x3) when XVEC, one at a
// time otherwise, the reference's two paths — then
// acc = fma(s, dot, acc); acc = fma(zero - 8 s, sum, acc).
template <int MR, int C, bool XVEC>
__global__ void __launch_bounds__(kWarps * 32) gemv_q4_kernel(const float* __restrict__ x, const uint4* __restrict__ q,
                                                               const float* __restrict__ scale, const float* __restrict__ zero,
                                                               const float* __restrict__ bias, float* __restrict__ y, uint32_t m,
                                                               uint32_t k, uint32_t n, uint32_t vecs, uint32_t group,
                                                               uint32_t groups) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t col0 = (blockIdx.x * kWarps + warp) * C;
    const uint32_t row0 = blockIdx.y * MR;
    if (col0 >= n) return;

    float acc[C][MR][2];
#pragma unroll
    for (int c = 0; c < C; ++c)
#pragma unroll
        for (int r = 0; r < MR; ++r) acc[c][r][0] = acc[c][r][1] = 0.0f;

    for (uint32_t v0 = lane; v0 < vecs; v0 += 64) {
        uint4 wq[2][C];
        float sc[2][C], lo[2][C];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const uint32_t v = v0 + 32 * h, col = col0 + c;
                const bool ok = v < vecs && col < n;
                wq[h][c] = ok ? ldg_stream(q + (size_t)col * vecs + v) : make_uint4(0, 0, 0, 0);
                const size_t gi = (size_t)col * groups + (v * 32) / group;
                sc[h][c] = ok ? __ldg(scale + gi) : 0.0f;
                lo[h][c] = ok ? __ldg(zero + gi) : 0.0f;
            }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t v = v0 + 32 * h;
            if (v >= vecs) continue;
            const uint32_t k0 = v * 32, count = min(32u, k - k0);
#pragma unroll
            for (int c = 0; c < C; ++c) lo[h][c] = __fsub_rn(lo[h][c], __fmul_rn(8.0f, sc[h][c]));
#pragma unroll
            for (int r = 0; r < MR; ++r) {
                if (row0 + r >= m) continue;
                float xv[32];
                load_x<32, XVEC>(x + (size_t)(row0 + r) * k, k0, count, xv);
                float sum = 0.0f;
                if (XVEC) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        sum = __fadd_rn(sum, __fadd_rn(__fadd_rn(xv[4 * j], xv[4 * j + 1]), __fadd_rn(xv[4 * j + 2], xv[4 * j + 3])));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) sum = __fadd_rn(sum, xv[j]);
                }
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    const uint32_t w[4] = {wq[h][c].x, wq[h][c].y, wq[h][c].z, wq[h][c].w};
                    float dot = 0.0f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        // even levels of the word in the bytes of `e`, odd ones in `o`
                        const uint32_t e = w[i] & 0x0F0F0F0Fu, o = (w[i] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                        for (int b = 0; b < 4; ++b) {
                            dot = __fmaf_rn((float)((e >> (8 * b)) & 0xFFu), xv[8 * i + 2 * b], dot);
                            dot = __fmaf_rn((float)((o >> (8 * b)) & 0xFFu), xv[8 * i + 2 * b + 1], dot);
                        }
                    }
                    float a = __fmaf_rn(sc[h][c], dot, acc[c][r][h]);
                    acc[c][r][h] = __fmaf_rn(lo[h][c], sum, a);
                }
            }
        }
    }

#pragma unroll
    for (int c = 0; c < C; ++c) {
        const uint32_t col = col0 + c;
#pragma unroll
        for (int r = 0; r < MR; ++r) {
            float p = warp_tree(__fadd_rn(acc[c][r][0], acc[c][r][1]));
            if (lane == 0 && col < n && row0 + r < m) {
                if (bias) p = __fadd_rn(p, bias[col]);
                y[(size_t)(row0 + r) * n + col] = p;
            }
        }
    }
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int MR, int C>
static void run_q8(cudaStream_t s, bool xvec, const float* x, uint32_t m, uint32_t k, const uint32_t* q, const float* scale,
                   const float* bias, uint32_t n, float* y) {
    const uint32_t vecs = (k + 15) / 16;
    dim3 grid(((n + C - 1) / C + kWarps - 1) / kWarps, (m + MR - 1) / MR);
    auto qp = reinterpret_cast<const uint4*>(q);
    if (xvec)
        gemv_q8_kernel<MR, C, true><<<grid, kWarps * 32, 0, s>>>(x, qp, scale, bias, y, m, k, n, vecs);
    else
        gemv_q8_kernel<MR, C, false><<<grid, kWarps * 32, 0, s>>>(x, qp, scale, bias, y, m, k, n, vecs);
}

template <int MR, int C>
static void run_q4(cudaStream_t s, bool xvec, const float* x, uint32_t m, uint32_t k, const uint32_t* q, const float* scale,
                   const float* zero, const float* bias, uint32_t n, uint32_t group, float* y) {
    const uint32_t vecs = (k + 31) / 32, groups = (k + group - 1) / group;
    dim3 grid(((n + C - 1) / C + kWarps - 1) / kWarps, (m + MR - 1) / MR);
    auto qp = reinterpret_cast<const uint4*>(q);
    if (xvec)
        gemv_q4_kernel<MR, C, true><<<grid, kWarps * 32, 0, s>>>(x, qp, scale, zero, bias, y, m, k, n, vecs, group, groups);
    else
        gemv_q4_kernel<MR, C, false><<<grid, kWarps * 32, 0, s>>>(x, qp, scale, zero, bias, y, m, k, n, vecs, group, groups);
}

// The reference's own rule for its vec4 path (crates/grilly-infer/src/quant.rs:279):
// x starts on a multiple of four elements and k is a multiple of four. For
// int4 it also selects the order `sum` is taken in, so it is part of the
// result, not only of the speed.
static inline bool x_vec4(const float* x, uint64_t k) { return aligned16(x) && k % 4 == 0; }

void launch_gemv_q8(cudaStream_t s, int /*sm_count*/, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                    const float* scale, const float* bias, uint64_t n, float* y) {
    const bool xv = x_vec4(x, k);
    const uint32_t M = (uint32_t)m, K = (uint32_t)k, N = (uint32_t)n;
    if (m == 1)
        run_q8<1, 4>(s, xv, x, M, K, q, scale, bias, N, y);
    else if (m == 2)
        run_q8<2, 4>(s, xv, x, M, K, q, scale, bias, N, y);
    else
        run_q8<4, 2>(s, xv, x, M, K, q, scale, bias, N, y);
}

void launch_gemv_q4(cudaStream_t s, int /*sm_count*/, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                    const float* scale, const float* zero, const float* bias, uint64_t n, uint64_t group, float* y) {
    const bool xv = x_vec4(x, k);
    const uint32_t M = (uint32_t)m, K = (uint32_t)k, N = (uint32_t)n, G = (uint32_t)group;
    if (m == 1)
        run_q4<1, 4>(s, xv, x, M, K, q, scale, zero, bias, N, G, y);
    else if (m == 2)
        run_q4<2, 2>(s, xv, x, M, K, q, scale, zero, bias, N, G, y);
    else
        run_q4<4, 2>(s, xv, x, M, K, q, scale, zero, bias, N, G, y);
}

}  // namespace gq
