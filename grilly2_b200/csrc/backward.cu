// The frozen-weight backward of the quantized linear: grad_x = grad . dequantize(W)
// and grad_bias = column sums of grad. Replaces LinearInt8Backward / LinearInt4Backward
// (crates/grilly-infer/src/quant.rs:326-349, quant4.rs:447-480), which write the
// whole dequantized weight (4 N K bytes) to memory and then run the generic float32
// matrix product over it; here a CTA dequantizes the 16 x 64 piece of W it is about to
// use into shared memory, with the dequantizer's own float32 expressions
// (q * scale; level * scale + (zero - 8 scale)), so the float32 weight never exists
// in HBM. Products are accumulated in float32 in increasing order of the output
// feature, which keeps the reference's bound for this operator,
// (N + 2) 2^-24 sum|grad w| against float64 (crates/grilly-infer/tests/quant.rs:14-17).
// Training-time path, off the decode step: FP32 pipes (a tensor-core tf32 product
// would not hold that bound).
// Algorithmic bytes: grad (M N 4) + packed W + its scales (+ zeros) + grad_x (M K 4).
#include "gq_internal.h"

namespace gq {

namespace {

constexpr uint32_t kTile = 64;   // outputs per CTA: 64 rows of grad x 64 columns of K
constexpr uint32_t kChunk = 16;  // output features per step

template <bool Q4>
__global__ void __launch_bounds__(256) linear_backward_kernel(const float* __restrict__ g, uint32_t m, const uint32_t* __restrict__ q,
                                                             const float* __restrict__ scale, const float* __restrict__ zero, uint32_t n, uint32_t k,
                                                             uint32_t words, uint32_t group, uint32_t groups, float* __restrict__ gx) {
    __shared__ float sg[kChunk][kTile + 4], sw[kChunk][kTile + 4];
    const uint32_t tx = threadIdx.x & 15u, ty = threadIdx.x >> 4;
    const uint32_t m0 = blockIdx.y * kTile, k0 = blockIdx.x * kTile;
    float acc[4][4] = {};
    for (uint32_t n0 = 0; n0 < n; n0 += kChunk) {
        // grad[m0 .. +63][n0 .. +15], stored [feature][row]
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const uint32_t idx = threadIdx.x + 256 * i, mm = idx >> 4, nn = idx & 15u;
            sg[nn][mm] = (m0 + mm < m && n0 + nn < n) ? g[(size_t)(m0 + mm) * n + n0 + nn] : 0.0f;
        }
        // W[n0 .. +15][k0 .. +63], dequantized as the dequantize kernels do
        if (!Q4) {
            const uint32_t nn = threadIdx.x >> 4, w = threadIdx.x & 15u, row = n0 + nn;  // a word = 4 codes
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (row < n && k0 + 4 * w < k) {
                const uint32_t packed = q[(size_t)row * words + (k0 >> 2) + w];
                const float s = scale[row];
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) v[j] = k0 + 4 * w + j < k ? __fmul_rn((float)(int)(int8_t)(packed >> (8 * j)), s) : 0.0f;
            }
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) sw[nn][4 * w + j] = v[j];
        } else if (threadIdx.x < 128) {
            const uint32_t nn = threadIdx.x >> 3, w = threadIdx.x & 7u, row = n0 + nn;  // a word = 8 levels
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (row < n && k0 + 8 * w < k) {
                const uint32_t packed = q[(size_t)row * words + (k0 >> 3) + w];
                const uint32_t gi = (k0 + 8 * w) / group;  // a group is a multiple of 32 columns: one per word
                const float s = scale[(size_t)row * groups + gi];
                const float lo = __fsub_rn(zero[(size_t)row * groups + gi], __fmul_rn(8.0f, s));
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j) v[j] = k0 + 8 * w + j < k ? __fmaf_rn((float)((packed >> (4 * j)) & 0xFu), s, lo) : 0.0f;
            }
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j) sw[nn][8 * w + j] = v[j];
        }
        __syncthreads();
#pragma unroll
        for (uint32_t nn = 0; nn < kChunk; ++nn) {
            const float4 a = *reinterpret_cast<const float4*>(&sg[nn][4 * ty]);
            const float4 b = *reinterpret_cast<const float4*>(&sw[nn][4 * tx]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i)
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i)
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            const uint32_t r = m0 + 4 * ty + i, c = k0 + 4 * tx + j;
            if (r < m && c < k) gx[(size_t)r * k + c] = acc[i][j];
        }
}

// grad_bias[c] = sum over the rows of grad[.][c], in row order: 32 columns x 8 row lanes per CTA
__global__ void __launch_bounds__(256) column_sum_kernel(const float* __restrict__ g, uint32_t m, uint32_t n, float* __restrict__ out) {
    __shared__ float part[8][33];
    const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5, c = blockIdx.x * 32 + tx;
    float acc = 0.0f;
    if (c < n)
        for (uint32_t r = ty; r < m; r += 8) acc = __fadd_rn(acc, g[(size_t)r * n + c]);
    part[ty][tx] = acc;
    __syncthreads();
    if (ty == 0 && c < n) {
        float tot = part[0][tx];
#pragma unroll
        for (uint32_t i = 1; i < 8; ++i) tot = __fadd_rn(tot, part[i][tx]);
        out[c] = tot;
    }
}

}  // namespace

void launch_linear_backward_q8(cudaStream_t s, const float* g, uint64_t m, const uint32_t* q, const float* scale, uint64_t n, uint64_t k, float* gx) {
    const uint32_t words = (uint32_t)((k + 15) / 16 * 4);
    linear_backward_kernel<false><<<dim3((uint32_t)((k + kTile - 1) / kTile), (uint32_t)((m + kTile - 1) / kTile)), 256, 0, s>>>(
        g, (uint32_t)m, q, scale, nullptr, (uint32_t)n, (uint32_t)k, words, 0u, 0u, gx);
}

void launch_linear_backward_q4(cudaStream_t s, const float* g, uint64_t m, const uint32_t* q, const float* scale, const float* zero, uint64_t n,
                               uint64_t k, uint64_t group, float* gx) {
    const uint32_t words = (uint32_t)((k + 31) / 32 * 4), groups = (uint32_t)((k + group - 1) / group);
    linear_backward_kernel<true><<<dim3((uint32_t)((k + kTile - 1) / kTile), (uint32_t)((m + kTile - 1) / kTile)), 256, 0, s>>>(
        g, (uint32_t)m, q, scale, zero, (uint32_t)n, (uint32_t)k, words, (uint32_t)group, groups, gx);
}

void launch_column_sum(cudaStream_t s, const float* g, uint64_t m, uint64_t n, float* out) {
    column_sum_kernel<<<(uint32_t)((n + 31) / 32), 256, 0, s>>>(g, (uint32_t)m, (uint32_t)n, out);
}

}  // namespace gq
