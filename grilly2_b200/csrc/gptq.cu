// GPTQ on the device: the calibration Hessian H = 2 X^T X and the column loop
// that quantizes a weight to int4 while pushing each column's rounding error
// into the columns not yet quantized. Replaces the numpy of
// python/grilly/infer/gptq.py:87-181 (the loop; 263 s per model there, most of
// it this loop, docs/inference.md:357-359) and the capture of
// python/grilly/infer/calibration.py:97-123 (the Hessian). The inverse
// Cholesky factor U (U^T U = H^-1, damped) is a K x K float64 factorisation done
// once per layer on the host, as the reference does, and handed in as float32.
//
//   for each block of 128 columns [start, end):
//     block kernel, one warp per weight row, U[start:end, start:end] in shared memory:
//       at the first column of a group: scale = max((max - min) / 15, 2^-23), lo = min of the group AS IT STANDS
//       per column j: level = clamp(rint((w_j - lo) / scale), 0, 15); deq = level * scale + lo
//                     e = (w_j - deq) / U[j][j];  w[j+1 : end] -= e * U[j][j+1 : end]
//       the block's levels are packed (8 per word, low nibble first), e is kept
//     update kernel: w[:, end:] -= E[:, 0:128] . U[start:end, end:]   (a plain tiled fp32 GEMM)
//
// Rows of the weight are independent, so the block kernel is parallel over
// rows and sequential only along the 128 columns of a block. With a diagonal H
// (U diagonal) no error moves and the result is the round-to-nearest
// quantizer's, level for level (the reference's own test of this property:
// tests/python/test_gptq.py:39-47): the group parameters and the rounding use
// the same float32 formulas as quantize_q4_kernel.
// Bound: the update GEMM, n k^2 / 2 multiply-adds in fp32 on the CUDA cores.
#include "gq_internal.h"

namespace gq {

namespace {

constexpr uint32_t kBlock = 128;    // columns per block (and the update GEMM's K)
constexpr uint32_t kRowsPerCta = 8; // warps per CTA in the block kernel

// H += 2 X^T X for X [rows][k]: 32 x 32 output tiles, rows taken 32 at a time through shared memory.
__global__ void __launch_bounds__(1024) hessian_add_kernel(const float* __restrict__ x, uint32_t rows, uint32_t k, float* __restrict__ h) {
    __shared__ float sa[32][33], sb[32][33];
    const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const uint32_t i0 = blockIdx.y * 32, j0 = blockIdx.x * 32;
    if (j0 + 31 < i0) return;  // the lower triangle is mirrored from the upper below
    float acc = 0.0f;
    for (uint32_t r0 = 0; r0 < rows; r0 += 32) {
        const uint32_t r = r0 + ty;
        sa[ty][tx] = (r < rows && i0 + tx < k) ? x[(size_t)r * k + i0 + tx] : 0.0f;
        sb[ty][tx] = (r < rows && j0 + tx < k) ? x[(size_t)r * k + j0 + tx] : 0.0f;
        __syncthreads();
#pragma unroll
        for (uint32_t rr = 0; rr < 32; ++rr) acc = __fmaf_rn(sa[rr][ty], sb[rr][tx], acc);
        __syncthreads();
    }
    const uint32_t i = i0 + ty, j = j0 + tx;
    if (i < k && j < k && i <= j) {
        const float v = h[(size_t)i * k + j] + 2.0f * acc;
        h[(size_t)i * k + j] = v;
        if (i != j) h[(size_t)j * k + i] = v;
    }
}

// One block of columns for kRowsPerCta rows. w: the working weight [n][k] (modified in place); u: U [k][k];
// err: [n][kBlock] this block's errors out; q / scale / zero: the packed result.
__global__ void __launch_bounds__(kRowsPerCta * 32) gptq_block_kernel(float* __restrict__ w, const float* __restrict__ u, uint32_t n, uint32_t k,
                                                                     uint32_t start, uint32_t group, uint32_t groups, uint32_t words,
                                                                     float* __restrict__ err, uint32_t* __restrict__ q, float* __restrict__ scale,
                                                                     float* __restrict__ zero) {
    extern __shared__ float su[];  // U[start + a][start + b], a, b < kBlock
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t i = threadIdx.x; i < kBlock * kBlock; i += blockDim.x) {
        const uint32_t a = i / kBlock, b = i % kBlock;
        su[i] = (start + a < k && start + b < k) ? u[(size_t)(start + a) * k + start + b] : 0.0f;
    }
    __syncthreads();
    const uint32_t row = blockIdx.x * kRowsPerCta + warp;
    if (row >= n) return;
    const uint32_t width = min(kBlock, k - start);
    // lane l holds columns start + 4 l .. start + 4 l + 3 of the row
    float v[4];
    float* wr = w + (size_t)row * k + start;
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) v[i] = 4 * lane + i < width ? wr[4 * lane + i] : 0.0f;
    uint32_t lv[4] = {0u, 0u, 0u, 0u};
    float e_mine[4] = {0.f, 0.f, 0.f, 0.f};
    float s = 1.0f, lo = 0.0f;
    for (uint32_t j = 0; j < width; ++j) {
        if ((start + j) % group == 0) {
            // the group's parameters from the weights as they stand (quantize_q4_kernel's formulas)
            const uint32_t gend = min(j + group, width);
            float mn = __uint_as_float(0x7f800000u), mx = __uint_as_float(0xff800000u);
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) {
                const uint32_t c = 4 * lane + i;
                if (c >= j && c < gend) mn = fminf(mn, v[i]), mx = fmaxf(mx, v[i]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            }
            s = fmaxf(__fdiv_rn(__fsub_rn(mx, mn), 15.0f), 1.1920928955078125e-7f);
            lo = mn;
            if (lane == 0) {
                const uint32_t g = (start + j) / group;
                scale[(size_t)row * groups + g] = s;
                zero[(size_t)row * groups + g] = __fadd_rn(lo, __fmul_rn(8.0f, s));
            }
        }
        const uint32_t owner = j >> 2, slot = j & 3u;
        float wj = slot == 0 ? v[0] : slot == 1 ? v[1] : slot == 2 ? v[2] : v[3];
        wj = __shfl_sync(0xffffffffu, wj, owner);
        const float level = fminf(fmaxf(rintf(__fdiv_rn(__fsub_rn(wj, lo), s)), 0.0f), 15.0f);
        const float deq = __fadd_rn(__fmul_rn(level, s), lo);
        const float e = __fdiv_rn(__fsub_rn(wj, deq), su[j * kBlock + j]);
        if (lane == owner) {
            lv[slot] = (uint32_t)level;
            e_mine[slot] = e;
        }
        // push the error into the block's later columns
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const uint32_t c = 4 * lane + i;
            if (c > j && c < width) v[i] = __fsub_rn(v[i], __fmul_rn(e, su[j * kBlock + c]));
        }
    }
    // results: the errors (for the update of the columns after the block), the block's packed levels
    float* er = err + (size_t)row * kBlock;
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) er[4 * lane + i] = 4 * lane + i < width ? e_mine[i] : 0.0f;
    // word t of the block holds columns 8 t .. 8 t + 7: lanes 2 t (low four nibbles) and 2 t + 1 (high four)
    const uint32_t nib = lv[0] | (lv[1] << 4) | (lv[2] << 8) | (lv[3] << 12);
    const uint32_t other = __shfl_xor_sync(0xffffffffu, nib, 1);
    if (!(lane & 1u)) {
        const uint32_t t = lane >> 1;
        if (8 * t < width) q[(size_t)row * words + (start >> 3) + t] = nib | (other << 16);
    }
}

// w[:, end:] -= E . U[start:end, end:]: tiles of 64 rows x 64 columns, E's 128 columns through shared memory in two halves.
__global__ void __launch_bounds__(256) gptq_update_kernel(float* __restrict__ w, const float* __restrict__ u, const float* __restrict__ err, uint32_t n,
                                                         uint32_t k, uint32_t start, uint32_t end) {
    __shared__ float se[64][65], sub[64][65];
    const uint32_t tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // each thread: 4 x 4 outputs
    const uint32_t r0 = blockIdx.y * 64, c0 = end + blockIdx.x * 64, width = end - start;
    float acc[4][4] = {};
    for (uint32_t kk = 0; kk < width; kk += 64) {
        for (uint32_t i = threadIdx.x; i < 64 * 64; i += 256) {
            const uint32_t a = i >> 6, b = i & 63u;
            se[a][b] = (r0 + a < n && kk + b < width) ? err[(size_t)(r0 + a) * kBlock + kk + b] : 0.0f;
            sub[a][b] = (kk + a < width && c0 + b < k) ? u[(size_t)(start + kk + a) * k + c0 + b] : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (uint32_t t = 0; t < 64; ++t) {
            float a4[4], b4[4];
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) a4[i] = se[4 * ty + i][t], b4[i] = sub[t][4 * tx + i];
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i)
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(a4[i], b4[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i)
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            const uint32_t r = r0 + 4 * ty + i, c = c0 + 4 * tx + j;
            if (r < n && c < k) w[(size_t)r * k + c] = __fsub_rn(w[(size_t)r * k + c], acc[i][j]);
        }
}

}  // namespace

void launch_hessian_add(cudaStream_t s, const float* x, uint64_t rows, uint64_t k, float* h) {
    const uint32_t tiles = (uint32_t)((k + 31) / 32);
    hessian_add_kernel<<<dim3(tiles, tiles), 1024, 0, s>>>(x, (uint32_t)rows, (uint32_t)k, h);
}

uint64_t gptq_error_floats(uint64_t n) { return n * kBlock; }

// The whole column loop; `w` is consumed (it ends as the compensated weights), err holds gptq_error_floats(n) floats.
void launch_gptq(cudaStream_t s, float* w, const float* u, uint64_t n, uint64_t k, uint64_t group, float* err, uint32_t* q, float* scale, float* zero) {
    const uint32_t groups = (uint32_t)((k + group - 1) / group), words = (uint32_t)((k + 31) / 32 * 4);
    const size_t smem = (size_t)kBlock * kBlock * 4;
    GQ_CUDA(cudaFuncSetAttribute(gptq_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    for (uint64_t start = 0; start < k; start += kBlock) {
        const uint64_t end = start + kBlock < k ? start + kBlock : k;
        gptq_block_kernel<<<(uint32_t)((n + kRowsPerCta - 1) / kRowsPerCta), kRowsPerCta * 32, smem, s>>>(w, u, (uint32_t)n, (uint32_t)k, (uint32_t)start,
                                                                                                  (uint32_t)group, groups, words, err, q, scale, zero);
        if (end < k)
            gptq_update_kernel<<<dim3((uint32_t)((k - end + 63) / 64), (uint32_t)((n + 63) / 64)), 256, 0, s>>>(w, u, err, (uint32_t)n, (uint32_t)k,
                                                                                                            (uint32_t)start, (uint32_t)end);
    }
}

}  // namespace gq
