// Weight packers and unpackers: fp32 -> int8 per-row / int4 group-wise and
// back. These replace the reference's GLSL shaders
//   crates/grilly-core/shaders/g2-quantize-q8.glsl:22-53
//   crates/grilly-core/shaders/g2-dequantize-q8.glsl:15-21
//   crates/grilly-core/shaders/g2-quantize-q4.glsl:30-70
//   crates/grilly-core/shaders/g2-dequantize-q4.glsl:16-24
// and must produce the same bits. What makes that hold under nvcc:
//   - the two divisions are IEEE (__fdiv_rn), which the shader's div_rn is
//     proven equal to (crates/grilly-core/tests/div_rn.rs:73-99);
//   - every product or difference the shader marks `precise` goes through
//     __fmul_rn / __fsub_rn / __fadd_rn, which the compiler never contracts
//     into an FMA; the one real fma (int4 dequantize) is __fmaf_rn;
//   - rintf rounds half to even, as roundEven does;
//   - max and min do not depend on the order they are taken in, so the
//     reductions are free to be shaped for the hardware.
//
// All four kernels are pure streaming work, bounded by HBM bandwidth:
// quantize reads 4 bytes and writes 1 (int8) or 0.5 (int4) per weight.
#include "gq_internal.h"

namespace gq {

static constexpr float kEps = 1.1920928955078125e-7f;  // float32 eps, the floor of every scale

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ uint32_t q8_of(float w, float inv) {
    float r = rintf(__fmul_rn(w, inv));
    r = fminf(fmaxf(r, -128.0f), 127.0f);
    return (uint32_t)(int)r & 0xFFu;
}

// One CTA per row. Pass 1 takes the row's absolute maximum; pass 2 re-reads
// the row (from L1/L2: it was just read) and writes one packed word per
// thread per step. VEC: the row starts on a 16-byte boundary and k % 4 == 0,
// so a word's four floats are one float4 load.
template <bool VEC>
__global__ void __launch_bounds__(256) quantize_q8_kernel(const float* __restrict__ w, uint32_t rows, uint32_t k,
                                                          uint32_t words, uint32_t* __restrict__ q,
                                                          float* __restrict__ scale) {
    __shared__ float s_part[8];
    __shared__ float s_amax;
    const uint32_t tid = threadIdx.x;
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* wr = w + (size_t)row * k;
        float m = 0.0f;
        if (VEC) {
            const float4* w4 = reinterpret_cast<const float4*>(wr);
            for (uint32_t i = tid; i < k / 4; i += 256) {
                float4 v = w4[i];
                m = fmaxf(fmaxf(m, fabsf(v.x)), fmaxf(fabsf(v.y), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
        } else {
            for (uint32_t i = tid; i < k; i += 256) m = fmaxf(m, fabsf(wr[i]));
        }
        m = warp_max(m);
        if ((tid & 31) == 0) s_part[tid >> 5] = m;
        __syncthreads();
        if (tid < 32) {
            float v = tid < 8 ? s_part[tid] : 0.0f;
            v = warp_max(v);
            if (tid == 0) s_amax = v;
        }
        __syncthreads();
        // torchao: max|w| / ((127 - (-128)) / 2), at least float32 eps
        const float sc = fmaxf(__fdiv_rn(s_amax, 127.5f), kEps);
        const float inv = __fdiv_rn(1.0f, sc);
        uint32_t* qr = q + (size_t)row * words;
        for (uint32_t word = tid; word < words; word += 256) {
            uint32_t packed = 0;
            const uint32_t i0 = word * 4;
            if (VEC) {
                if (i0 < k) {
                    float4 v = reinterpret_cast<const float4*>(wr)[word];
                    packed = q8_of(v.x, inv) | (q8_of(v.y, inv) << 8) | (q8_of(v.z, inv) << 16) | (q8_of(v.w, inv) << 24);
                }
            } else {
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j)
                    if (i0 + j < k) packed |= q8_of(wr[i0 + j], inv) << (8 * j);
            }
            qr[word] = packed;
        }
        if (tid == 0) scale[row] = sc;
        __syncthreads();  // s_amax is rewritten by the next row
    }
}

// One thread per packed word: four weights out. The single multiply is what
// makes this bit-exact against the host (crates/grilly-infer/tests/quant.rs:94-103).
template <bool VEC>
__global__ void __launch_bounds__(256) dequantize_q8_kernel(const uint32_t* __restrict__ q, const float* __restrict__ scale,
                                                            uint32_t rows, uint32_t k, uint32_t words, float* __restrict__ w) {
    const uint32_t kw = (k + 3) / 4;  // words that hold values
    const size_t total = (size_t)rows * kw;
    for (size_t id = (size_t)blockIdx.x * 256 + threadIdx.x; id < total; id += (size_t)gridDim.x * 256) {
        const uint32_t row = (uint32_t)(id / kw), word = (uint32_t)(id % kw);
        const uint32_t packed = q[(size_t)row * words + word];
        const float sc = scale[row];
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = __fmul_rn((float)(int)(int8_t)(packed >> (8 * j)), sc);
        float* out = w + (size_t)row * k + word * 4;
        if (VEC) {
            *reinterpret_cast<float4*>(out) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j)
                if (word * 4 + j < k) out[j] = v[j];
        }
    }
}

// int4: one CTA per row, each thread owning whole words (8 consecutive
// values; a group is a multiple of 32 values, so a word never straddles
// one). The row is taken in chunks of whole groups that fit the shared
// arrays: (1) every thread records the min/max of each of its words,
// (2) one thread per group reduces its words' entries and writes the
// group's scale and zero point, (3) every thread re-reads its words and
// writes the packed levels. Rows pad with zero words to a whole 16-byte
// vector, as the shader's last group does (g2-quantize-q4.glsl:53-57).
static constexpr uint32_t kQ4ChunkWords = 2048;  // 16384 values of a row per pass

template <bool VEC>
__global__ void __launch_bounds__(256) quantize_q4_kernel(const float* __restrict__ w, uint32_t rows, uint32_t k,
                                                          uint32_t group, uint32_t words, uint32_t groups,
                                                          uint32_t chunk_groups, uint32_t* __restrict__ q,
                                                          float* __restrict__ scale, float* __restrict__ zero) {
    extern __shared__ float smem[];
    const uint32_t gw = group / 8;  // words per group
    float* s_min = smem;
    float* s_max = smem + chunk_groups * gw;
    float* s_lo = s_max + chunk_groups * gw;
    float* s_sc = s_lo + chunk_groups;
    const uint32_t tid = threadIdx.x;
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* wr = w + (size_t)row * k;
        uint32_t* qr = q + (size_t)row * words;
        for (uint32_t g0 = 0; g0 < groups; g0 += chunk_groups) {
            const uint32_t ng = min(chunk_groups, groups - g0);
            const uint32_t word0 = g0 * gw;
            const uint32_t nwords = ng * gw;  // may run past the row's last valued word
            // (1) per-word extremes
            for (uint32_t t = tid; t < nwords; t += 256) {
                const uint32_t i0 = (word0 + t) * 8;
                float lo = INFINITY, hi = -INFINITY;
                if (VEC && i0 + 8 <= k) {
                    const float4 a = *reinterpret_cast<const float4*>(wr + i0);
                    const float4 b = *reinterpret_cast<const float4*>(wr + i0 + 4);
                    lo = fminf(fminf(fminf(a.x, a.y), fminf(a.z, a.w)), fminf(fminf(b.x, b.y), fminf(b.z, b.w)));
                    hi = fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)), fmaxf(fmaxf(b.x, b.y), fmaxf(b.z, b.w)));
                } else {
                    for (uint32_t j = 0; j < 8; ++j)
                        if (i0 + j < k) {
                            lo = fminf(lo, wr[i0 + j]);
                            hi = fmaxf(hi, wr[i0 + j]);
                        }
                }
                s_min[t] = lo;
                s_max[t] = hi;
            }
            __syncthreads();
            // (2) per-group parameters
            for (uint32_t g = tid; g < ng; g += 256) {
                float lo = INFINITY, hi = -INFINITY;
                for (uint32_t t = g * gw; t < (g + 1) * gw; ++t) {
                    lo = fminf(lo, s_min[t]);
                    hi = fmaxf(hi, s_max[t]);
                }
                float s, z;
                if ((size_t)(g0 + g) * group >= k) {  // a group past the row's end (g2-quantize-q4.glsl:37-41)
                    s = 1.0f, z = 0.0f, lo = 0.0f;
                } else {
                    s = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), 15.0f), kEps);
                    z = __fadd_rn(lo, __fmul_rn(8.0f, s));
                }
                s_lo[g] = lo;
                s_sc[g] = s;
                scale[(size_t)row * groups + g0 + g] = s;
                zero[(size_t)row * groups + g0 + g] = z;
            }
            __syncthreads();
            // (3) levels
            for (uint32_t t = tid; t < nwords; t += 256) {
                const uint32_t word = word0 + t;
                if (word >= words) continue;
                const uint32_t i0 = word * 8;
                const float lo = s_lo[t / gw], s = s_sc[t / gw];
                uint32_t packed = 0;
                if (VEC && i0 + 8 <= k) {
                    const float4 a = *reinterpret_cast<const float4*>(wr + i0);
                    const float4 b = *reinterpret_cast<const float4*>(wr + i0 + 4);
                    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                    for (uint32_t j = 0; j < 8; ++j) {
                        float lv = rintf(__fdiv_rn(__fsub_rn(v[j], lo), s));
                        lv = fminf(fmaxf(lv, 0.0f), 15.0f);
                        packed |= (uint32_t)(int)lv << (4 * j);
                    }
                } else {
                    for (uint32_t j = 0; j < 8; ++j)
                        if (i0 + j < k) {
                            float lv = rintf(__fdiv_rn(__fsub_rn(wr[i0 + j], lo), s));
                            lv = fminf(fmaxf(lv, 0.0f), 15.0f);
                            packed |= (uint32_t)(int)lv << (4 * j);
                        }
                }
                qr[word] = packed;
            }
            __syncthreads();
        }
        // padding words past the last group's words (k not a multiple of 32 leaves
        // up to three; a group count that covers them already wrote zeros above)
        for (uint32_t word = groups * gw + tid; word < words; word += 256) qr[word] = 0;
    }
}

// One thread per packed word: eight weights out, w = fma(level, s, zero - 8 s)
// (one fused multiply-add, as the host's mul_add: crates/grilly-infer/tests/quant4.rs:115-127).
template <bool VEC>
__global__ void __launch_bounds__(256) dequantize_q4_kernel(const uint32_t* __restrict__ q, const float* __restrict__ scale,
                                                            const float* __restrict__ zero, uint32_t rows, uint32_t k,
                                                            uint32_t group, uint32_t words, uint32_t groups,
                                                            float* __restrict__ w) {
    const uint32_t kw = (k + 7) / 8;
    const size_t total = (size_t)rows * kw;
    for (size_t id = (size_t)blockIdx.x * 256 + threadIdx.x; id < total; id += (size_t)gridDim.x * 256) {
        const uint32_t row = (uint32_t)(id / kw), word = (uint32_t)(id % kw);
        const uint32_t packed = q[(size_t)row * words + word];
        const uint32_t g = word * 8 / group;
        const float s = scale[(size_t)row * groups + g];
        const float lo = __fsub_rn(zero[(size_t)row * groups + g], __fmul_rn(8.0f, s));
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __fmaf_rn((float)((packed >> (4 * j)) & 0xFu), s, lo);
        float* out = w + (size_t)row * k + word * 8;
        if (VEC) {
            reinterpret_cast<float4*>(out)[0] = make_float4(v[0], v[1], v[2], v[3]);
            reinterpret_cast<float4*>(out)[1] = make_float4(v[4], v[5], v[6], v[7]);
        } else {
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j)
                if (word * 8 + j < k) out[j] = v[j];
        }
    }
}

__global__ void __launch_bounds__(256) fill_u32_kernel(uint32_t* dst, size_t n, uint32_t word) {
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) dst[i] = word;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static inline uint32_t grid_for(size_t items, uint32_t per_block, uint32_t cap) {
    size_t blocks = (items + per_block - 1) / per_block;
    if (blocks < 1) blocks = 1;
    return (uint32_t)(blocks < cap ? blocks : cap);
}

void launch_quantize_q8(cudaStream_t s, const float* w, uint64_t rows, uint64_t k, uint32_t* q, float* scale) {
    const uint32_t words = (uint32_t)((k + 15) / 16 * 4);
    const uint32_t grid = grid_for(rows, 1, 148 * 32);
    if (aligned16(w) && k % 4 == 0)
        quantize_q8_kernel<true><<<grid, 256, 0, s>>>(w, (uint32_t)rows, (uint32_t)k, words, q, scale);
    else
        quantize_q8_kernel<false><<<grid, 256, 0, s>>>(w, (uint32_t)rows, (uint32_t)k, words, q, scale);
}

void launch_dequantize_q8(cudaStream_t s, const uint32_t* q, const float* scale, uint64_t rows, uint64_t k, float* w) {
    const uint32_t words = (uint32_t)((k + 15) / 16 * 4);
    const uint32_t grid = grid_for(rows * ((k + 3) / 4), 256, 148 * 16);
    if (aligned16(w) && k % 4 == 0)
        dequantize_q8_kernel<true><<<grid, 256, 0, s>>>(q, scale, (uint32_t)rows, (uint32_t)k, words, w);
    else
        dequantize_q8_kernel<false><<<grid, 256, 0, s>>>(q, scale, (uint32_t)rows, (uint32_t)k, words, w);
}

void launch_quantize_q4(cudaStream_t s, const float* w, uint64_t rows, uint64_t k, uint64_t group, uint32_t* q,
                        float* scale, float* zero) {
    const uint32_t words = (uint32_t)((k + 31) / 32 * 4);
    const uint32_t groups = (uint32_t)((k + group - 1) / group);
    const uint32_t gw = (uint32_t)(group / 8);
    uint32_t chunk_groups = kQ4ChunkWords / gw;
    if (chunk_groups < 1) chunk_groups = 1;
    if (chunk_groups > groups) chunk_groups = groups;
    const size_t smem = ((size_t)chunk_groups * gw * 2 + (size_t)chunk_groups * 2) * sizeof(float);
    if (smem > 200 * 1024) fail("int4 group_size %llu is larger than the quantizer's shared-memory staging allows", (unsigned long long)group);
    const uint32_t grid = grid_for(rows, 1, 148 * 32);
    const bool vec = aligned16(w) && k % 4 == 0;  // every word of the row then starts 16-byte aligned
    auto kernel = vec ? quantize_q4_kernel<true> : quantize_q4_kernel<false>;
    if (smem > 48 * 1024) GQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<grid, 256, smem, s>>>(w, (uint32_t)rows, (uint32_t)k, (uint32_t)group, words, groups, chunk_groups, q, scale, zero);
}

void launch_dequantize_q4(cudaStream_t s, const uint32_t* q, const float* scale, const float* zero, uint64_t rows,
                          uint64_t k, uint64_t group, float* w) {
    const uint32_t words = (uint32_t)((k + 31) / 32 * 4);
    const uint32_t groups = (uint32_t)((k + group - 1) / group);
    const uint32_t grid = grid_for(rows * ((k + 7) / 8), 256, 148 * 16);
    if (aligned16(w) && k % 8 == 0)
        dequantize_q4_kernel<true><<<grid, 256, 0, s>>>(q, scale, zero, (uint32_t)rows, (uint32_t)k, (uint32_t)group, words, groups, w);
    else
        dequantize_q4_kernel<false><<<grid, 256, 0, s>>>(q, scale, zero, (uint32_t)rows, (uint32_t)k, (uint32_t)group, words, groups, w);
}

void launch_fill_u32(cudaStream_t s, uint32_t* dst, uint64_t n, uint32_t word) {
    fill_u32_kernel<<<grid_for(n, 256, 148 * 16), 256, 0, s>>>(dst, n, word);
}

}  // namespace gq
