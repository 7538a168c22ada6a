// Prefill GEMM for int8 per-row weights on the fifth-generation tensor cores in
// EXACT integer arithmetic (tcgen05.mma kind::i8), replacing the reference's tiled SIMT kernel
//   crates/grilly-core/shaders/g2-linear-q8-tiled.glsl:41-100
// y[m][n] = (sum_k x[m][k] * q[n][k]) * scale[n] + bias[n], the scale applied in the float32
// epilogue as the reference does (:95-96).
//
// Why not tf32 (gemm_tc.cu): there the weight has to be widened to float32 on its way to the
// tensor core and x travels as 4 bytes per element; measured, that kernel is bound by what the
// SMs can pull out of L2 (~10 TB/s over the GPU at 57 flops per byte = 570 TFLOP/s). Here
// nothing is widened. x is held, as in the decode kernels, as an exact fixed-point integer
// X = rint(x 2^(22-e)), 2^e > max|x| over the row, split into THREE signed base-256 digit
// planes (3 bytes per element, written once per call by a small kernel), and the packed weight
// is the tensor core's operand exactly as it lies in HBM. The int8 rate is four times the tf32
// rate, so three planes cost less tensor time than one tf32 pass, and a tile of 256 features x
// 80 rows of x needs 128 (256 + 240) bytes per 128 k = 83 flops per byte. The result is exact
// up to X (2^-23 of the row's max |x| per element: finer than tf32's 2^-11 per element whenever
// a row's largest value is less than 4096 times the element) and one float32 rounding.
//
// Data flow per CTA tile (256 features x 80 rows of x), 128 k per pipeline stage:
//   TMA      q[128 features][128 bytes] x 2 -> shared memory, 128-byte swizzle: the two A operands
//   TMA      planes[d][80 rows][128 bytes], d = 0, 1, 2 -> shared memory: the B operand, 240 rows
//   1 thread issues 2 x 4 tcgen05.mma (M = 128, N = 240, K = 32 bytes) into two 128 x 240 int32
//            accumulators in tensor memory (columns d * 80 + r); tcgen05.commit frees the stage
//   8 warps  (epilogue) read a feature's 3 x 80 sums, join the digits as a 64-bit integer
//            (exact), convert once, scale by 2^(e-22) (exact) and scale[n], add bias[n], store y:
//            for a fixed row of x a warp writes 32 consecutive floats.
// A non-finite x gives a row of NaN.
//
// Algorithmic work: 2 M N K flops per call. Bound: the tensor pipe (int8 rate / 3), with the
// L2 -> SM operand traffic next.
#include "gq_internal.h"
#include "tc_common.cuh"

namespace gq {

namespace {

constexpr uint32_t kND = 3;                      // digit planes
constexpr uint32_t kChunk = 128;                 // bytes of K per stage
constexpr uint32_t kABytes = 128 * kChunk;       // 16 KB per A operand (128 features)
constexpr uint32_t kTmemCols = 512;              // accumulators at columns 0 and 256

// A tile is NA x 128 features by XR rows of x (XR a multiple of 16): N = 3 XR columns per accumulator. Prefill runs
// <2, 80>; fewer rows of x run one A operand and a narrower B, so that a decode batch costs the bytes of its rows only.
template <int NA, int XR>
struct Tile {
    static constexpr uint32_t kFT = 128 * NA, kN = XR * kND, kPlaneBytes = XR * kChunk;  // whole 1 KB swizzle atoms
    static constexpr uint32_t kStageBytes = NA * kABytes + kND * kPlaneBytes;
    static constexpr int kStages = (224 * 1024) / kStageBytes < 8 ? (224 * 1024) / kStageBytes : 8;
    static constexpr int kEpilogueWarps = 4 * NA;
    static constexpr int kThreads = (2 + kEpilogueWarps) * 32;  // warp 0 TMA, warp 1 MMA, then the epilogue
    static constexpr size_t kSmem = (size_t)kStages * kStageBytes + 256 + 1024;
};

// Row r of x -> planes[d][r][0 .. kp) and xinv[r] = 2^(e-22); rows m .. mpad - 1 are zeros.
__global__ void __launch_bounds__(256) x_planes_kernel(const float* __restrict__ x, uint32_t m, uint32_t k, uint32_t kp, uint32_t mpad,
                                                       uint8_t* __restrict__ planes, float* __restrict__ xinv) {
    GQ_GRID_DEP_SYNC();
    __shared__ float red[8];
    const uint32_t row = blockIdx.x, tid = threadIdx.x, words = kp / 4;
    uint32_t* out[kND];
#pragma unroll
    for (uint32_t d = 0; d < kND; ++d) out[d] = reinterpret_cast<uint32_t*>(planes + ((size_t)d * mpad + row) * kp);
    if (row >= m) {
        for (uint32_t w = tid; w < words; w += 256)
#pragma unroll
            for (uint32_t d = 0; d < kND; ++d) out[d][w] = 0u;
        if (tid == 0) xinv[row] = 0.0f;
        return;
    }
    const float* xr = x + (size_t)row * k;
    const bool vec = (k & 3u) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    auto load4 = [&](uint32_t w) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        const uint32_t i = 4 * w;
        if (vec) {
            if (i < k) v = __ldg(reinterpret_cast<const float4*>(xr + i));
        } else {
            if (i < k) v.x = __ldg(xr + i);
            if (i + 1 < k) v.y = __ldg(xr + i + 1);
            if (i + 2 < k) v.z = __ldg(xr + i + 2);
            if (i + 3 < k) v.w = __ldg(xr + i + 3);
        }
        return v;
    };
    float amax = 0.0f;
    bool bad = false;
    for (uint32_t w = tid; w < words; w += 256) {
        const float4 v = load4(w);
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        bad |= !(fabsf(v.x) <= 3.402823466e+38f) | !(fabsf(v.y) <= 3.402823466e+38f) | !(fabsf(v.z) <= 3.402823466e+38f) |
               !(fabsf(v.w) <= 3.402823466e+38f);
    }
    if (bad) amax = __uint_as_float(0x7f800000u);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((tid & 31) == 0) red[tid >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
    uint32_t b = __float_as_uint(amax) >> 23;
    float mult, inv;
    if (b == 255) {
        mult = 0.0f, inv = __uint_as_float(0x7fc00000u);  // a non-finite row of x gives NaN outputs
    } else if (amax == 0.0f) {
        mult = inv = 0.0f;
    } else {
        b = max(b, 32u);
        mult = __uint_as_float((275u - b) << 23);  // 2^(22 - e), 2^e > max |x|
        inv = __uint_as_float((b - 21u) << 23);    // 2^(e - 22)
    }
    if (tid == 0) xinv[row] = inv;
    for (uint32_t w = tid; w < words; w += 256) {
        const float4 v = load4(w);
        const float xv[4] = {v.x, v.y, v.z, v.w};
        uint32_t word[kND] = {0u, 0u, 0u};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int X = __float2int_rn(xv[j] * mult);  // |X| <= 2^22
            const int d0 = (int)(int8_t)X;
            X = (X - d0) >> 8;
            const int d1 = (int)(int8_t)X;
            const int d2 = (X - d1) >> 8;  // |d2| <= 64
            word[0] |= ((uint32_t)d0 & 0xFFu) << (8 * j), word[1] |= ((uint32_t)d1 & 0xFFu) << (8 * j), word[2] |= ((uint32_t)d2 & 0xFFu) << (8 * j);
        }
#pragma unroll
        for (uint32_t d = 0; d < kND; ++d) out[d][w] = word[d];
    }
}

template <int NA, int XR>
__global__ void __launch_bounds__((Tile<NA, XR>::kThreads), 1)
    gemm_i8_q8_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const float* __restrict__ xinv,
                      const float* __restrict__ scale, const float* __restrict__ bias, float* __restrict__ y, uint32_t m, uint32_t mpad,
                      uint32_t k, uint32_t n, uint32_t band, uint32_t* status) {
    using T = Tile<NA, XR>;
    constexpr uint32_t kFT = T::kFT, kXR = XR, kN = T::kN, kPlaneBytes = T::kPlaneBytes, kStageBytes = T::kStageBytes;
    constexpr int kStages = T::kStages, kEpilogueWarps = T::kEpilogueWarps;
    extern __shared__ uint8_t smem_unaligned[];
    uint8_t* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)kStages * kStageBytes);  // [kStages] the TMA's bytes landed
    uint64_t* empty = full + kStages;                                                     // [kStages] the MMAs read the stage
    uint64_t* dfull = empty + kStages;                                                    // the accumulators are complete
    uint64_t* dempty = dfull + 1;                                                         // ... and read out (every epilogue warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dempty + 1);
    volatile uint32_t* failed = tmem_slot + 1;

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t ftiles = (n + kFT - 1) / kFT, xtiles = mpad / kXR, tiles = ftiles * xtiles;
    const uint32_t chunks = (k + kChunk - 1) / kChunk;
    // Tile order: bands of `band` row tiles whose digit planes (with the whole weight) stay in L2; inside a band the
    // CTAs that run together share a pair of feature tiles and walk the band's rows.
    auto place = [&](uint32_t tile, uint32_t& f0, uint32_t& m0) {
        const uint32_t per_band = band * ftiles, b = tile / per_band, in_band = tile - b * per_band;
        const uint32_t rows_here = min(band, xtiles - b * band);  // the last band may be shorter
        f0 = (in_band / rows_here) * kFT, m0 = (b * band + in_band % rows_here) * kXR;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        mbar_init(dfull, 1);
        mbar_init(dempty, kEpilogueWarps);
        *failed = 0;
        mbar_fence_init();
        tma_prefetch_map(&xmap);
        tma_prefetch_map(&wmap);
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    // the digit planes are written by the kernel ahead in the stream: nothing reads them before this
    GQ_GRID_DEP_SYNC();

    if (warp == 0) {
        if (lane == 0) {
            uint32_t s = 0, round = 0;
            for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
                uint32_t f0, m0;
                place(tile, f0, m0);
                for (uint32_t c = 0; c < chunks; ++c) {
                    if (round && !mbar_wait(empty + s, (round - 1) & 1, failed, status, kStatusEmptyWaitTimedOut)) return;
                    uint8_t* st = smem + (size_t)s * kStageBytes;
                    mbar_arrive_expect_tx(full + s, kStageBytes);
#pragma unroll
                    for (uint32_t a = 0; a < (uint32_t)NA; ++a)
                        tma_load_2d(st + a * kABytes, &wmap, (int32_t)(c * kChunk), (int32_t)(f0 + 128 * a), full + s);
#pragma unroll
                    for (uint32_t d = 0; d < kND; ++d)
                        tma_load_2d(st + NA * kABytes + d * kPlaneBytes, &xmap, (int32_t)(c * kChunk), (int32_t)(d * mpad + m0), full + s);
                    if (++s == kStages) s = 0, ++round;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(2, 1, 1, 128, kN);  // s32 accumulate, s8 weights x s8 digits
            uint32_t s = 0, round = 0, t = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++t) {
                if (t) ok = mbar_wait(dempty, (t - 1) & 1, failed, status, kStatusMmaWaitTimedOut);
                tc_fence_after_sync();
                for (uint32_t c = 0; c < chunks && ok; ++c) {
                    ok = mbar_wait(full + s, round & 1, failed, status, kStatusFullWaitTimedOut);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + (size_t)s * kStageBytes), b_addr = a_addr + NA * kABytes;
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j) {
                        const uint64_t bd = umma_desc_k128(b_addr + 32 * j);
#pragma unroll
                        for (uint32_t a = 0; a < (uint32_t)NA; ++a)
                            umma_i8_ss(tmem + 256 * a, umma_desc_k128(a_addr + a * kABytes + 32 * j), bd, idesc, (c | j) != 0);
                    }
                    umma_commit(empty + s);
                    if (++s == kStages) s = 0, ++round;
                }
                if (ok) umma_commit(dfull);
            }
        }
    } else {
        // epilogue: thread = one feature (a lane of tensor memory) of one of the two accumulators
        const uint32_t quarter = warp & 3, half = (warp - 2) >> 2;
        uint32_t t = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++t) {
            uint32_t f0, m0;
            place(tile, f0, m0);
            const uint32_t col = f0 + 128 * half + 32 * quarter + lane;
            ok = ok && mbar_wait(dfull, t & 1, failed, status, kStatusMmaWaitTimedOut);
            if (ok) {
                tc_fence_after_sync();
                const float sc = col < n ? scale[col] : 0.0f;
                const float bs = (bias && col < n) ? bias[col] : 0.0f;
#pragma unroll 1
                for (uint32_t r0 = 0; r0 < kXR; r0 += 16) {
                    uint32_t d0[16], d1[16], d2[16];
                    const uint32_t at = tmem_addr(tmem, 32 * quarter, 256 * half + r0);
                    tmem_ld16(at, d0);
                    tmem_ld16(at + kXR, d1);
                    tmem_ld16(at + 2 * kXR, d2);
                    tmem_wait_ld();
                    if (col < n) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const uint32_t r = m0 + r0 + i;
                            if (r < m) {
                                // the three digit sums joined exactly; one rounding to float32; 2^(e-22) is a power of two
                                const long long T = (long long)(int)d0[i] + ((long long)(int)d1[i] << 8) + ((long long)(int)d2[i] << 16);
                                float v = __fmul_rn(__fmul_rn(__ll2float_rn(T), __ldg(xinv + r)), sc);
                                if (bias) v = __fadd_rn(v, bs);
                                y[(size_t)r * n + col] = v;
                            }
                        }
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(dempty);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

// rows of x per tile by the number of rows of the call
inline uint64_t pad_to(uint64_t m, uint64_t xr) { return (m + xr - 1) / xr * xr; }
// Up to 64 rows: one A operand and the narrowest B that holds the rows. Beyond: two A operands and 80 rows of x a tile, or
// 64 where that makes the busiest CTA's share smaller (256 rows x 14336 features: 224 tiles either way, in two waves).
inline uint32_t tile_rows_for(uint64_t m, uint64_t n, int sm_count) {
    if (m <= 64) return m <= 16 ? 16u : m <= 32 ? 32u : 64u;
    const uint64_t ft = (n + 255) / 256;
    const uint64_t c80 = (ft * ((m + 79) / 80) + sm_count - 1) / sm_count * 80, c64 = (ft * ((m + 63) / 64) + sm_count - 1) / sm_count * 64;
    return c64 < c80 ? 64u : 80u;
}
// the scratch is sized without knowing the features: room for either padding
inline uint64_t padded_rows_most(uint64_t m) {
    if (m <= 64) return pad_to(m, tile_rows_for(m, 1, 1));
    return pad_to(m, 80) > pad_to(m, 64) ? pad_to(m, 80) : pad_to(m, 64);
}
inline uint64_t planes_bytes(uint64_t m, uint64_t k) { return (kND * padded_rows_most(m) * ((k + 15) / 16 * 16) + 255) / 256 * 256; }

template <int NA, int XR>
void launch_tiles(cudaStream_t s, int sm_count, uint32_t* status, const uint8_t* planes, const float* xinv, uint64_t m, uint64_t mpad, uint64_t k,
                  const uint32_t* q, const float* scale, const float* bias, uint64_t n, float* y) {
    using T = Tile<NA, XR>;
    const uint64_t rowbytes = (k + 15) / 16 * 16;
    const CUtensorMap xmap = make_tensor_map_2d(planes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rowbytes, kND * mpad, rowbytes, kChunk, XR, Swizzle::B128);
    const CUtensorMap wmap = make_tensor_map_2d(q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rowbytes, n, rowbytes, kChunk, 128, Swizzle::B128);
    const uint64_t tiles = ((n + T::kFT - 1) / T::kFT) * (mpad / XR);
    const uint32_t grid = (uint32_t)(tiles < (uint64_t)sm_count ? tiles : (uint64_t)sm_count);
    // a band's digit planes: at most ~32 MB, so that they and the weight fit the 126 MB L2 together
    uint64_t band = (32ull << 20) / (kND * XR * rowbytes);
    band = band < 1 ? 1 : band > mpad / XR ? mpad / XR : band;
    GQ_CUDA(cudaFuncSetAttribute(gemm_i8_q8_kernel<NA, XR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T::kSmem));
    launch_after(gemm_i8_q8_kernel<NA, XR>, dim3(grid), dim3(T::kThreads), T::kSmem, s, xmap, wmap, xinv, scale, bias, y, (uint32_t)m, (uint32_t)mpad,
                 (uint32_t)k, (uint32_t)n, (uint32_t)band, status);
}

}  // namespace

// Bytes of scratch a call needs: the three digit planes of x and a float per row.
uint64_t gemm_q8_i8_scratch_bytes(uint64_t m, uint64_t k) { return planes_bytes(m, k) + padded_rows_most(m) * 4; }

// Returns false when the shape is outside this kernel: K beyond 2^17 (the int32 sums) or a weight that is not 16-byte
// aligned. `scratch` holds gemm_q8_i8_scratch_bytes(m, k) bytes. Two launches: x -> digit planes, the product.
bool launch_gemm_q8_i8(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                       const float* scale, const float* bias, uint64_t n, float* y, void* scratch) {
    if (m == 0 || n == 0 || k == 0 || k > (1u << 17) || (reinterpret_cast<uintptr_t>(q) & 15) != 0) return false;
    const uint32_t xr = tile_rows_for(m, n, sm_count);
    const uint64_t rowbytes = (k + 15) / 16 * 16, mpad = pad_to(m, xr);
    if (kND * mpad > 0x7fffffffull || m * n > (1ull << 40)) return false;
    uint8_t* planes = reinterpret_cast<uint8_t*>(scratch);
    float* xinv = reinterpret_cast<float*>(planes + planes_bytes(m, k));
    launch_after(x_planes_kernel, dim3((uint32_t)mpad), dim3(256), 0, s, x, (uint32_t)m, (uint32_t)k, (uint32_t)rowbytes, (uint32_t)mpad, planes, xinv);
    if (m > 64) {
        if (xr == 64) launch_tiles<2, 64>(s, sm_count, status, planes, xinv, m, mpad, k, q, scale, bias, n, y);
        else launch_tiles<2, 80>(s, sm_count, status, planes, xinv, m, mpad, k, q, scale, bias, n, y);
    } else if (xr == 16) {
        launch_tiles<1, 16>(s, sm_count, status, planes, xinv, m, mpad, k, q, scale, bias, n, y);
    } else if (xr == 32) {
        launch_tiles<1, 32>(s, sm_count, status, planes, xinv, m, mpad, k, q, scale, bias, n, y);
    } else {
        launch_tiles<1, 64>(s, sm_count, status, planes, xinv, m, mpad, k, q, scale, bias, n, y);
    }
    return true;
}

}  // namespace gq
