// Prefill GEMM for int8 per-row weights on the fifth-generation tensor cores
// (tcgen05, kind::tf32), replacing the reference's tiled SIMT kernel
//   crates/grilly-core/shaders/g2-linear-q8-tiled.glsl:41-100
// y[m][n] = (sum_k x[m][k] * q[n][k]) * scale[n] + bias[n], the scale applied
// in the float32 epilogue as the reference does (:95-96). int8 codes are exact
// in tf32; only x is rounded (to tf32 by the tensor core), which is what the
// 2e-3 tolerance of this path allows for.
//
// Data flow per CTA tile of 128 output features x 256 rows of x, K taken 32 at
// a time (one pipeline stage):
//   TMA      x[256 rows][32 floats] -> shared memory, 128-byte swizzle: the B operand as it lies
//   TMA      q[128 features][32 bytes] -> shared memory (raw int8)
//   4 warps  read their feature's 32 bytes, widen to float32 in registers and store them to TENSOR
//            MEMORY (tcgen05.st): the A operand, one feature per TMEM lane, one k per column. The
//            dequantised weights never touch shared memory, whose bandwidth is what a tf32 MMA fed
//            from it twice over would run out of first.
//   1 thread issues 4 x tcgen05.mma (M = 128 features, N = 256 rows of x, K = 8) into a 128 x 256
//            float32 accumulator in TMEM; tcgen05.commit frees the stage and the A slot.
//   4 warps  (epilogue) read the accumulator, multiply by scale[n], add bias[n] and store y. The
//            accumulator is [feature][row of x], so for a fixed row of x a warp writes 32 consecutive
//            floats of y: coalesced.
//
// Bound: the tensor pipe (2 M N K flops per call); weights stream once per
// 256 rows of x and stay in L2 across row tiles.
#include "gq_internal.h"
#include "tc_common.cuh"

namespace gq {

namespace {

constexpr uint32_t kFT = 128;                 // features per tile (MMA M)
constexpr uint32_t kXT = 256;                 // rows of x per tile (MMA N)
constexpr uint32_t kKS = 32;                  // k per stage
constexpr uint32_t kXBytes = kXT * kKS * 4;   // 32 KB
constexpr uint32_t kWBytes = kFT * kKS;       // 4 KB
constexpr uint32_t kStageBytes = kXBytes + kWBytes;
constexpr int kStages = 5;
constexpr int kASlots = 4;                    // A operand ring in TMEM, 32 columns each
constexpr uint32_t kTmemCols = 512;           // 256 accumulator + 128 A ring (power of two)
constexpr int kThreads = 384;                 // warps: 0 TMA, 1 MMA, 2-3 idle, 4-7 dequant, 8-11 epilogue

__global__ void __launch_bounds__(kThreads, 1)
    gemm_tf32_q8_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
                        const float* __restrict__ scale, const float* __restrict__ bias, float* __restrict__ y, uint32_t m,
                        uint32_t k, uint32_t n, uint32_t* status) {
    extern __shared__ uint8_t smem_unaligned[];
    uint8_t* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kStages * kStageBytes);
    uint64_t* full = bars;                 // [kStages]  TMA landed
    uint64_t* empty = full + kStages;      // [kStages]  MMA read x (1) + dequant warps read w (4)
    uint64_t* afull = empty + kStages;     // [kASlots]  dequant warps stored A (4)
    uint64_t* aempty = afull + kASlots;    // [kASlots]  MMA consumed A (1)
    uint64_t* dfull = aempty + kASlots;    // accumulator complete (1)
    uint64_t* dempty = dfull + 1;          // accumulator drained (4)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dempty + 1);
    volatile uint32_t* failed = tmem_slot + 1;

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t ftiles = (n + kFT - 1) / kFT, xtiles = (m + kXT - 1) / kXT, tiles = ftiles * xtiles;
    const uint32_t ksteps = (k + kKS - 1) / kKS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 5);
        }
        for (int a = 0; a < kASlots; ++a) {
            mbar_init(afull + a, 4);
            mbar_init(aempty + a, 1);
        }
        mbar_init(dfull, 1);
        mbar_init(dempty, 4);
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
    const uint32_t tmem_d = tmem, tmem_a = tmem + 256;  // columns 0-255: D; 256-383: the A ring

    if (warp == 0) {
        if (lane == 0) {
            uint32_t s = 0, round = 0;
            for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
                const uint32_t f0 = (tile / xtiles) * kFT, m0 = (tile % xtiles) * kXT;
                for (uint32_t ks = 0; ks < ksteps; ++ks) {
                    if (round && !mbar_wait(empty + s, (round - 1) & 1, failed, status, kStatusEmptyWaitTimedOut)) return;
                    uint8_t* st = smem + (size_t)s * kStageBytes;
                    mbar_arrive_expect_tx(full + s, kXBytes + kWBytes);
                    tma_load_2d(st, &xmap, (int32_t)(ks * kKS), (int32_t)m0, full + s);
                    tma_load_2d(st + kXBytes, &wmap, (int32_t)(ks * kKS), (int32_t)f0, full + s);
                    if (++s == kStages) s = 0, ++round;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(1, 2, 2, kFT, kXT);  // f32 accumulate, tf32 x tf32
            uint32_t s = 0, round = 0, a = 0, around = 0, t = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++t) {
                if (t) ok = mbar_wait(dempty, (t - 1) & 1, failed, status, kStatusMmaWaitTimedOut);
                for (uint32_t ks = 0; ks < ksteps && ok; ++ks) {
                    ok = mbar_wait(full + s, round & 1, failed, status, kStatusFullWaitTimedOut) &&
                         mbar_wait(afull + a, around & 1, failed, status, kStatusMmaWaitTimedOut);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t x_addr = smem_u32(smem + (size_t)s * kStageBytes);
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j)
                        umma_tf32_ts(tmem_d, tmem_a + a * 32 + j * 8, umma_desc_k128(x_addr + 32 * j), idesc, ks | j);
                    umma_commit(empty + s);
                    umma_commit(aempty + a);
                    if (++s == kStages) s = 0, ++round;
                    if (++a == kASlots) a = 0, ++around;
                }
                if (ok) umma_commit(dfull);
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // dequant: thread = one feature of the tile = one TMEM lane
        const uint32_t sub = warp & 3, row = 32 * sub + lane;
        uint32_t s = 0, round = 0, a = 0, around = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
            for (uint32_t ks = 0; ks < ksteps; ++ks) {
                ok = ok && mbar_wait(full + s, round & 1, failed, status, kStatusFullWaitTimedOut);
                if (ok && around) ok = mbar_wait(aempty + a, (around - 1) & 1, failed, status, kStatusMmaWaitTimedOut);
                if (ok) {
                    const uint4* src = reinterpret_cast<const uint4*>(smem + (size_t)s * kStageBytes + kXBytes + row * kKS);
                    const uint4 lo = src[0], hi = src[1];
                    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                    uint32_t f[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) f[i] = __float_as_uint((float)(int)(int8_t)(w[i >> 2] >> (8 * (i & 3))));
                    tc_fence_after_sync();
                    tmem_st32(tmem_addr(tmem_a, 32 * sub, a * 32), f);
                    tmem_wait_st();
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(afull + a);
                    mbar_arrive(empty + s);
                }
                if (++s == kStages) s = 0, ++round;
                if (++a == kASlots) a = 0, ++around;
            }
        }
    } else if (warp >= 8) {
        // epilogue: thread = one feature; the accumulator's columns are rows of x
        const uint32_t sub = warp & 3;
        uint32_t t = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++t) {
            const uint32_t f0 = (tile / xtiles) * kFT, m0 = (tile % xtiles) * kXT;
            const uint32_t col = f0 + 32 * sub + lane;
            ok = ok && mbar_wait(dfull, t & 1, failed, status, kStatusMmaWaitTimedOut);
            if (ok) {
                tc_fence_after_sync();
                const float sc = col < n ? scale[col] : 0.0f;
                const float bs = (bias && col < n) ? bias[col] : 0.0f;
                for (uint32_t c0 = 0; c0 < kXT; c0 += 32) {
                    uint32_t d[32];
                    tmem_ld32(tmem_addr(tmem_d, 32 * sub, c0), d);
                    tmem_wait_ld();
                    if (col < n) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const uint32_t r = m0 + c0 + i;
                            if (r < m) {
                                float v = __fmul_rn(__uint_as_float(d[i]), sc);
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

}  // namespace

// Returns false when the shape does not meet the tensor maps' rules: x rows
// must start 16-byte aligned (k % 4 == 0 and an aligned base).
bool launch_gemm_q8_tc(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                       const float* scale, const float* bias, uint64_t n, float* y) {
    if (k % 4 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0) return false;
    const uint64_t rowbytes = (k + 15) / 16 * 16;
    const CUtensorMap xmap = make_tensor_map_2d(x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, k, m, k * 4, kKS, kXT, Swizzle::B128);
    const CUtensorMap wmap = make_tensor_map_2d(q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rowbytes, n, rowbytes, kKS, kFT, Swizzle::None);
    const uint64_t tiles = ((n + kFT - 1) / kFT) * ((m + kXT - 1) / kXT);
    const uint32_t grid = (uint32_t)(tiles < (uint64_t)sm_count ? tiles : (uint64_t)sm_count);
    const size_t smem = (size_t)kStages * kStageBytes + 256 + 1024;
    GQ_CUDA(cudaFuncSetAttribute(gemm_tf32_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    gemm_tf32_q8_kernel<<<grid, kThreads, smem, s>>>(xmap, wmap, scale, bias, y, (uint32_t)m, (uint32_t)k, (uint32_t)n, status);
    return true;
}

}  // namespace gq
