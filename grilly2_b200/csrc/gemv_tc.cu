// Decode GEMV on the fifth-generation tensor cores (tcgen05, kind::i8) for
// int8 per-row weights and one or two rows of x.
//
// Arithmetic (as in gemv_dp4a.cu, with ONE exponent per row of x): x is held
// as an exact fixed-point integer X = rint(x 2^(30-e)), 2^e > max|x| over the
// row, split into four signed base-256 digit planes. The packed weights are
// the MMA's A operand exactly as they lie in HBM — a TMA tensor-map load with
// the 128-byte swizzle puts a [128 features x 128 bytes of K] tile in shared
// memory in the layout the tensor core reads, no instruction touches a
// weight — and the digit planes are the B operand's columns (four per row of
// x). D[feature][digit] accumulates in int32 in tensor memory over the whole
// of K, exactly; the epilogue recombines the digits in float64 (exact), scales
// by 2^(e-30), rounds to float32 once, and applies the row scale and bias as
// the reference does: y = (sum_k x q) * scale + bias. |D| <= K * 2^14, so K
// up to 2^17 cannot overflow.
//
// Roles: warp 0 streams weight tiles with TMA into a ring of 16 KB stages;
// warp 1 issues the MMAs (one thread) and owns the TMEM allocation; warp 4
// reads the accumulator out of tensor memory and warps 4-7 finish and write
// y; every warp helps convert x first. One CTA per SM, each owning a
// contiguous range of output features within one feature of the others.
//
// Measured (B200, 14336 x 4096, one row of x): 16.7 us per call, of which
// ~2.9 us is launch + x conversion + epilogue and the rest the 32 pipeline
// steps at ~0.4 us each, whether the step loads only or multiplies only: a
// [128 x 128 B] tile costs the TMA unit ~800 cycles (128 row segments) and four
// K = 32 MMAs cost the tensor core about the same, whatever M and N are. The
// warp-level kernel in gemv_imma.cu is faster today (12.9 us) and is what AUTO
// picks; this kernel is selected with GQ_KERNEL_UMMA.
//
// Algorithmic bytes per launch: packed weights + scales + x + y (+ bias).
// Bound: HBM bandwidth.
#include "gq_internal.h"
#include "tc_common.cuh"

namespace gq {

namespace {

constexpr int kThreads = 384;            // producer, MMA, four epilogue warps; six more that only help convert x
constexpr uint32_t kStage = 128 * 128;   // one A tile: 128 features x 128 bytes of K
constexpr uint32_t kBoxRows = 128;       // rows per TMA box: the whole tile in one instruction (16-row boxes ran 35% slower)
constexpr int kMaxStages = 10;
constexpr uint32_t kTmemCols = 256;      // two accumulators of 128 columns (features)

// x (MR rows) -> the B operand: for every 128 bytes of K one 1 KB swizzle atom
// of 8 rows x 128 bytes, row n = 4 * xrow + digit, byte o of the row stored at
// n * 128 + (((o >> 4) ^ n) << 4) + (o & 15). Also writes 2^(e-30) per row.
template <int MR, bool XVEC>
__device__ void prepare_digits(const float* __restrict__ x, uint32_t k, uint32_t chunks, uint8_t* xdig, float* xinv,
                               float* red) {
    constexpr int kCache = 4;  // float4 per thread kept in registers between the two passes
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t n4 = chunks * 32;  // groups of four k, padding included
    auto load4 = [&](const float* xr, uint32_t idx) {
        const uint32_t i = idx * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (XVEC) {
            if (i < k) v = __ldg(reinterpret_cast<const float4*>(xr + i));  // k % 4 == 0 here
        } else {
            if (i < k) v.x = __ldg(xr + i);
            if (i + 1 < k) v.y = __ldg(xr + i + 1);
            if (i + 2 < k) v.z = __ldg(xr + i + 2);
            if (i + 3 < k) v.w = __ldg(xr + i + 3);
        }
        return v;
    };
#pragma unroll
    for (int r = 0; r < MR; ++r) {
        const float* xr = x + (size_t)r * k;
        float4 cache[kCache];
#pragma unroll
        for (int c = 0; c < kCache; ++c) cache[c] = load4(xr, tid + c * kThreads);  // all requested at once
        float amax = 0.0f;
        bool bad = false;
        auto fold = [&](const float4& v) {
            const float a = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
            amax = fmaxf(amax, a);
            bad |= !(fabsf(v.x) <= 3.402823466e+38f) | !(fabsf(v.y) <= 3.402823466e+38f) | !(fabsf(v.z) <= 3.402823466e+38f) |
                   !(fabsf(v.w) <= 3.402823466e+38f);
        };
#pragma unroll
        for (int c = 0; c < kCache; ++c) fold(cache[c]);
        for (uint32_t idx = tid + kCache * kThreads; idx < n4; idx += kThreads) fold(load4(xr, idx));
        if (bad) amax = __uint_as_float(0x7f800000u);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (lane == 0) red[r * 16 + warp] = amax;
        __syncthreads();
        amax = 0.0f;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) amax = fmaxf(amax, red[r * 16 + w]);
        uint32_t b = __float_as_uint(amax) >> 23;
        float mult, inv;
        if (b == 255) {
            mult = 0.0f, inv = __uint_as_float(0x7fc00000u);  // a non-finite row of x gives NaN outputs
        } else if (amax == 0.0f) {
            mult = inv = 0.0f;
        } else {
            b = max(b, 32u);
            mult = __uint_as_float((283u - b) << 23);  // 2^(30 - e)
            inv = __uint_as_float((b - 29u) << 23);    // 2^(e - 30)
        }
        if (tid == 0) xinv[r] = inv;
        auto emit = [&](uint32_t idx, const float4& v) {
            const float xv[4] = {v.x, v.y, v.z, v.w};
            int dg[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int X = __float2int_rn(xv[j] * mult);
                dg[j][0] = (int)(int8_t)X;
                X = (X - dg[j][0]) >> 8;
                dg[j][1] = (int)(int8_t)X;
                X = (X - dg[j][1]) >> 8;
                dg[j][2] = (int)(int8_t)X;
                dg[j][3] = (X - dg[j][2]) >> 8;
            }
            const uint32_t i = idx * 4, chunk = i >> 7, o = i & 127;
#pragma unroll
            for (int d = 0; d < 4; ++d) {
                const uint32_t n = 4 * r + d;
                const uint32_t word = ((uint32_t)dg[0][d] & 0xFFu) | (((uint32_t)dg[1][d] & 0xFFu) << 8) |
                                      (((uint32_t)dg[2][d] & 0xFFu) << 16) | ((uint32_t)dg[3][d] << 24);
                *reinterpret_cast<uint32_t*>(xdig + (size_t)chunk * 1024 + n * 128 + ((((o >> 4) ^ n) & 7) << 4) + (o & 15)) = word;
            }
        };
#pragma unroll
        for (int c = 0; c < kCache; ++c)
            if (tid + c * kThreads < n4) emit(tid + c * kThreads, cache[c]);
        for (uint32_t idx = tid + kCache * kThreads; idx < n4; idx += kThreads) emit(idx, load4(xr, idx));
    }
}

template <int MR, bool XVEC>
__global__ void __launch_bounds__(kThreads, 1)
    gemv_tc_q8_kernel(const __grid_constant__ CUtensorMap wmap, const float* __restrict__ x, const float* __restrict__ scale,
                      const float* __restrict__ bias, float* __restrict__ y, uint32_t k, uint32_t n, uint32_t chunks,
                      uint32_t nstages, uint32_t* status) {
    extern __shared__ uint8_t smem_unaligned[];
    uint8_t* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);  // swizzle atoms need 1 KB alignment
    uint8_t* stages = smem;                                   // nstages x 16 KB, each 1024-aligned
    uint8_t* xdig = stages + (size_t)nstages * kStage;        // chunks x 1 KB
    uint64_t* full = reinterpret_cast<uint64_t*>(xdig + (size_t)chunks * 1024);
    uint64_t* empty = full + kMaxStages;
    uint64_t* dfull = empty + kMaxStages;   // [2] accumulator ready
    uint64_t* dempty = dfull + 2;           // [2] accumulator drained
    float* xinv = reinterpret_cast<float*>(dempty + 2);  // [2]
    float* red = xinv + 2;                                // [2][16]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(red + 32);
    volatile uint32_t* failed = tmem_slot + 1;
    int* dsm = reinterpret_cast<int*>(tmem_slot + 4);  // [8][129]: the digit rows of one tile

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t per = n / gridDim.x, extra = n % gridDim.x;
    const uint32_t cb = blockIdx.x * per + min(blockIdx.x, extra), ce = cb + per + (blockIdx.x < extra ? 1u : 0u);
    const uint32_t tiles = (ce - cb + 127) / 128;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < nstages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(dfull + a, 1);
            mbar_init(dempty + a, 1);  // the warp that reads the accumulator out
        }
        *failed = 0;
        mbar_fence_init();
        tma_prefetch_map(&wmap);
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);

    // The first weight tiles are requested before x is converted: they do not depend on it.
    uint32_t ps = 0, pround = 0, ptile = 0, pchunk = 0;  // producer position (warp 0, lane 0)
    auto produce_one = [&]() -> bool {  // issues the next stage; false when there is nothing left or a wait gave up
        if (ptile >= tiles) return false;
        if (pround && !mbar_wait(empty + ps, (pround - 1) & 1, failed, status, kStatusEmptyWaitTimedOut)) return false;
        const uint32_t row0 = cb + 128 * ptile, rows = min(128u, ce - row0);
        const uint32_t boxes = (rows + kBoxRows - 1) / kBoxRows;
        mbar_arrive_expect_tx(full + ps, boxes * kBoxRows * 128);
        for (uint32_t b = 0; b < boxes; ++b)
            tma_load_2d(stages + (size_t)ps * kStage + b * kBoxRows * 128, &wmap, (int32_t)(pchunk * 128),
                        (int32_t)(row0 + b * kBoxRows), full + ps);
        if (++pchunk == chunks) pchunk = 0, ++ptile;
        if (++ps == nstages) ps = 0, ++pround;
        return true;
    };
    if (threadIdx.x == 0)
        for (uint32_t i = 0; i < nstages; ++i)
            if (!produce_one()) break;

    prepare_digits<MR, XVEC>(x, k, chunks, xdig, xinv, red);
    fence_proxy_async_smem();  // the digit planes were written by ordinary stores; the tensor core reads them
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0)
            while (produce_one()) {
            }
    } else if (warp == 1) {
        if (lane == 0) {
            // The tensor core streams A's rows through an array that holds B: an instruction's time goes
            // with M, not N. So the eight digit rows are A — one 1 KB swizzle atom per 128 bytes of K, read
            // as all eight 8-row groups of an M = 64 operand by giving the descriptor a zero group stride
            // (rows 8-63 of D repeat rows 0-7) — and the 128 features of the weight tile are B (N = 128).
            constexpr uint32_t idesc = umma_idesc(2, 1, 1, 64, 128);
            uint32_t s = 0, round = 0;
            bool ok = true;
            for (uint32_t tile = 0; tile < tiles && ok; ++tile) {
                const uint32_t a = tile & 1;
                if (tile >= 2) ok = mbar_wait(dempty + a, ((tile >> 1) - 1) & 1, failed, status, kStatusMmaWaitTimedOut);
                tc_fence_after_sync();
                for (uint32_t c = 0; c < chunks && ok; ++c) {
                    ok = mbar_wait(full + s, round & 1, failed, status, kStatusFullWaitTimedOut);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t w_addr = smem_u32(stages + (size_t)s * kStage), x_addr = smem_u32(xdig + (size_t)c * 1024);
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j)
                        umma_i8_ss(tmem + a * 128, umma_desc_k128(x_addr + 32 * j, 0), umma_desc_k128(w_addr + 32 * j), idesc, c | j);
                    umma_commit(empty + s);  // the stage is free once these MMAs have read it
                    if (++s == nstages) s = 0, ++round;
                }
                if (ok) umma_commit(dfull + a);
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // Epilogue, warps 4-7. D is [digit row][feature]: rows 0-7 sit in TMEM lanes 0-7, which warp 4
        // (4 % 4 == 0) may read; it moves them to shared memory, then one thread per feature recombines
        // the digits and writes y.
        const uint32_t et = threadIdx.x - 128;  // 0 … 127: the feature of the tile this thread finishes
        bool ok = true;
        for (uint32_t tile = 0; tile < tiles; ++tile) {
            const uint32_t a = tile & 1;
            if (warp == 4) {
                ok = ok && mbar_wait(dfull + a, (tile >> 1) & 1, failed, status, kStatusMmaWaitTimedOut);
                if (ok) {
                    tc_fence_after_sync();
#pragma unroll
                    for (uint32_t c0 = 0; c0 < 128; c0 += 16) {
                        uint32_t d[16];
                        tmem_ld16(tmem_addr(tmem, 0, a * 128 + c0), d);
                        tmem_wait_ld();
                        if (lane < 8) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) dsm[lane * 129 + c0 + i] = (int)d[i];
                        }
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(dempty + a);  // the accumulator may be overwritten
            }
            named_barrier_sync(2, 128);
            const uint32_t row = cb + 128 * tile + et;
            if (*failed == 0 && row < ce) {
                const float sc = scale[row];
#pragma unroll
                for (int r = 0; r < MR; ++r) {
                    const double T = (double)dsm[(4 * r) * 129 + et] + 256.0 * (double)dsm[(4 * r + 1) * 129 + et] +
                                     65536.0 * (double)dsm[(4 * r + 2) * 129 + et] + 16777216.0 * (double)dsm[(4 * r + 3) * 129 + et];
                    float out = __fmul_rn((float)(T * (double)xinv[r]), sc);  // (sum x q) * scale
                    if (bias) out = __fadd_rn(out, bias[row]);
                    y[(size_t)r * n + row] = out;
                }
            }
            named_barrier_sync(2, 128);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

// Returns false when the shape is outside this kernel (more than two rows of
// x, or x too long for its digit planes to stay in shared memory).
bool launch_gemv_q8_tc(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                       const float* scale, const float* bias, uint64_t n, float* y) {
    if (m > 2 || k > (1u << 17)) return false;
    const uint64_t rowbytes = (k + 15) / 16 * 16;
    const uint32_t chunks = (uint32_t)((rowbytes + 127) / 128);
    const size_t fixed = (size_t)chunks * 1024 + (2 * kMaxStages + 4) * 8 + 48 * 4 + 8 * 129 * 4 + 64 + 1024;  // + alignment slack
    const size_t budget = 226 * 1024;
    if (fixed + 2 * (size_t)kStage > budget) return false;
    uint32_t nstages = (uint32_t)((budget - fixed) / kStage);
    if (nstages > (uint32_t)kMaxStages) nstages = kMaxStages;
    const size_t smem = fixed + (size_t)nstages * kStage;
    const CUtensorMap wmap = make_tensor_map_2d(q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rowbytes, n, rowbytes, 128, kBoxRows, Swizzle::B128);
    const uint32_t grid = (uint32_t)(n < (uint64_t)sm_count ? n : (uint64_t)sm_count);
    const bool xvec = aligned16(x) && k % 4 == 0;
    auto launch = [&](auto kernel) {
        GQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kernel<<<grid, kThreads, smem, s>>>(wmap, x, scale, bias, y, (uint32_t)k, (uint32_t)n, chunks, nstages, status);
    };
    if (m == 1)
        xvec ? launch(gemv_tc_q8_kernel<1, true>) : launch(gemv_tc_q8_kernel<1, false>);
    else
        xvec ? launch(gemv_tc_q8_kernel<2, true>) : launch(gemv_tc_q8_kernel<2, false>);
    return true;
}

}  // namespace gq
