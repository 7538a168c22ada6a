// Decode GEMV for one or two rows of x on the warp-level integer tensor
// instruction (mma.sync m16n8k32, 8-bit operands, int32 accumulate).
//
// Same arithmetic as gemv_dp4a.cu: x is held as an exact fixed-point number
// per block of weights,
//     x[k] ~= X[k] 2^(e-30),  X = d0 + 256 d1 + 65536 d2 + 2^24 d3  (signed base-256 digits),
// and the packed weights multiply the four digit planes in exact integer
// arithmetic. Here the digit planes are the COLUMNS of the MMA's B operand
// (four per row of x, so two rows fill the eight columns) and sixteen output
// features are its rows, so one warp instruction performs 16 x 32 x 8
// multiply-adds: per weight the kernel issues ~0.8 thread instructions — 3/8
// to split int4 nibbles into bytes, the rest loads and the per-block float32
// epilogue — against 1.7-3.9 for the dp4a kernel and ~5 for the float one.
// Measured on a B200 the warp-level integer MMA itself is the limit: the
// tensor pipe retires one m16n8k32 in about 20 cycles per SM, so this kernel
// tops out near 4.5 TB/s for int8 weights and 2.5 TB/s for int4; the tcgen05
// kernels exist to lift that.
//
// Mapping. A "block" is 64 bytes of one weight row: four 16-byte vectors, 128
// int4 levels or 64 int8 values; it is also the block x's exponent is shared
// over, and for int4 it must lie inside one quantization group (group_size a
// multiple of 128; other group sizes take the dp4a kernel). Thread (g, t) of a
// warp, g = lane / 4, t = lane % 4, loads vector t of the block for feature
// rows g and g + 8 of a 16-row tile — so a warp load covers eight rows x 64
// contiguous bytes — and word j of those vectors feeds MMA j. The k order
// inside an MMA is therefore a permutation of the memory order; the digit
// planes of x are laid out in shared memory in the same permutation, once per
// CTA, so it costs nothing.
//
// Work split. One CTA per SM owns a contiguous range of output features, the
// ranges differing by at most one feature, taken in panels of 128 rows. The
// 16 warps of a CTA split K: warp w takes blocks w, w + 16, … of every row in
// the panel (so the B fragments it loaded for a block serve all the panel's
// tiles), and the 16 partial sums per output are added through shared memory
// in a fixed order: the result is deterministic and equal on every replay.
//
// Algorithmic bytes per launch: packed weights + scales (+ zero points) + x +
// y (+ bias), each once. Bound: HBM bandwidth.
#include "async_common.cuh"
#include "gq_internal.h"
#include "math_common.cuh"

namespace gq {

namespace {

constexpr int kWarps = 16;                       // consumer warps per CTA; they split K
constexpr int kThreads = (kWarps + 1) * 32;      // plus the producer warp
constexpr int kPanel = 128;                      // rows a CTA reduces at a time
constexpr uint32_t kPartBytes = 2048;            // bytes of a weight row per stage: 32 blocks, two per consumer warp
constexpr int kBlocksPerWarp = kPartBytes / 64 / kWarps;
constexpr uint32_t kRowStride = kPartBytes + 64;  // 64 mod 128: rows land in different banks
constexpr uint32_t kStageBytes = 16 * kRowStride;
constexpr int kMaxStages = 5;

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// D(16x8, s32) += A(16x32, u8 row-major) * B(32x8, s8 column-major)
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 2^(30-e) and 2^(e-30) for a block whose largest |x| is amax (2^e > amax);
// (0, 0) for a zero block, (0, NaN) for a non-finite one.
__device__ __forceinline__ void block_scales(float amax, float& mult, float& inv) {
    uint32_t b = __float_as_uint(amax) >> 23;
    if (b == 255) {
        mult = 0.0f;
        inv = __uint_as_float(0x7fc00000u);
        return;
    }
    if (amax == 0.0f) {
        mult = inv = 0.0f;
        return;
    }
    b = max(b, 32u);
    mult = __uint_as_float((283u - b) << 23);
    inv = __uint_as_float((b - 29u) << 23);
}

__device__ __forceinline__ void digits_of(int X, int (&d)[4]) {
    d[0] = (int)(int8_t)X;
    X = (X - d[0]) >> 8;
    d[1] = (int)(int8_t)X;
    X = (X - d[1]) >> 8;
    d[2] = (int)(int8_t)X;
    d[3] = (X - d[2]) >> 8;
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return ((uint32_t)a & 0xFFu) | (((uint32_t)b & 0xFFu) << 8) | (((uint32_t)c & 0xFFu) << 16) | ((uint32_t)d << 24);
}

// One row of x -> B fragments. xb[((blk * 4 + t) * 8 + col) * R + reg], col =
// 4 * xrow + digit, R = 8 registers per (block, t, col) for int4 (word j,
// parity p -> 2j + p: the even and the odd nibbles of word j of vector t) and
// 4 for int8 (word j). One packed word of weights (8 or 4 values of x) per
// thread; the 16 words of a block sit in 16 adjacent lanes.
template <bool IS4, bool XVEC, int PRO>
__device__ __forceinline__ void prepare_x(const float* __restrict__ xr, uint32_t xrow, uint32_t k, uint32_t nblocks,
                                          uint32_t* xb, float* xinv, float* xsum, const Prologue& pro, float rinv) {
    static_assert(PRO == 0 || (!IS4 && XVEC), "prologues are built for int8 weights and an aligned row of x");
    constexpr int E = IS4 ? 8 : 4;  // values of x per packed word
    constexpr int R = IS4 ? 8 : 4;
    for (uint32_t base = 0; base < nblocks * 16; base += kWarps * 32) {  // the consumer threads, 0 … 511, run this
        const uint32_t wd = base + threadIdx.x;
        const bool live = wd < nblocks * 16;
        const uint32_t k0 = wd * E, blk = wd >> 4, t = (wd >> 2) & 3, j = wd & 3;
        float xv[E];
        if (PRO == 1) {  // x' = (x + residual) * rinv * w; CTA 0 also stores x + residual
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f), w4 = v;
            if (live && k0 < k) {
                v = __ldg(reinterpret_cast<const float4*>(xr + k0));
                if (pro.res) {
                    const float4 r4 = __ldg(reinterpret_cast<const float4*>(pro.res + k0));
                    v.x = __fadd_rn(v.x, r4.x), v.y = __fadd_rn(v.y, r4.y), v.z = __fadd_rn(v.z, r4.z), v.w = __fadd_rn(v.w, r4.w);
                }
                if (pro.h_out && blockIdx.x == 0) *reinterpret_cast<float4*>(pro.h_out + k0) = v;
                w4 = __ldg(reinterpret_cast<const float4*>(pro.w + k0));
            }
            xv[0] = __fmul_rn(__fmul_rn(v.x, rinv), w4.x), xv[1] = __fmul_rn(__fmul_rn(v.y, rinv), w4.y);
            xv[2] = __fmul_rn(__fmul_rn(v.z, rinv), w4.z), xv[3] = __fmul_rn(__fmul_rn(v.w, rinv), w4.w);
        } else if (PRO == 2) {  // x'[j] = silu(x[j]) * x[k + j]
            float4 g4 = make_float4(0.f, 0.f, 0.f, 0.f), u4 = g4;
            if (live && k0 < k) g4 = __ldg(reinterpret_cast<const float4*>(xr + k0)), u4 = __ldg(reinterpret_cast<const float4*>(xr + k + k0));
            xv[0] = silu_mul_fast(g4.x, u4.x), xv[1] = silu_mul_fast(g4.y, u4.y), xv[2] = silu_mul_fast(g4.z, u4.z), xv[3] = silu_mul_fast(g4.w, u4.w);
        } else if (XVEC) {
#pragma unroll
            for (int h = 0; h < E / 4; ++h) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (live && k0 + 4 * h < k) v = __ldg(reinterpret_cast<const float4*>(xr + k0) + h);
                xv[4 * h] = v.x, xv[4 * h + 1] = v.y, xv[4 * h + 2] = v.z, xv[4 * h + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < E; ++i) xv[i] = (live && k0 + i < k) ? __ldg(xr + k0 + i) : 0.0f;
        }
        float amax = 0.0f, sum = 0.0f;
        bool bad = false;
#pragma unroll
        for (int i = 0; i < E; ++i) {
            amax = fmaxf(amax, fabsf(xv[i]));
            bad |= !(fabsf(xv[i]) <= 3.402823466e+38f);
            sum += xv[i];
        }
        if (bad) amax = __uint_as_float(0x7f800000u);
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        if (!live) continue;
        float mult, inv;
        block_scales(amax, mult, inv);
        int d[E][4];
#pragma unroll
        for (int i = 0; i < E; ++i) digits_of(__float2int_rn(xv[i] * mult), d[i]);
        uint32_t* dst = xb + ((size_t)(blk * 4 + t) * 8 + 4 * xrow) * R;
#pragma unroll
        for (int dg = 0; dg < 4; ++dg) {
            if (IS4) {
                dst[dg * R + 2 * j] = pack4(d[0][dg], d[2][dg], d[4][dg], d[6][dg]);
                dst[dg * R + 2 * j + 1] = pack4(d[1][dg], d[3][dg], d[5][dg], d[7][dg]);
            } else {
                dst[dg * R + j] = pack4(d[0][dg], d[1][dg], d[2][dg], d[3][dg]);
            }
        }
        if ((wd & 15) == 0) {
            xinv[blk] = inv;
            if (IS4) xsum[blk] = sum;
        }
    }
}

// ── the kernel ───────────────────────────────────────────────────────────
// Warp 16 is the producer: it streams the CTA's weight rows into a ring of
// shared-memory stages with bulk (TMA) copies, one copy per row so that rows
// can sit kRowStride bytes apart (a stride that is 64 mod 128 keeps the
// 16-byte fragment reads of eight different rows in different banks). A
// stage holds one 16-row tile x up to 2048 bytes of each row. Warps 0-15
// consume: all of them work on the same stage, each on its own 64-byte
// blocks, so up to five stages — 160 KB per SM — are in flight while they
// compute, and HBM never waits for the arithmetic.
// 1 / sqrt(mean((x + residual)^2) + eps) over one row of k values, by the 512 consumer threads (add_rms_norm_kernel's
// arithmetic: squares in float32, their sum in float64). `red` is 16 doubles of shared memory.
__device__ __forceinline__ float row_rms_inverse(const float* __restrict__ xr, const Prologue& pro, uint32_t k, double* red) {
    double ss = 0.0;
    for (uint32_t i = threadIdx.x * 4; i < k; i += kWarps * 32 * 4) {
        float4 v = __ldg(reinterpret_cast<const float4*>(xr + i));
        if (pro.res) {
            const float4 r4 = __ldg(reinterpret_cast<const float4*>(pro.res + i));
            v.x = __fadd_rn(v.x, r4.x), v.y = __fadd_rn(v.y, r4.y), v.z = __fadd_rn(v.z, r4.z), v.w = __fadd_rn(v.w, r4.w);
        }
        ss += (double)__fmul_rn(v.x, v.x), ss += (double)__fmul_rn(v.y, v.y), ss += (double)__fmul_rn(v.z, v.z), ss += (double)__fmul_rn(v.w, v.w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    named_barrier_sync(2, kWarps * 32);
    double t = 0.0;
#pragma unroll
    for (int i = 0; i < kWarps; ++i) t += red[i];
    const float mean = __fdiv_rn((float)t, (float)k);
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, pro.eps)));
}

template <bool IS4, int MR, bool XVEC, int PRO>
__global__ void __launch_bounds__(kThreads, 1)
    gemv_imma_kernel(const float* __restrict__ x, const uint8_t* __restrict__ q, const float* __restrict__ scale,
                     const float* __restrict__ zero, const float* __restrict__ bias, float* __restrict__ y, uint32_t k,
                     uint32_t n, uint32_t vecs, uint32_t groups, uint32_t gshift, uint32_t gblocks, uint32_t nblocks,
                     uint32_t nstages, uint32_t* status, Prologue pro, bool early) {
    // Launched so that it may start before the kernel ahead of it has finished: nothing below touches global memory
    // before a griddepcontrol.wait, except the producer's weight copies when `early` says that kernel did not write them.
    constexpr int R = IS4 ? 8 : 4;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* stages = smem_raw;                                                  // nstages * kStageBytes
    uint32_t* xb = reinterpret_cast<uint32_t*>(stages + (size_t)nstages * kStageBytes);  // nblocks * 32 * R words
    float* xinv = reinterpret_cast<float*>(xb + (size_t)nblocks * 32 * R);      // MR * nblocks
    float* xsum = xinv + MR * nblocks;                                           // MR * nblocks (int4)
    float* partial = xsum + (IS4 ? MR * nblocks : 0);                            // kWarps * kPanel * MR
    uint64_t* full = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(partial + kWarps * kPanel * MR) + 7) & ~uintptr_t(7));
    uint64_t* empty = full + kMaxStages;
    volatile uint32_t* failed = reinterpret_cast<volatile uint32_t*>(empty + kMaxStages);

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // this CTA's features [cb, ce); the first n % gridDim CTAs take one more
    const uint32_t per = n / gridDim.x, extra = n % gridDim.x;
    const uint32_t cb = blockIdx.x * per + min(blockIdx.x, extra), ce = cb + per + (blockIdx.x < extra ? 1u : 0u);
    const uint32_t rowbytes = vecs * 16;
    const uint32_t parts = (rowbytes + kPartBytes - 1) / kPartBytes;  // stages per tile
    const uint32_t tiles = (ce - cb + 15) / 16;

    if (warp == kWarps) {
        // ── producer: sets the barriers up itself; the consumers meet it on named barrier 4 after converting x, so neither waits
        // for the other at the start ──
        if (lane == 0) {
            for (uint32_t s = 0; s < nstages; ++s) {
                mbar_init(full + s, 1);        // the producer's arrive.expect_tx
                mbar_init(empty + s, kWarps);  // one arrival per consumer warp
            }
            *failed = 0;
            mbar_fence_init();
        }
        __syncwarp();
        asm volatile("bar.arrive 4, %0;" ::"n"(kThreads) : "memory");
        if (!early) asm volatile("griddepcontrol.wait;" ::: "memory");
        uint32_t s = 0, round = 0;
        for (uint32_t tile = 0; tile < tiles; ++tile) {
            const uint32_t row0 = cb + 16 * tile, nrows = min(16u, ce - row0);
            for (uint32_t part = 0; part < parts; ++part) {
                if (round && !mbar_wait(empty + s, (round - 1) & 1, failed, status, kStatusEmptyWaitTimedOut)) return;
                const uint32_t bytes = min(kPartBytes, rowbytes - part * kPartBytes);
                if (lane == 0) mbar_arrive_expect_tx(full + s, nrows * bytes);
                __syncwarp();
                if (lane < nrows)
                    bulk_load(stages + (size_t)s * kStageBytes + lane * kRowStride,
                              q + (size_t)(row0 + lane) * rowbytes + (size_t)part * kPartBytes, bytes, full + s);
                if (++s == nstages) s = 0, ++round;
            }
        }
        return;
    }

    // ── consumers ──
    asm volatile("griddepcontrol.wait;" ::: "memory");  // x may be the output of the kernel ahead
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // only now: see launch_after
    const uint32_t g = lane >> 2, t = lane & 3;
    __shared__ double s_red[kWarps];
    float rinv = 0.0f;
    if (PRO == 1) rinv = row_rms_inverse(x, pro, k, s_red);
#pragma unroll
    for (int r = 0; r < MR; ++r)
        prepare_x<IS4, XVEC, PRO>(x + (size_t)r * k, r, k, nblocks, xb, xinv + r * nblocks, xsum + r * nblocks, pro, rinv);
    named_barrier_sync(1, kWarps * 32);
    asm volatile("bar.sync 4, %0;" ::"n"(kThreads) : "memory");  // the producer's barriers are ready

    // this thread finishes feature row g (even t) or g + 8 (odd t) of each tile, for row t / 2 of x
    const uint32_t rowoff = g + 8 * (t & 1), xrow = t >> 1;
    const bool owner = xrow < MR;
    const bool odd = t & 1;

    // Group parameters (scale, zero) of the rows this warp finishes, for its (up to two) blocks of a
    // stage. They stream from HBM like the weights, so they are requested kMaxStages stages ahead
    // with 4-byte cp.async copies into a small per-warp ring and read back from shared memory.
    float* pring = reinterpret_cast<float*>(const_cast<uint32_t*>(failed) + 4);  // [kMaxStages][kWarps][kBlocksPerWarp][16][2]
    auto param_slot = [&](uint32_t slot, int bi) {
        return pring + ((((size_t)slot * kWarps + warp) * kBlocksPerWarp + bi) * 16 + rowoff) * 2;
    };
    auto issue_params = [&](uint32_t slot, uint32_t tile, uint32_t part) {
        if (IS4 && t < 2 && tile < tiles) {
            const uint32_t row = cb + 16 * tile + rowoff;
#pragma unroll
            for (int bi = 0; bi < kBlocksPerWarp; ++bi) {
                const uint32_t blk = part * (kPartBytes / 64) + warp + kWarps * bi;
                if (row < ce && blk < nblocks) {
                    const uint32_t grp = gblocks == 1 ? blk : (gshift < 32 ? blk >> gshift : blk / gblocks);
                    const uint32_t dst = smem_u32(param_slot(slot, bi));
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(scale + (size_t)row * groups + grp) : "memory");
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4), "l"(zero + (size_t)row * groups + grp) : "memory");
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");  // one group per stage, empty or not
    };
    uint32_t ptile = 0, ppart = 0;  // the stage whose parameters are requested next
    auto advance_params = [&]() {
        if (++ppart == parts) ppart = 0, ++ptile;
    };
    for (uint32_t i = 0; i < (uint32_t)kMaxStages; ++i) {
        issue_params(i, ptile, ppart);
        advance_params();
    }
    uint32_t pslot = 0;

    float acc = 0.0f;
    bool ok = true;
    uint32_t s = 0, round = 0;
    for (uint32_t tile = 0; tile < tiles; ++tile) {
        for (uint32_t part = 0; part < parts; ++part) {
            asm volatile("cp.async.wait_group %0;" ::"n"(kMaxStages - 1) : "memory");  // this stage's parameters have landed
            __syncwarp();
            ok = ok && mbar_wait(full + s, round & 1, failed, status, kStatusFullWaitTimedOut);
            if (ok) {
                const uint8_t* st = stages + (size_t)s * kStageBytes;
#pragma unroll
                for (int bi = 0; bi < kBlocksPerWarp; ++bi) {
                    const uint32_t b = warp + kWarps * bi;             // block within the part
                    const uint32_t blk = part * (kPartBytes / 64) + b;  // block within the row
                    if (blk >= nblocks) break;
                    const uint4 u4 = *reinterpret_cast<const uint4*>(st + g * kRowStride + 64 * b + 16 * t);        // row g
                    const uint4 l4 = *reinterpret_cast<const uint4*>(st + (g + 8) * kRowStride + 64 * b + 16 * t);  // row g + 8
                    uint32_t bf[R];  // B fragments: this lane's column is g (digit g % 4 of x row g / 4)
                    if (g < 4 * MR) {
                        const uint4* src = reinterpret_cast<const uint4*>(xb + ((size_t)(blk * 4 + t) * 8 + g) * R);
#pragma unroll
                        for (int i = 0; i < R / 4; ++i) {
                            const uint4 v = src[i];
                            bf[4 * i] = v.x, bf[4 * i + 1] = v.y, bf[4 * i + 2] = v.z, bf[4 * i + 3] = v.w;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < R; ++i) bf[i] = 0;
                    }
                    int d[4] = {0, 0, 0, 0};
                    const uint32_t u[4] = {u4.x, u4.y, u4.z, u4.w}, l[4] = {l4.x, l4.y, l4.z, l4.w};
                    if (IS4) {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            mma_u8s8(d, u[j] & 0x0F0F0F0Fu, l[j] & 0x0F0F0F0Fu, (u[j] >> 4) & 0x0F0F0F0Fu,
                                     (l[j] >> 4) & 0x0F0F0F0Fu, bf[2 * j], bf[2 * j + 1]);
                    } else {
                        mma_s8s8(d, u[0], l[0], u[1], l[1], bf[0], bf[1]);
                        mma_s8s8(d, u[2], l[2], u[3], l[3], bf[2], bf[3]);
                    }
                    // d[0], d[1]: row g, columns 2t, 2t+1; d[2], d[3]: row g + 8. Even t holds digits 0,1
                    // (the low half of X), odd t digits 2,3: swap halves with the neighbour so that each
                    // of the pair ends with one complete row.
                    const int pg = d[0] + (d[1] << 8), ph = d[2] + (d[3] << 8);
                    const int got = __shfl_xor_sync(0xffffffffu, odd ? pg : ph, 1);
                    const float T = odd ? __fmaf_rn(65536.0f, (float)ph, (float)got) : __fmaf_rn(65536.0f, (float)got, (float)pg);
                    if (owner) {
                        const float inv = xinv[xrow * nblocks + blk];
                        if (IS4) {
                            const float2 sz = *reinterpret_cast<const float2*>(param_slot(pslot, bi));
                            const float mn = __fsub_rn(sz.y, __fmul_rn(8.0f, sz.x));  // min = zero - 8 s
                            acc = __fmaf_rn(__fmul_rn(sz.x, inv), T, acc);
                            acc = __fmaf_rn(mn, xsum[xrow * nblocks + blk], acc);
                        } else {
                            acc = __fmaf_rn(inv, T, acc);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + s);  // this warp has read the stage
            if (++s == nstages) s = 0, ++round;
            issue_params(pslot, ptile, ppart);  // the slot just read is free again (the __syncwarp above orders it)
            advance_params();
            if (++pslot == (uint32_t)kMaxStages) pslot = 0;
        }
        // the tile is complete for this warp's share of K
        const uint32_t pr = (tile % (kPanel / 16)) * 16 + rowoff;
        if (owner) partial[((size_t)warp * kPanel + pr) * MR + xrow] = acc;
        acc = 0.0f;
        if ((tile + 1) % (kPanel / 16) == 0 || tile + 1 == tiles) {
            // a panel of up to 128 rows: fixed-order sum of the 16 partials, one thread per output
            named_barrier_sync(1, kWarps * 32);
            const uint32_t p0 = cb + (tile / (kPanel / 16)) * kPanel, prow = min((uint32_t)kPanel, ce - p0);
            for (uint32_t i = threadIdx.x; i < prow * MR; i += kWarps * 32) {
                const uint32_t prr = i / MR, r = i % MR, col = p0 + prr;
                float v = 0.0f;
#pragma unroll
                for (int w = 0; w < kWarps; ++w) v += partial[((size_t)w * kPanel + prr) * MR + r];
                if (!IS4) v = __fmul_rn(v, scale[col]);  // the row scale multiplies the finished sum
                if (bias) v = __fadd_rn(v, bias[col]);
                y[(size_t)r * n + col] = v;
            }
            named_barrier_sync(1, kWarps * 32);
        }
    }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <bool IS4, int MR>
bool run(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t k, const uint32_t* q, const float* scale,
         const float* zero, const float* bias, uint64_t n, uint64_t group, float* y, bool early, int kind = 0, Prologue pro = Prologue()) {
    const uint32_t vecs = (uint32_t)(IS4 ? (k + 31) / 32 : (k + 15) / 16);
    const uint32_t nblocks = (vecs + 3) / 4;
    const uint32_t groups = IS4 ? (uint32_t)((k + group - 1) / group) : 0;
    const uint32_t gblocks = IS4 ? (uint32_t)(group / 128) : 1;
    uint32_t gshift = 32;  // log2(gblocks) when it is a power of two, else 32 (the kernel then divides)
    for (uint32_t sft = 0; sft < 32; ++sft)
        if ((1u << sft) == gblocks) gshift = sft;
    constexpr int R = IS4 ? 8 : 4;
    const size_t fixed = ((size_t)nblocks * 32 * R + (size_t)MR * nblocks * (IS4 ? 2 : 1) + (size_t)kWarps * kPanel * MR + 1) * 4 +
                         2 * kMaxStages * 8 + 32 + (IS4 ? (size_t)kMaxStages * kWarps * kBlocksPerWarp * 16 * 2 * 4 : 0);
    const size_t budget = 226 * 1024;
    if (fixed + 2 * (size_t)kStageBytes > budget) return false;
    uint32_t nstages = (uint32_t)((budget - fixed) / kStageBytes);
    if (nstages > kMaxStages) nstages = kMaxStages;
    const uint32_t grid = (uint32_t)(n < (uint64_t)sm_count ? n : (uint64_t)sm_count);
    // A small layer asks only for the stages a CTA fills (a kernel launched behind it can then be resident beside it).
    const uint64_t rows_per_cta = (n + grid - 1) / grid, rowbytes64 = (uint64_t)vecs * 16;
    const uint64_t used = ((rows_per_cta + 15) / 16 + 1) * ((rowbytes64 + kPartBytes - 1) / kPartBytes);
    if (used < nstages) nstages = (uint32_t)(used < 2 ? 2 : used);
    const size_t smem = fixed + (size_t)nstages * kStageBytes;
    const bool xvec = aligned16(x) && k % 4 == 0;
    using Kernel = void (*)(const float*, const uint8_t*, const float*, const float*, const float*, float*, uint32_t, uint32_t, uint32_t,
                            uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t*, Prologue, bool);
    Kernel kernel = xvec ? gemv_imma_kernel<IS4, MR, true, 0> : gemv_imma_kernel<IS4, MR, false, 0>;
    if (kind != 0) {
        if (IS4 || MR != 1 || !xvec) return false;  // prologues: int8 weights, one aligned row of x
        if (kind == 1 && (!aligned16(pro.w) || (pro.res && !aligned16(pro.res)) || (pro.h_out && !aligned16(pro.h_out)))) return false;
        if constexpr (!IS4 && MR == 1) kernel = kind == 1 ? gemv_imma_kernel<false, 1, true, 1> : gemv_imma_kernel<false, 1, true, 2>;
    }
    GQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    launch_after(kernel, dim3(grid), dim3(kThreads), smem, s, x, reinterpret_cast<const uint8_t*>(q), scale, zero, bias, y, (uint32_t)k,
                 (uint32_t)n, vecs, groups, gshift, gblocks, nblocks, nstages, status, pro, early);
    return true;
}

}  // namespace

// Returns false when the shape is outside this kernel (more than two rows of
// x, an int4 group size that is not a multiple of 128, or a row of x too long
// for shared memory); the caller then takes the dp4a kernel.
bool launch_gemv_q4_imma(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                         const float* scale, const float* zero, const float* bias, uint64_t n, uint64_t group, float* y,
                         bool weights_settled) {
    if (group % 128 != 0 || m > 2) return false;
    return m == 1 ? run<true, 1>(s, sm_count, status, x, k, q, scale, zero, bias, n, group, y, weights_settled)
                  : run<true, 2>(s, sm_count, status, x, k, q, scale, zero, bias, n, group, y, weights_settled);
}

// y = W . f(x) for one row of x, f the prologue `kind` (math_common.cuh). False when the shape or alignment is not this kernel's.
bool launch_gemv_q8_imma_fused(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t k, const uint32_t* q,
                               const float* scale, const float* bias, uint64_t n, float* y, int kind, const Prologue& pro, bool weights_settled) {
    return run<false, 1>(s, sm_count, status, x, k, q, scale, nullptr, bias, n, 0, y, weights_settled, kind, pro);
}

bool launch_gemv_q8_imma(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                         const float* scale, const float* bias, uint64_t n, float* y, bool weights_settled) {
    if (m > 2) return false;
    return m == 1 ? run<false, 1>(s, sm_count, status, x, k, q, scale, nullptr, bias, n, 0, y, weights_settled)
                  : run<false, 2>(s, sm_count, status, x, k, q, scale, nullptr, bias, n, 0, y, weights_settled);
}

}  // namespace gq
