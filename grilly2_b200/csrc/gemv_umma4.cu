// Decode linear for int4 group-128 weights and 1 to 16 rows of x on the
// fifth-generation tensor cores (tcgen05.mma kind::i8, accumulators in tensor
// memory), ONE pass over the weight whatever the number of rows.
//
// Why it is shaped like this (measured on B200 with a loop of back-to-back
// instructions at full clock): a kind::i8 tcgen05.mma takes ~83 ns (~163
// cycles at 1965 MHz; ~175 when a fresh A tile streams from shared memory)
// whatever M (64 / 128) and N (<= 128) are. Time therefore goes with the
// NUMBER of instructions, so the operand that is streamed — the weight — is
// the 128-row A operand, each instruction eats 128 features x 32 bytes of it,
// and every row of x rides along for free as more columns of B (N = 16, 32 or
// 64). The same figure is this formulation's ceiling: two instructions per 4 KB
// of packed weight and SM is 3.6 TB/s over 148 SMs, 0.56 of the measured HBM
// rate, at ANY number of rows up to 16 — above what the warp-level kernel
// reaches in passes of four rows, below what it reaches at one to four rows,
// which is why AUTO keeps that kernel and this one is chosen with
// GQ_KERNEL_UMMA. Today it runs at about half its ceiling (14336 x 4096: ~26 us
// at 1 row, ~51 us at 16): stores to tensor memory do not overlap the
// multiplications they feed, and the drain warps' per-group work is latency
// bound.
//
// Arithmetic. The packed weight is never unpacked to one byte per level. Byte
// j of a group of 128 k holds levels 2j (low nibble) and 2j + 1 (high nibble):
// b = lo + 16 hi. With x in fixed point, X = rint(x 2^(26-e)), 2^e > max|x| of
// the group, and U_j = X[2j], V_j = X[2j+1] - 16 X[2j] (|V| < 2^31):
//     sum_k level_k X_k = sum_j b_j U_j + sum_j hi_j V_j .
// The first sum multiplies the RAW bytes exactly as they lie in HBM (u8); the
// second needs only the high nibbles, (w >> 4) & 0x0f0f0f0f. Four warps copy
// both to TENSOR MEMORY (tcgen05.st), the A operand of all four instructions. U and V are split in four signed base-256
// digits, the columns of B (column 4 r + d = digit d of row r of x); all four
// MMAs of a group (two 32-byte K slices, raw and high) accumulate into one
// int32 tile D[128 features][N] — exact. Eight warps drain D group by group
// (a thread owns a feature, i.e. a TMEM lane), recombine the digits in float32,
// and apply the group's scale and zero point as the reference does:
//     y[r][f] = sum_g  s[f][g] (sum_k level x) + (zero[f][g] - 8 s[f][g]) (sum_k x).
// The only approximation is X (2^-27 of the group's max |x|). A non-finite x
// gives NaN outputs.
//
// Work split. The digits of x for all of K do not fit shared memory beside the
// weight ring when there are many rows (16 rows x 4096 k = 256 KB), so K is cut
// in slices: CTA c works on slice c % slices for the feature tiles
// c / slices, + lanes, ... and keeps only its slice's digits (<= 64 KB). With
// more than one slice the partial sums go to a scratch buffer and the last CTA
// to finish a tile (a counter per tile, left at zero again) adds them in slice
// order — deterministic — and writes y. The host picks (slices, tile height) to
// minimise instructions per CTA (gemv_umma4_plan).
//
// Pipeline per CTA: warp 0 = TMA producer (one box of tile_rows x 128 bytes =
// two groups per stage, 128-byte swizzle, 4 to 8 stages); warp 1 = MMA issuer
// and TMEM owner; warps 4-7 move a stage's raw bytes and high nibbles to tensor
// memory (both A operands are read from there); warps 8-15 = drain. x is
// converted to digit tiles once per call by a small kernel of its own
// (x_digits_kernel), and each CTA bulk-copies its slice's tiles. Every wait is
// bounded (status word -> GQ_ERR).
//
// Replaces, for these shapes, the decode branch of Int4Weight::linear
// (crates/grilly-infer/src/quant4.rs:371-442, g2-linear-q4.glsl:43-111), which
// reads W twice at 16 rows; this reads it once.
// Algorithmic bytes per launch: packed weights + scales + zeros + x + y
// (+ bias). Bound: HBM bandwidth, with the tensor-core instruction count
// (K / 64 per 128 features) about level with it.
#include <type_traits>

#include "gq_internal.h"
#include "tc_common.cuh"

namespace gq {

namespace {

constexpr int kThreads = 512;
constexpr uint32_t kStageBytes = 128 * 128;  // 128 feature rows x 128 raw bytes (two groups)
constexpr int kMaxStages = 8;
constexpr int kMinStages = 4;
constexpr uint32_t kMaxTilesPerCta = 64;     // tiles whose partial sums a CTA may have outstanding when K is split
constexpr uint32_t kDBufs = 4;               // accumulator tiles in flight
constexpr uint32_t kACol0 = 256;             // TMEM columns 0-255: D ring; 256-447: three A tiles of 64 columns (32 raw, 32 high nibbles)
constexpr uint32_t kABufs = 3;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSmemBudget = 224 * 1024;
constexpr uint64_t kCounterBytes = 256 * 1024;  // the scratch begins with the tiles' arrival counters (always at the same place, so
                                                // that they are zero between launches whatever shapes share the scratch), then the partial sums

struct Plan {
    uint32_t slices, gps, tile_rows, tiles, lanes, grid;
    uint32_t nstages;      // ring depth: what the digits leave of shared memory
    uint32_t digit_bytes;  // bytes of one group's digit tile: NC rows of 128 bytes, or 8 rows when x has one or two rows (the
                           // descriptor then reads the same eight rows for every 8-column block of B: columns 8.. repeat 0..7)
};

// digits of one group's tile: row n (column of D) of 128 bytes — bytes 0-63 the digits of U, 64-127 of V — in 8-row
// 128-byte-swizzled atoms, as the tensor core's K-major descriptors read them.
__device__ __forceinline__ uint32_t digit_offset(uint32_t n, uint32_t o) {
    return (n >> 3) * 1024u + (n & 7u) * 128u + ((((o >> 4) ^ n) & 7u) << 4) + (o & 15u);
}

__device__ __forceinline__ void split_digits(int X, uint32_t (&word)[4], int shift) {
    const int d0 = (int)(int8_t)X;
    X = (X - d0) >> 8;
    const int d1 = (int)(int8_t)X;
    X = (X - d1) >> 8;
    const int d2 = (int)(int8_t)X;
    const int d3 = (X - d2) >> 8;
    word[0] |= ((uint32_t)d0 & 0xFFu) << shift, word[1] |= ((uint32_t)d1 & 0xFFu) << shift;
    word[2] |= ((uint32_t)d2 & 0xFFu) << shift, word[3] |= ((uint32_t)d3 & 0xFFu) << shift;
}

// x -> digit tiles, once per call: CTA = eight half-warps, a half-warp converts one (group, row) of 128 values, lane l the
// 8 values 8 l .. 8 l + 7. Output: groups tiles of `dbytes` in the layout above, then per group 16 (sum of x, 2^(e-26)) pairs.
__global__ void __launch_bounds__(128) x_digits_kernel(const float* __restrict__ x, uint32_t m, uint32_t k, uint32_t groups, uint32_t dbytes,
                                                       uint8_t* __restrict__ out) {
    GQ_GRID_DEP_SYNC();
    const uint32_t lane = threadIdx.x & 31, l = lane & 15u;
    const uint32_t item = (blockIdx.x * 128 + threadIdx.x) >> 4;
    if (item >= groups * m) return;  // uniform per half-warp; the shuffles below stay inside the half
    const uint32_t hmask = 0xFFFFu << (lane & 16u);
    uint8_t* digits = out;
    float2* xsinv = reinterpret_cast<float2*>(out + (size_t)groups * dbytes);
    {
          {
            const uint32_t gl = item / m, r = item - gl * m;
            const float* xr = x + (size_t)r * k + (size_t)gl * 128u + 8u * l;
            const float4 a = __ldg(reinterpret_cast<const float4*>(xr)), b = __ldg(reinterpret_cast<const float4*>(xr) + 1);
            const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            float amax = 0.0f;
            bool bad = false;
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i])), bad |= !(fabsf(v[i]) <= 3.402823466e+38f);
            if (bad) amax = __uint_as_float(0x7f800000u);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(hmask, amax, o));
            uint32_t e = __float_as_uint(amax) >> 23;
            float mult, inv;
            if (e == 255) {
                mult = 0.0f, inv = __uint_as_float(0x7fc00000u);
            } else if (amax == 0.0f) {
                mult = inv = 0.0f;
            } else {
                e = max(e, 32u);
                mult = __uint_as_float((279u - e) << 23);  // 2^(26 - e'), 2^e' > amax
                inv = __uint_as_float((e - 25u) << 23);    // 2^(e' - 26)
            }
            uint32_t uw[4] = {0u, 0u, 0u, 0u}, vw[4] = {0u, 0u, 0u, 0u};
            int sum_lo = 0, sum_hi = 0;  // X = lo + 65536 hi, lo a signed 16-bit number: both sums stay inside int32
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const int X0 = __float2int_rn(v[2 * p] * mult), X1 = __float2int_rn(v[2 * p + 1] * mult);
                const int l0 = (int)(int16_t)X0, l1 = (int)(int16_t)X1;
                sum_lo += l0 + l1, sum_hi += ((X0 - l0) >> 16) + ((X1 - l1) >> 16);
                split_digits(X0, uw, 8 * p);
                split_digits(X1 - 16 * X0, vw, 8 * p);
            }
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) {
                sum_lo += __shfl_xor_sync(hmask, sum_lo, o);
                sum_hi += __shfl_xor_sync(hmask, sum_hi, o);
            }
            uint8_t* tile = digits + (size_t)gl * dbytes;
#pragma unroll
            for (int d = 0; d < 4; ++d) {
                *reinterpret_cast<uint32_t*>(tile + digit_offset(4 * r + d, 4 * l)) = uw[d];
                *reinterpret_cast<uint32_t*>(tile + digit_offset(4 * r + d, 64 + 4 * l)) = vw[d];
            }
            if (l == 0) xsinv[gl * 16 + r] = make_float2(__fmaf_rn((float)sum_hi, 65536.0f, (float)sum_lo) * inv, inv);
          }
    }
}

template <int NC>
__global__ void __launch_bounds__(kThreads, 1)
    gemv_q4_umma_kernel(const __grid_constant__ CUtensorMap wmap, const uint8_t* __restrict__ xdigits, const float* __restrict__ scale,
                        const float* __restrict__ zero, const float* __restrict__ bias, float* __restrict__ y, float* __restrict__ partials,
                        uint32_t* __restrict__ counters, uint32_t m, uint32_t k, uint32_t n, uint32_t groups, Plan plan, uint32_t* status) {
    extern __shared__ uint8_t smem_unaligned[];
    uint8_t* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    const uint32_t nstages = plan.nstages, dbytes = plan.digit_bytes;
    const uint32_t b_sbo = dbytes == 1024u ? 0u : 1024u;  // stride between 8-column blocks of B (0: all blocks read the same eight rows)
    uint8_t* ring = smem;                                          // nstages x 16 KB
    uint8_t* digits = ring + (size_t)nstages * kStageBytes;        // gps tiles of dbytes
    float2* xsinv = reinterpret_cast<float2*>(digits + (size_t)plan.gps * dbytes);  // [gps][16]: (sum of x, 2^(e-26)) per group and row
    uint64_t* full = reinterpret_cast<uint64_t*>(xsinv + (size_t)plan.gps * 16);
    uint64_t* empty = full + kMaxStages;
    uint64_t* afull = empty + kMaxStages;   // [4] an A tile is in tensor memory
    uint64_t* aempty = afull + 4;        // [4] ... and has been multiplied
    uint64_t* dfull = aempty + 4;        // [kDBufs] an accumulator is complete
    uint64_t* dempty = dfull + kDBufs;   // [kDBufs] ... and has been read out
    uint64_t* dgfull = dempty + kDBufs;  // the slice's digit tiles have landed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dgfull + 1);
    volatile uint32_t* failed = tmem_slot + 1;
    uint32_t* last_flags = tmem_slot + 2;  // [kMaxTilesPerCta] K split: was this CTA the last to finish the tile

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t slice = blockIdx.x % plan.slices, tlane = blockIdx.x / plan.slices;
    const uint32_t g_begin = slice * plan.gps, g_end = min(groups, g_begin + plan.gps);
    const uint32_t ngroups = g_end > g_begin ? g_end - g_begin : 0u;
    const uint32_t nstage_tile = (ngroups + 1) >> 1;
    constexpr uint32_t kDrainWarps = NC == 64 ? 8 : 4;

    GQ_GRID_DEP_SYNC();
    if (tid == 0) {
        for (uint32_t s = 0; s < nstages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 4);  // the four warps that read a stage out
        }
        for (uint32_t a = 0; a < kABufs; ++a) {
            mbar_init(afull + a, 4);
            mbar_init(aempty + a, 1);
        }
        for (uint32_t d = 0; d < kDBufs; ++d) {
            mbar_init(dfull + d, 1);
            mbar_init(dempty + d, kDrainWarps);
        }
        mbar_init(dgfull, 1);
        *failed = 0;
        mbar_fence_init();
        tma_prefetch_map(&wmap);
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
    __syncthreads();

    // ── the producer fills the ring once before anything else happens (the weights do not depend on x) ──
    uint32_t ps = 0, pround = 0, ptile = tlane, pi = 0;  // producer position (warp 0, lane 0)
    auto produce_one = [&]() -> bool {  // requests the next stage; false when nothing is left or a wait gave up
        if (!ngroups || ptile >= plan.tiles) return false;
        if (pround && !mbar_wait(empty + ps, (pround - 1) & 1, failed, status, kStatusEmptyWaitTimedOut)) return false;
        if (pi == 0) {
            // The tile's scales and zero points (contiguous: tile_rows x groups floats each) are asked into L2 a ring's depth
            // before the drain warps read them: under a full weight stream a miss costs them ~2.7 us.
            const size_t first = (size_t)ptile * plan.tile_rows * groups * 4, last = min((size_t)(ptile + 1) * plan.tile_rows, (size_t)n) * groups * 4;
            const size_t lo = first & ~(size_t)15, bytes = (last - lo) & ~(size_t)15;
            if (bytes) {
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<const uint8_t*>(scale) + lo), "r"((uint32_t)bytes) : "memory");
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<const uint8_t*>(zero) + lo), "r"((uint32_t)bytes) : "memory");
            }
        }
        mbar_arrive_expect_tx(full + ps, plan.tile_rows * 128u);
        tma_load_2d(ring + (size_t)ps * kStageBytes, &wmap, (int32_t)((g_begin + 2 * pi) * 64u), (int32_t)(ptile * plan.tile_rows), full + ps);
        if (++pi == nstage_tile) pi = 0, ptile += plan.lanes;
        if (++ps == nstages) ps = 0, ++pround;
        return true;
    };
    if (warp == 0) {
        if (lane == 0)
            for (uint32_t i = 0; i < nstages; ++i)
                if (!produce_one()) break;
    }
    if (warp == 0 && lane == 0 && ngroups) {
        // the slice's digit tiles and (sum, 2^(e-26)) pairs, as the conversion kernel left them in global memory: bulk copies
        const uint32_t dig_bytes = ngroups * dbytes, xs_bytes = ngroups * 128u;
        mbar_arrive_expect_tx(dgfull, dig_bytes + xs_bytes);
        for (uint32_t off = 0; off < dig_bytes; off += 32768u)
            bulk_load(digits + off, xdigits + (size_t)g_begin * dbytes + off, min(32768u, dig_bytes - off), dgfull);
        bulk_load(xsinv, xdigits + (size_t)groups * dbytes + (size_t)g_begin * 128u, xs_bytes, dgfull);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0)
            while (produce_one()) {
            }
    } else if (warp == 1) {
        if (lane == 0 && ngroups) {
            // Both A operands come from tensor memory (the raw bytes and the high nibbles, written there by warps 4-7): a
            // kind::i8 instruction whose A streams from shared memory took ~175 cycles in a loop of fresh tiles, ~97 with A
            // in tensor memory.
            constexpr uint32_t idesc = umma_idesc(2, 0, 1, 128, NC);  // s32 accumulate, u8 weights x s8 digits
            uint32_t it = 0, dcount = 0;
            bool ok = mbar_wait(dgfull, 0, failed, status, kStatusFullWaitTimedOut);
            for (uint32_t tile = tlane; tile < plan.tiles && ok; tile += plan.lanes) {
                for (uint32_t i = 0; i < nstage_tile && ok; ++i, ++it) {
                    const uint32_t ng = min(2u, ngroups - 2 * i), abuf = it % kABufs;
                    ok = mbar_wait(afull + abuf, (it / kABufs) & 1, failed, status, kStatusMmaWaitTimedOut);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t a_raw = tmem + kACol0 + abuf * 64, a_hi = a_raw + 32;
                    for (uint32_t gi = 0; gi < ng && ok; ++gi) {
                        const uint32_t dc = dcount + gi, db = dc % kDBufs;
                        if (dc >= kDBufs) ok = mbar_wait(dempty + db, (dc / kDBufs - 1) & 1, failed, status, kStatusMmaWaitTimedOut);
                        if (!ok) break;
                        tc_fence_after_sync();
                        const uint32_t x_addr = smem_u32(digits + (size_t)(2 * i + gi) * dbytes);
#pragma unroll
                        for (uint32_t h = 0; h < 2; ++h) {  // raw bytes x digits of U, high nibbles x digits of V
                            umma_i8_ts(tmem + db * NC, a_raw + (2 * gi + h) * 8, umma_desc_k128(x_addr + 32 * h, b_sbo), idesc, h != 0);
                            umma_i8_ts(tmem + db * NC, a_hi + (2 * gi + h) * 8, umma_desc_k128(x_addr + 64 + 32 * h, b_sbo), idesc, true);
                        }
                        umma_commit(dfull + db);
                    }
                    if (!ok) break;
                    umma_commit(aempty + abuf);
                    dcount += ng;
                }
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ── the stage's raw bytes and high nibbles -> tensor memory: thread = one feature row = one TMEM lane ──
        const uint32_t sub = warp & 3u, row = 32 * sub + lane;
        uint32_t s = 0, round = 0, it = 0;
        bool ok = ngroups != 0;
        for (uint32_t tile = tlane; tile < plan.tiles && ok; tile += plan.lanes) {
            for (uint32_t i = 0; i < nstage_tile && ok; ++i, ++it) {
                const uint32_t abuf = it % kABufs;
                if (lane == 0) {
                    ok = mbar_wait(full + s, round & 1, failed, status, kStatusFullWaitTimedOut);
                    if (ok && it >= kABufs) ok = mbar_wait(aempty + abuf, (it / kABufs - 1) & 1, failed, status, kStatusMmaWaitTimedOut);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                const uint8_t* src = ring + (size_t)s * kStageBytes + row * 128u;
                uint32_t raw[32], hi[32];  // a store to tensor memory reads its registers until tcgen05.wait::st: two arrays
#pragma unroll
                for (uint32_t c = 0; c < 8; ++c) {
                    const uint4 w = *reinterpret_cast<const uint4*>(src + ((c ^ (row & 7u)) << 4));
                    raw[4 * c] = w.x, raw[4 * c + 1] = w.y, raw[4 * c + 2] = w.z, raw[4 * c + 3] = w.w;
                }
#pragma unroll
                for (uint32_t c = 0; c < 32; ++c) hi[c] = (raw[c] >> 4) & 0x0f0f0f0fu;
                tc_fence_after_sync();
                tmem_st32(tmem_addr(tmem, 32 * sub, kACol0 + abuf * 64), raw);
                tmem_st32(tmem_addr(tmem, 32 * sub, kACol0 + abuf * 64 + 32), hi);
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(afull + abuf);
                    mbar_arrive(empty + s);  // the stage has been read: the producer may refill it
                }
                if (++s == nstages) s = 0, ++round;
            }
        }
    } else if (warp >= 8 && warp < 8 + kDrainWarps) {
        // ── drain: thread = one feature; per group read the int32 digit sums, recombine, scale, accumulate ──
        constexpr uint32_t CW = NC < 32 ? NC : 32;  // columns this warp reads: rows r0 .. r0 + CW / 4 - 1 of x
        constexpr uint32_t RW = CW / 4;
        const uint32_t sub = warp & 3u, half = (warp - 8) >> 2, r0 = half * 8, f = 32 * sub + lane;
        bool ok = ngroups != 0;
        if (ok && lane == 0) ok = mbar_wait(dgfull, 0, failed, status, kStatusFullWaitTimedOut);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        const uint32_t my_tiles_d = tlane < plan.tiles ? (plan.tiles - tlane + plan.lanes - 1) / plan.lanes : 0u;
        const uint32_t total = my_tiles_d * ngroups;  // the CTA's groups, tile after tile: one accumulator tile each
        const bool frow = f < plan.tile_rows;
        // scale and zero point of flat group g for this thread's feature
        auto sz_ptr = [&](uint32_t g, const float* base) {
            const uint32_t tl = g / ngroups, gl = g - tl * ngroups, feature = (tlane + tl * plan.lanes) * plan.tile_rows + f;
            return base + (size_t)((frow && feature < n) ? feature : 0) * groups + g_begin + gl;
        };
        // The accumulator is read 16 columns (four rows of x) at a time: step q = group q / kParts, columns 16 (q % kParts).
        constexpr uint32_t kParts = CW / 16;
        const uint32_t steps = total * kParts;
        // waits for the step's accumulator (at its first part) and requests the columns (the registers are valid after finish_load)
        auto wait_and_load = [&](uint32_t q, uint32_t (&d)[16]) {
            const uint32_t g = q / kParts, part = q % kParts, db = g % kDBufs;
            if (part == 0) {
                if (lane == 0 && ok) ok = mbar_wait(dfull + db, (g / kDBufs) & 1, failed, status, kStatusMmaWaitTimedOut);
                ok = __shfl_sync(0xffffffffu, ok, 0);
            }
            if (!ok) return;
            tc_fence_after_sync();
            tmem_ld16(tmem_addr(tmem, 32 * sub, db * NC + half * 32 + part * 16), d);
        };
        auto finish_load = [&](uint32_t q, uint32_t (&d)[16]) {
            if (!ok) return;
            tmem_wait_ld();
#pragma unroll
            for (uint32_t i = 0; i < 16; ++i) asm volatile("" : "+r"(d[i]));  // nothing reads the registers before the wait above
            if (q % kParts == kParts - 1) {  // the whole accumulator has been read: the tensor core may overwrite it
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(dempty + (q / kParts) % kDBufs);
            }
        };
        float acc[RW];
        float s_cur[4], z_cur[4], s_nxt[4], z_nxt[4];
        auto ldg_pinned = [](const float* p) {  // a load the compiler cannot sink to its use: it is requested HERE
            float v;
            asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
            return v;
        };
        auto fetch_sz = [&](uint32_t g0, float (&sv)[4], float (&zv)[4]) {
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
                const bool have = g0 + j < total;
                sv[j] = have ? ldg_pinned(sz_ptr(g0 + j, scale)) : 0.0f;
                zv[j] = have ? ldg_pinned(sz_ptr(g0 + j, zero)) : 0.0f;
            }
        };
        auto math = [&](uint32_t q, const uint32_t (&d)[16], float s, float z, auto part_c) {
            constexpr uint32_t PART = decltype(part_c)::value;
            const uint32_t g = q / kParts, tl = g / ngroups, gl = g - tl * ngroups;
            if (gl == 0) {
#pragma unroll
                for (uint32_t r = 0; r < 4; ++r) acc[PART * 4 + r] = 0.0f;
            }
            const float zm = __fmaf_rn(-8.0f, s, z);
            const float2* xi = xsinv + gl * 16 + r0 + PART * 4;
#pragma unroll
            for (uint32_t r = 0; r < 4; ++r) {
                if (r0 + PART * 4 + r < m) {
                    // |digit sum| < 2^22: 12582912 + c is exact in float32, so two full-rate instructions convert it
                    const float f0 = __int_as_float((int)d[4 * r] + 0x4B400000) - 12582912.0f;
                    const float f1 = __int_as_float((int)d[4 * r + 1] + 0x4B400000) - 12582912.0f;
                    const float f2 = __int_as_float((int)d[4 * r + 2] + 0x4B400000) - 12582912.0f;
                    const float f3 = __int_as_float((int)d[4 * r + 3] + 0x4B400000) - 12582912.0f;
                    const float t = __fmaf_rn(__fmaf_rn(__fmaf_rn(f3, 256.0f, f2), 256.0f, f1), 256.0f, f0);
                    const float2 c = xi[r];  // (sum of x over the group, 2^(e-26))
                    acc[PART * 4 + r] = __fmaf_rn(zm, c.x, __fmaf_rn(s, t * c.y, acc[PART * 4 + r]));
                }
            }
            if (gl == ngroups - 1 && PART == kParts - 1) {  // the tile's results
                const uint32_t feature = (tlane + tl * plan.lanes) * plan.tile_rows + f;
                if (frow && feature < n && ok) {
                    if (plan.slices == 1) {
                        const float bs = bias ? bias[feature] : 0.0f;
#pragma unroll
                        for (uint32_t r = 0; r < RW; ++r)
                            if (r0 + r < m) y[(size_t)(r0 + r) * n + feature] = bias ? __fadd_rn(acc[r], bs) : acc[r];
                    } else {  // K is split: this slice's partial sums; they are added up once the CTA has done all its tiles
#pragma unroll
                        for (uint32_t r = 0; r < RW; ++r)
                            if (r0 + r < m) __stcg(partials + ((size_t)slice * m + r0 + r) * n + feature, acc[r]);
                    }
                }
            }
        };
        // Two register sets of 16: while one is worked on, the next columns are already on their way out of tensor memory;
        // and the scales of the next four groups are requested while the current four are in use.
        uint32_t da[16], dbuf[16];
        using P0 = std::integral_constant<uint32_t, 0>;
        using P1 = std::integral_constant<uint32_t, kParts - 1>;  // odd steps: part 1 when a group has two parts, else part 0
        if (steps) {
            fetch_sz(0, s_cur, z_cur);
            wait_and_load(0, da);
            finish_load(0, da);
        }
        constexpr uint32_t kStepsPerChunk = 4 * kParts;  // four groups
        for (uint32_t q = 0; q < steps && ok; q += kStepsPerChunk) {
            fetch_sz(q / kParts + 4, s_nxt, z_nxt);
#pragma unroll
            for (uint32_t j = 0; j < kStepsPerChunk; j += 2) {
                const uint32_t q0 = q + j;
                if (q0 >= steps || !ok) break;
                if (q0 + 1 < steps) wait_and_load(q0 + 1, dbuf);
                math(q0, da, s_cur[j / kParts], z_cur[j / kParts], P0{});
                if (q0 + 1 < steps) finish_load(q0 + 1, dbuf);
                if (q0 + 2 < steps) wait_and_load(q0 + 2, da);
                if (q0 + 1 < steps && ok) math(q0 + 1, dbuf, s_cur[(j + 1) / kParts], z_cur[(j + 1) / kParts], P1{});
                if (q0 + 2 < steps) finish_load(q0 + 2, da);
            }
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) s_cur[j] = s_nxt[j], z_cur[j] = z_nxt[j];
        }
        if (plan.slices > 1) {
            // One fence and one round of counters for all the CTA's tiles (a round per tile cost ~4 us each). The last CTA to
            // arrive at a tile adds the slices' partial sums in slice order (deterministic), writes y and leaves the counter at
            // zero for the next launch.
            __threadfence();
            named_barrier_sync(5, kDrainWarps * 32);
            const uint32_t dt = tid - 8 * 32, my_tiles = tlane < plan.tiles ? (plan.tiles - tlane + plan.lanes - 1) / plan.lanes : 0u;
            if (dt < my_tiles) {
                const uint32_t tile = tlane + dt * plan.lanes;
                const uint32_t old = atomicAdd(counters + tile, 1u);
                last_flags[dt] = old == plan.slices - 1;
                if (old == plan.slices - 1) counters[tile] = 0;
            }
            named_barrier_sync(5, kDrainWarps * 32);
            __threadfence();
            for (uint32_t j = 0; j < my_tiles; ++j) {
                if (!last_flags[j]) continue;
                const uint32_t feature = (tlane + j * plan.lanes) * plan.tile_rows + f;
                if (!(f < plan.tile_rows && feature < n && ok)) continue;
                const float bs = bias ? bias[feature] : 0.0f;
#pragma unroll
                for (uint32_t r = 0; r < RW; ++r) {
                    if (r0 + r < m) {
                        float tot = 0.0f;  // eight slices' values are requested before the first is used
#pragma unroll
                        for (uint32_t s0 = 0; s0 < 16; s0 += 8) {
                            if (s0 >= plan.slices) break;
                            float part[8];
#pragma unroll
                            for (uint32_t sl = 0; sl < 8; ++sl) part[sl] = s0 + sl < plan.slices ? __ldcg(partials + ((size_t)(s0 + sl) * m + r0 + r) * n + feature) : 0.0f;
#pragma unroll
                            for (uint32_t sl = 0; sl < 8; ++sl)
                                if (s0 + sl < plan.slices) tot = s0 + sl == 0 ? part[0] : __fadd_rn(tot, part[sl]);
                        }
                        y[(size_t)(r0 + r) * n + feature] = bias ? __fadd_rn(tot, bs) : tot;
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

// (slices, tile height) that minimise the time of the busiest CTA: its tensor-core instructions, plus what splitting K
// costs (one round of fences and counters at the end, and the partial sums' traffic).
Plan make_plan(uint64_t m, uint64_t n, uint64_t groups, uint32_t nc, int sm_count) {
    const uint32_t digit_bytes = m <= 2 ? 1024u : nc * 128u;
    const uint32_t fixed = 1024 + (2 * kMaxStages + 9 + 2 * kDBufs) * 8 + 16 + kMaxTilesPerCta * 4 + 64;
    Plan best{};
    double best_cost = 1e30;
    const uint32_t tiles_min = (uint32_t)((n + 127) / 128);
    for (uint32_t ks = 1; ks <= 16 && ks <= groups; ++ks) {
        const uint32_t gps = (uint32_t)((groups + ks - 1) / ks);
        const uint64_t resident = (uint64_t)gps * (digit_bytes + 128) + fixed;
        if (resident + (uint64_t)kMinStages * kStageBytes > kSmemBudget) continue;
        uint32_t nstages = (uint32_t)((kSmemBudget - resident) / kStageBytes);
        if (nstages > (uint32_t)kMaxStages) nstages = kMaxStages;
        const uint32_t slices = (uint32_t)((groups + gps - 1) / gps);
        if (slices > (uint32_t)sm_count || slices > 16) continue;
        const uint32_t lanes_max = (uint32_t)sm_count / slices;
        for (uint32_t t = tiles_min; t <= tiles_min + 2 * (uint32_t)sm_count && t <= n; ++t) {
            const uint32_t tile_rows = (uint32_t)((n + t - 1) / t);
            const uint32_t tiles = (uint32_t)((n + tile_rows - 1) / tile_rows);
            const uint32_t lanes = tiles < lanes_max ? tiles : lanes_max;
            const uint32_t rounds = (tiles + lanes - 1) / lanes;
            if (slices > 1 && rounds > kMaxTilesPerCta) continue;
            // cycles: 4 instructions of ~96 cycles per group and tile (a stage holds two groups); when K is split, ~4 us for the
            // closing round and the partial sums' traffic at ~22 bytes per cycle per SM
            double cost = (double)rounds * ((gps + 1) / 2 * 2) * 4.0 * 96.0 + (nstages < 6 ? 300.0 * (6 - nstages) : 0.0);
            if (slices > 1) cost += 8000.0 + (double)slices * m * n * 8.0 / (sm_count * 22.0);
            if (cost < best_cost) best_cost = cost, best = Plan{slices, gps, tile_rows, tiles, lanes, lanes * slices, nstages, digit_bytes};
        }
    }
    return best;
}

}  // namespace

static uint64_t digits_region_bytes(uint64_t groups, uint32_t digit_bytes) { return (groups * (digit_bytes + 128ull) + 1023) / 1024 * 1024; }

uint64_t gemv_q4_umma_scratch_bytes(uint64_t m, uint64_t k, uint64_t n, int sm_count) {
    if (m < 1 || m > 16 || k == 0 || k % 128 || n == 0) return 0;
    const uint32_t nc = m <= 4 ? 16 : m <= 8 ? 32 : 64;
    const Plan p = make_plan(m, n, k / 128, nc, sm_count);
    if (p.grid == 0) return 0;
    if ((uint64_t)p.tiles * 4 > kCounterBytes) return 0;
    return kCounterBytes + digits_region_bytes(k / 128, p.digit_bytes) + (p.slices > 1 ? (uint64_t)p.slices * m * n * 4 : 0);
}

// Returns false when the shape is not this kernel's: group_size 128, in_features a multiple of 128, 1 to 16 rows of x,
// 16-byte aligned x and weights. `scratch` holds gemv_q4_umma_scratch_bytes bytes whose first 256 KB (the counters) are zero
// between launches. Two launches: x -> digit tiles (tiny), then the linear, which starts streaming weights while the first runs.
bool launch_gemv_q4_umma(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                         const float* scale, const float* zero, const float* bias, uint64_t n, uint64_t group, float* y, void* scratch) {
    if (m < 1 || m > 16 || group != 128 || k == 0 || k % 128 || n == 0 || n > 0x7fffffffull || k > (1ull << 24)) return false;
    if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(x)) & 15) != 0) return false;
    const uint32_t nc = m <= 4 ? 16 : m <= 8 ? 32 : 64;
    const uint64_t groups = k / 128, row_bytes = k / 2;
    const Plan p = make_plan(m, n, groups, nc, sm_count);
    if (p.grid == 0 || (uint64_t)p.tiles * 4 > kCounterBytes) return false;
    uint32_t* counters = reinterpret_cast<uint32_t*>(scratch);
    uint8_t* xdigits = reinterpret_cast<uint8_t*>(scratch) + kCounterBytes;
    float* partials = reinterpret_cast<float*>(xdigits + digits_region_bytes(groups, p.digit_bytes));
    const CUtensorMap wmap = make_tensor_map_2d(q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, row_bytes, n, row_bytes, 128, p.tile_rows, Swizzle::B128);
    const size_t smem = 1024 + (size_t)p.nstages * kStageBytes + (size_t)p.gps * (p.digit_bytes + 128) + (2 * kMaxStages + 9 + 2 * kDBufs) * 8 + 16 +
                        kMaxTilesPerCta * 4 + 64;
    launch_after(x_digits_kernel, dim3((uint32_t)((groups * m + 7) / 8)), dim3(128), 0, s, x, (uint32_t)m, (uint32_t)k, (uint32_t)groups, p.digit_bytes, xdigits);
    auto go = [&](auto kernel) {
        GQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        launch_after(kernel, dim3(p.grid), dim3(kThreads), smem, s, wmap, (const uint8_t*)xdigits, scale, zero, bias, y, partials, counters, (uint32_t)m,
                     (uint32_t)k, (uint32_t)n, (uint32_t)groups, p, status);
    };
    if (nc == 16) go(gemv_q4_umma_kernel<16>);
    else if (nc == 32) go(gemv_q4_umma_kernel<32>);
    else go(gemv_q4_umma_kernel<64>);
    return true;
}

}  // namespace gq
