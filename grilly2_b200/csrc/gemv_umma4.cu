// Decode linear for int4 group-128 weights and 1 to 16 rows of x on the
// fifth-generation tensor cores (tcgen05.mma kind::i8, accumulators in tensor
// memory), ONE pass over the weight whatever the number of rows.
//
// Two kernels share the arithmetic, the digit tiles of x and the nibble warps. The first (gemv_q4_umma_kernel,
// described here) keeps the rows of x on the lanes of tensor memory and the weight as the wide B operand; the
// second (gemv_q4_lanes_kernel, further down, with its own account) exchanges the operands so that a read-out thread
// owns one output feature. The second is the faster on every shape measured and is what GQ_KERNEL_AUTO runs up to
// in_features 16384.
//
// Why it is shaped like this (measured on B200 with loops of back-to-back
// instructions): a kind::i8 tcgen05.mma takes ~83 ns for any N up to 64, ~92 ns
// at N = 128 and ~133 ns at N = 256 (M = 64; K = 32 bytes). Time goes with the
// NUMBER of instructions far more than with their width, so the operand that is
// streamed — the weight — is the WIDE one: it is the B operand, up to 256
// features x 32 bytes per instruction, read by the tensor core straight from the
// shared memory the TMA wrote it to, and the rows of x are the 64-row A operand
// (16 rows x 4 digit planes). Two instructions per 8 KB of packed weight and SM
// = 4.5 TB/s over 148 SMs, 0.69 of the measured HBM rate, at ANY number of rows
// up to 16. (A first version streamed the weight as the 128-row A operand out
// of tensor memory: half the bytes per instruction, and the stores to tensor
// memory did not overlap the multiplications they fed.)
//
// Arithmetic. The packed weight is never unpacked to one byte per level. Byte
// j of a group of 128 k holds levels 2j (low nibble) and 2j + 1 (high nibble):
// b = lo + 16 hi. With x in fixed point, X = rint(x 2^(26-e)), 2^e > max|x| of
// the group, and U_j = X[2j], V_j = X[2j+1] - 16 X[2j] (|V| < 2^31):
//     sum_k level_k X_k = sum_j b_j U_j + sum_j hi_j V_j .
// The first sum multiplies the RAW bytes exactly as they lie in HBM (u8); the
// second needs only the high nibbles, (w >> 4) & 0x0f0f0f0f, which four warps
// write to a second shared-memory buffer (a thread = two feature rows; the same
// threads bring the stage's scales and zero points). U and V are split in four
// signed base-256 digits, the rows of A (one row per row of x and digit); all
// four MMAs of a group (two 32-byte K slices, raw and high) accumulate into one
// int32 tile D[64][features] — exact. An M = 64 accumulator occupies lanes 0-15
// of each 32-lane quarter of tensor memory, so the two groups of a stage sit in
// the lower and upper half-lanes of the same columns, and sixteen warps drain
// both with 16-lane loads (every thread busy). The rows are ordered so that a
// thread receives digits 2 p and 2 p + 1 of one row of x: it joins them as
// integers (D + 256 D'), converts once, and applies the group's scale and zero
// point as the reference does:
//     y[r][f] = sum_g  s[f][g] (sum_k level x) + (zero[f][g] - 8 s[f][g]) (sum_k x).
// The only approximation is X (2^-27 of the group's max |x|). A non-finite x
// gives NaN outputs.
//
// Work split. The digits of x for all of K do not fit shared memory beside the
// weight ring when there are many rows (16 rows x 4096 k = 256 KB), so K is cut
// in slices: CTA c works on slice c % slices for the feature tiles c / slices,
// + lanes, ... and converts and keeps only its slice of x. With more than one
// slice the partial sums go to a scratch buffer and a second, small kernel adds
// them in slice order (deterministic) and adds the bias. The host picks
// (slices, tile width) to minimise the busiest CTA's time (make_plan).
//
// Pipeline per CTA (704 threads): warp 0 = TMA producer (one box of tile_rows x
// 128 bytes = two groups per stage, 128-byte swizzle); warp 1 = MMA issuer and
// TMEM owner; warps 2-5 = high nibbles + scales, a stage at a time; warps
// 6-21 = drain. Every wait is bounded (status word -> GQ_ERR).
//
// Where the time goes today (per-warp clock stamps, 14336 x 4096 at 16 rows): a stage's eight instructions take
// ~0.76 us, its drain ~1.4 us, and the drain is what the stages queue behind. Taking the high-nibble instructions out
// leaves the drain as slow, so it is not tensor memory the two compete for; its loads from tensor memory return in
// ~0.1 us; replacing the integer-to-float conversions by exact magic-number arithmetic made it slower. What the 16
// warps do share with the four nibble warps is the shared-memory pipe: a 16-byte load costs four wavefronts however
// many lanes read the same address, so the (s, s', z - 8 s, z' - 8 s') of a column pair costs every warp four
// wavefronts per block of eight columns — ~1000 wavefronts per stage for the drain, ~500 for the nibbles,
// ~550 more for the tensor core's operand reads and ~200 for the TMA's writes: ~2300 cycles = 1.2 us of the pipe per
// stage. While the nibble warps work on the stages ahead, a stage takes ~2.0 us at 16 rows; once they have finished
// the CTA's last tile, the same drain takes ~1.2 us. With one row of x only the four drain warps of the first lane
// quarter have rows, all four on one scheduler, and a stage still takes ~1.4 us: the read-out is then a chain of
// waits in those warps, not a pipe that is full.
// Not the way the weight arrives: with the TMA boxes (128 bytes from each of the tile's rows, K / 2 bytes apart)
// replaced by contiguous copies of the same size (wrong bytes, timing only) a call took 6 % less, and asking each
// row's K slice into L2 ahead of the boxes (cp.async.bulk.prefetch.L2) made it slower. Nor a branch between the
// drain's column blocks: without it (and 28 bytes of spills) a call took 5 % more.
//
// Replaces, for these shapes, the decode branch of Int4Weight::linear
// (crates/grilly-infer/src/quant4.rs:371-442, g2-linear-q4.glsl:43-111), which
// reads W twice at 16 rows; this reads it once.
// Algorithmic bytes per launch: packed weights + scales + zeros + x + y
// (+ bias). Bound: HBM bandwidth, with the tensor-core instruction count
// (K / 64 per 256 features) just above it.
#include <type_traits>

#include "gq_internal.h"
#include "tc_common.cuh"

namespace gq {

namespace {

constexpr int kThreads = 704;  // 88 registers per thread
constexpr uint32_t kFirstNibbleWarp = 2, kNibbleWarps = 4, kFirstDrainWarp = 6, kDrainWarps = 16;
constexpr uint32_t kTileMax = 256;   // features per tile = N of the instruction
constexpr uint32_t kSzSlots = 4;     // stages whose scales are in shared memory at a time
constexpr int kMaxStages = 4;
constexpr int kMinStages = 2;
constexpr uint32_t kTmemCols = 512;  // two accumulators of 256 columns
constexpr uint32_t kSmemBudget = 227 * 1024;
constexpr uint32_t kMaxTileStages = 16;  // stages of a tile (pairs of groups of a K slice)
constexpr uint32_t kBarrierBytes = (2 * kMaxStages + 4 + 4 + kMaxTileStages) * 8 + 16;

struct Plan {
    uint32_t slices, gps, tile_rows, tiles, lanes, grid;
    uint32_t nstages;   // ring depth: what the digits leave of shared memory
    uint32_t rows_pad;  // digit rows kept per group: 16, 32 or 64 (4 per row of x); the instruction reads 64, the rest is whatever follows
};

// Row of A (and of the accumulator) that holds digit d of row r of x: rows 16 s .. 16 s + 15 go to quarter s of tensor
// memory, and a 16-lane load hands a thread rows j and j + 8 of it, so digit pairs (0, 1) and (2, 3) sit 8 rows apart.
__device__ __forceinline__ uint32_t digit_row(uint32_t r, uint32_t d) { return 16u * (r >> 2) + 2u * (r & 3u) + (d >> 1) + 8u * (d & 1u); }

// digits of one group's tile: row n of 128 bytes — bytes 0-63 the digits of U, 64-127 of V — in 8-row
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

// One (group, row) of x = 128 values -> its rows of the group's digit tile and its (sum of x, 2^(e-26)) pair; a half-warp
// does it, lane l the 8 values 8 l .. 8 l + 7 (already loaded: a, b).
__device__ __forceinline__ void convert_item(const float4 a, const float4 b, uint32_t l, uint32_t hmask, uint8_t* tile, uint32_t r, float2* xs_out) {
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
#pragma unroll
    for (int d = 0; d < 4; ++d) {
        *reinterpret_cast<uint32_t*>(tile + digit_offset(digit_row(r, d), 4 * l)) = uw[d];
        *reinterpret_cast<uint32_t*>(tile + digit_offset(digit_row(r, d), 64 + 4 * l)) = vw[d];
    }
    if (l == 0) *xs_out = make_float2(__fmaf_rn((float)sum_hi, 65536.0f, (float)sum_lo) * inv, inv);
}

// x -> digit tiles, once per call: CTA = eight half-warps, a half-warp converts one (group, row) of 128 values. Output:
// `groups` tiles of rows_pad x 128 bytes in the layout above (the rows of x the call does not have are zero), then per
// group 16 (sum of x, 2^(e-26)) pairs (zero for rows m .. 15).
__global__ void __launch_bounds__(128) x_digits_kernel(const float* __restrict__ x, uint32_t m, uint32_t k, uint32_t groups, uint32_t rows_pad,
                                                       uint8_t* __restrict__ out) {
    GQ_GRID_DEP_SYNC();
    const uint32_t lane = threadIdx.x & 31, l = lane & 15u, hmask = 0xFFFFu << (lane & 16u);
    const uint32_t item = (blockIdx.x * 128 + threadIdx.x) >> 4, rows = rows_pad >> 2;
    if (item >= groups * rows) return;  // uniform per half-warp
    const uint32_t gl = item / rows, r = item - gl * rows;
    uint8_t* tile = out + (size_t)gl * rows_pad * 128u;
    float2* xsinv = reinterpret_cast<float2*>(out + (size_t)groups * rows_pad * 128u) + gl * 16;
    if (r >= m) {
#pragma unroll
        for (uint32_t d = 0; d < 4; ++d) {
            *reinterpret_cast<uint32_t*>(tile + digit_offset(digit_row(r, d), 4 * l)) = 0u;
            *reinterpret_cast<uint32_t*>(tile + digit_offset(digit_row(r, d), 64 + 4 * l)) = 0u;
        }
        if (l == 0) xsinv[r] = make_float2(0.0f, 0.0f);
        if (r == rows - 1 && l < 16 - rows) xsinv[rows + l] = make_float2(0.0f, 0.0f);  // the pairs of rows beyond rows_pad / 4
        return;
    }
    const float4* p = reinterpret_cast<const float4*>(x + (size_t)r * k + (size_t)gl * 128u + 8u * l);
    convert_item(__ldg(p), __ldg(p + 1), l, hmask, tile, r, xsinv + r);
    if (r == rows - 1 && l < 16 - rows) xsinv[rows + l] = make_float2(0.0f, 0.0f);
}

// Shared-memory matrix descriptor for a K-major operand of 32 bytes of K in unswizzled core-matrix order: a core matrix is
// 8 rows x 16 bytes stored contiguously (128 bytes); the two core matrices of a row block lie `lbo` bytes apart, row
// blocks `sbo` bytes apart.
__device__ __forceinline__ uint64_t umma_desc_plain(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | ((uint64_t)1 << 46);
}

// 16 lanes x 256 bits, eight times along the columns: register 4 i + {0, 1} = lane (t / 4), columns 8 i + 2 (t % 4) + {0, 1};
// register 4 i + {2, 3} = lane (t / 4) + 8, same columns (t = the thread's index in the warp). No memory clobber: the compiler
// may move shared-memory loads across it; what orders the registers' uses is tmem_wait_ld_of.
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t addr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(addr));
}
// Waits for the thread's loads from tensor memory; the registers pass through it, so nothing reads them earlier.
__device__ __forceinline__ void tmem_wait_ld_of(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]));
}

// two float32 lanes in one 64-bit register: d = a * b + c on both
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ float2 unpack2(uint64_t v) {
    float2 r;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
    return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__global__ void __launch_bounds__(kThreads, 1)
    gemv_q4_umma_kernel(const __grid_constant__ CUtensorMap wmap, const uint8_t* __restrict__ xdigits, const float* __restrict__ scale,
                        const float* __restrict__ zero, const float* __restrict__ bias, float* __restrict__ y, float* __restrict__ partials,
                        uint32_t m, uint32_t k, uint32_t n, uint32_t groups, Plan plan, uint32_t* status) {
    extern __shared__ uint8_t smem_unaligned[];
    uint8_t* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    const uint32_t nstages = plan.nstages, gps = plan.gps, tile_rows = plan.tile_rows;
    const uint32_t stage_bytes = tile_rows * 128u, dstride = plan.rows_pad * 128u, slot_bytes = tile_rows * 16u;
    uint8_t* ring = smem;                                    // nstages x (tile_rows x 128 raw bytes, as the TMA leaves them)
    uint8_t* digits = ring + (size_t)nstages * stage_bytes;  // gps tiles of dstride bytes (the instruction reads 8 KB from each: the tail is whatever follows)
    uint8_t* hibuf = digits + (size_t)gps * dstride;         // two buffers of a stage's high nibbles: four K slices of tile_rows x 32 bytes each
    uint8_t* szring = hibuf + 2 * stage_bytes;                   // kSzSlots x [2 groups][tile_rows / 2] float4 (s, s', z - 8 s, z' - 8 s') of two features
    float2* xsinv = reinterpret_cast<float2*>(szring + kSzSlots * slot_bytes);  // [gps][16]: (sum of x, 2^(e-26)) per group and row
    uint64_t* full = reinterpret_cast<uint64_t*>(xsinv + (size_t)gps * 16);
    uint64_t* empty = full + kMaxStages;
    uint64_t* hfull = empty + kMaxStages;  // [2] a stage's high nibbles and scales are in shared memory
    uint64_t* hempty = hfull + 2;          // [2] ... and the nibbles have been multiplied
    uint64_t* dfull = hempty + 2;          // [2] an accumulator (two groups) is complete
    uint64_t* dempty = dfull + 2;          // [2] ... and has been read out
    uint64_t* dgfull = dempty + 2;         // [kMaxTileStages] the digit tiles of the slice's stage i are in shared memory
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dgfull + kMaxTileStages);
    volatile uint32_t* failed = tmem_slot + 1;

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t slice = blockIdx.x % plan.slices, tlane = blockIdx.x / plan.slices;
    const uint32_t g_begin = slice * gps, g_end = min(groups, g_begin + gps);
    const uint32_t ngroups = g_end > g_begin ? g_end - g_begin : 0u;
    const uint32_t nstage_tile = (ngroups + 1) >> 1;
    const uint32_t my_tiles = (ngroups && tlane < plan.tiles) ? (plan.tiles - tlane + plan.lanes - 1) / plan.lanes : 0u;

    // The kernel ahead in the stream is always this call's x_digits_kernel, which itself began by waiting for everything
    // before it: the weights, scales and zero points are settled, and only the digit tiles are still being written. So the
    // set-up and the first weight stages run while that kernel does; the digit copies alone wait for it (below).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        for (uint32_t s = 0; s < nstages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1 + kNibbleWarps);  // the raw multiplications (one commit) and the warps that read the stage
        }
        for (uint32_t h = 0; h < 2; ++h) {
            mbar_init(hfull + h, kNibbleWarps);
            mbar_init(hempty + h, 1);
        }
        for (uint32_t d = 0; d < 2; ++d) {
            mbar_init(dfull + d, 1);
            mbar_init(dempty + d, kDrainWarps);
        }
        for (uint32_t i = 0; i < kMaxTileStages; ++i) mbar_init(dgfull + i, 1);
        *failed = 0;
        mbar_fence_init();
        tma_prefetch_map(&wmap);
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
    // a slice that ends in half a stage: the missing group's (sum of x, 2^(e-26)) pairs are zero (its weights are the zeros
    // the TMA fills in beyond K; the copies below bring the pairs of the groups that exist)
    for (uint32_t i = ngroups * 16 + tid; i < gps * 16; i += kThreads) xsinv[i] = make_float2(0.0f, 0.0f);
    __syncthreads();

    // ── the producer fills the ring before anything else happens (the weights do not depend on x) ──
    uint32_t ps = 0, pround = 0, ptile = tlane, pi = 0;  // producer position (warp 0, lane 0)
    auto produce_one = [&]() -> bool {  // requests the next stage; false when nothing is left or a wait gave up
        if (!my_tiles || ptile >= plan.tiles) return false;
        if (pround && !mbar_wait(empty + ps, (pround - 1) & 1, failed, status, kStatusEmptyWaitTimedOut)) return false;
        mbar_arrive_expect_tx(full + ps, stage_bytes);
        tma_load_2d(ring + (size_t)ps * stage_bytes, &wmap, (int32_t)((g_begin + 2 * pi) * 64u), (int32_t)(ptile * tile_rows), full + ps);
        if (++pi == nstage_tile) pi = 0, ptile += plan.lanes;
        if (++ps == nstages) ps = 0, ++pround;
        return true;
    };
    if (warp == 0 && lane == 0 && my_tiles) {
        // stage by stage: the weights of ring stage i, then the digit tiles of the slice's stage i (bulk copies of what the
        // conversion kernel left in global memory; they stay for all the CTA's tiles)
        const uint8_t* dsrc = xdigits + (size_t)g_begin * dstride;
        for (uint32_t i = 0; i < nstages; ++i) produce_one();
        asm volatile("griddepcontrol.wait;" ::: "memory");  // the digit tiles are complete and visible from here on
        for (uint32_t i = 0; i < nstage_tile; ++i) {
            {
                const uint32_t ng = min(2u, ngroups - 2 * i), bytes = ng * dstride;
                mbar_arrive_expect_tx(dgfull + i, bytes + (i == 0 ? ngroups * 128u : 0u));
                for (uint32_t off = 0; off < bytes; off += 8192u)
                    bulk_load(digits + (size_t)2 * i * dstride + off, dsrc + (size_t)2 * i * dstride + off, min(8192u, bytes - off), dgfull + i);
                if (i == 0) bulk_load(xsinv, xdigits + (size_t)groups * dstride + (size_t)g_begin * 128u, ngroups * 128u, dgfull);
            }
        }
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
        if (lane == 0 && my_tiles) {
            const uint32_t idesc = umma_idesc(2, 1, 0, 64, tile_rows);  // s32 accumulate, s8 digits x u8 weights
            const uint32_t hi_addr = smem_u32(hibuf);
            const uint32_t total = my_tiles * nstage_tile;
            // Two queues, each in stage order: raw bytes x digits of U (needs the stage's weights, its digits, and its
            // accumulator drained) and high nibbles x digits of V (needs the eight warps' buffer). Whichever is ready is
            // issued; the raw multiplications may run one stage ahead, so that the warps have a stage's time.
            auto ready = [](uint64_t* bar, uint32_t parity) {
                uint32_t done;
                asm volatile(
                    "{\n\t.reg .pred p;\n\t"
                    "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                    "selp.u32 %0, 1, 0, p;\n\t}"
                    : "=r"(done)
                    : "r"(smem_u32(bar)), "r"(parity)
                    : "memory");
                return done != 0;
            };
            uint32_t raw_next = 0, hi_next = 0;
            long long idle_since = 0;
            while (hi_next < total) {
                bool progressed = false;
                if (raw_next < total && raw_next <= hi_next + 1) {
                    const uint32_t it = raw_next, s = it % nstages, buf = it & 1u, i = it % nstage_tile;
                    if (ready(full + s, (it / nstages) & 1) && (it >= nstage_tile || ready(dgfull + i, 0)) &&
                        (it < 2 || ready(dempty + buf, ((it >> 1) - 1) & 1))) {
                        tc_fence_after_sync();
                        const uint32_t raw_addr = smem_u32(ring + (size_t)s * stage_bytes);
                        // group 2 i in the lower half-lanes of the accumulator, group 2 i + 1 in the upper
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) {
                            const uint32_t gi = j >> 1, h = j & 1u;
                            const uint32_t x_addr = smem_u32(digits + (size_t)(2 * i + gi) * dstride);
                            umma_i8_ss(tmem_addr(tmem, 16 * gi, buf * kTileMax), umma_desc_k128(x_addr + 32 * h), umma_desc_k128(raw_addr + 32 * j), idesc, h != 0);
                        }
                        umma_commit(empty + s);
                        ++raw_next, progressed = true;
                    }
                }
                if (hi_next < raw_next && ready(hfull + (hi_next & 1u), (hi_next >> 1) & 1)) {
                    const uint32_t it = hi_next, buf = it & 1u, i = it % nstage_tile;
                    tc_fence_after_sync();
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j) {
                        const uint32_t gi = j >> 1, h = j & 1u;
                        const uint32_t x_addr = smem_u32(digits + (size_t)(2 * i + gi) * dstride);
                        umma_i8_ss(tmem_addr(tmem, 16 * gi, buf * kTileMax), umma_desc_k128(x_addr + 64 + 32 * h),
                                   umma_desc_plain(hi_addr + buf * stage_bytes + j * tile_rows * 32u, 128, 256), idesc, true);
                    }
                    umma_commit(hempty + buf);
                    umma_commit(dfull + buf);
                    ++hi_next, progressed = true;
                }
                if (progressed) {
                    idle_since = 0;
                } else if (*failed) {
                    break;
                } else if (idle_since == 0) {
                    idle_since = clock64();
                    __nanosleep(40);
                } else if (clock64() - idle_since > 4000000000ll) {  // ~2 s with nothing to issue: give up as mbar_wait does
                    *failed = kStatusMmaWaitTimedOut;
                    atomicCAS(status, 0u, (uint32_t)kStatusMmaWaitTimedOut);
                    break;
                } else {
                    __nanosleep(40);  // nothing to issue: leave the issue slots to the warps that share this scheduler
                }
            }
        }
    } else if (warp >= kFirstNibbleWarp && warp < kFirstDrainWarp) {
        // ── per stage: the high nibbles of the thread's two feature rows (row and row + 128), and the rows' scales and zero
        // points ──
        const uint32_t row = tid - kFirstNibbleWarp * 32;  // 0 .. 127
        uint32_t s = 0, round = 0, it = 0;
        bool ok = true;
        for (uint32_t tl = 0; tl < my_tiles && ok; ++tl) {
            const uint32_t f0 = (tlane + tl * plan.lanes) * tile_rows;
            for (uint32_t i = 0; i < nstage_tile && ok; ++i, ++it) {
                // the scales first: their latency runs under the wait for the stage
                float sv[2][2], zv[2][2];
#pragma unroll
                for (uint32_t rr = 0; rr < 2; ++rr) {
                    const uint32_t rw = row + 128 * rr;
                    const bool fvalid = rw < tile_rows && f0 + rw < n;
                    const size_t at = (size_t)(fvalid ? f0 + rw : 0) * groups + g_begin + 2 * i;
#pragma unroll
                    for (uint32_t g = 0; g < 2; ++g) {
                        const bool have = fvalid && 2 * i + g < ngroups;
                        sv[rr][g] = have ? __ldg(scale + at + g) : 0.0f;
                        zv[rr][g] = have ? __ldg(zero + at + g) : 0.0f;
                    }
                }
                if (lane == 0) ok = mbar_wait(full + s, round & 1, failed, status, kStatusFullWaitTimedOut);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                // row by row (eight 16-byte pieces in registers at a time): the first row is read before the wait for the
                // nibble buffer, the second after it
                uint4 w[8];
                auto read_row = [&](uint32_t rw) {
                    if (rw >= tile_rows) return;
                    const uint8_t* src = ring + (size_t)s * stage_bytes + rw * 128u;
#pragma unroll
                    for (uint32_t c = 0; c < 8; ++c) {
                        w[c] = *reinterpret_cast<const uint4*>(src + ((c ^ (rw & 7u)) << 4));
                        w[c].x = (w[c].x >> 4) & 0x0f0f0f0fu, w[c].y = (w[c].y >> 4) & 0x0f0f0f0fu;
                        w[c].z = (w[c].z >> 4) & 0x0f0f0f0fu, w[c].w = (w[c].w >> 4) & 0x0f0f0f0fu;
                    }
                };
                auto write_row = [&](uint32_t rw, uint32_t rr) {
                    if (rw >= tile_rows) return;
                    uint8_t* dst = hibuf + (it & 1u) * stage_bytes + (rw >> 3) * 256u + (rw & 7u) * 16u;
#pragma unroll
                    for (uint32_t c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(dst + (c >> 1) * tile_rows * 32u + (c & 1u) * 128u) = w[c];
                    float* slot = reinterpret_cast<float*>(szring + (it % kSzSlots) * slot_bytes) + (rw >> 1) * 4 + (rw & 1u);
                    slot[0] = sv[rr][0], slot[2] = __fmaf_rn(-8.0f, sv[rr][0], zv[rr][0]);
                    slot[tile_rows * 2] = sv[rr][1], slot[tile_rows * 2 + 2] = __fmaf_rn(-8.0f, sv[rr][1], zv[rr][1]);
                };
                read_row(row);
                if (it >= 2) {  // the buffer the stage before last used
                    if (lane == 0) ok = mbar_wait(hempty + (it & 1u), ((it >> 1) - 1) & 1, failed, status, kStatusMmaWaitTimedOut);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                }
                write_row(row, 0);
                read_row(row + 128);
                __syncwarp();
                if (lane == 0) mbar_arrive(empty + s);  // the stage has been read: with the raw multiplications done the producer may refill it
                write_row(row + 128, 1);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(hfull + (it & 1u));
                if (++s == nstages) s = 0, ++round;
            }
        }
    } else if (warp >= kFirstDrainWarp) {
        // ── drain: warp = (quarter of tensor memory = four rows of x, 64 columns); thread t holds, for column block i of
        // eight, columns 8 i + 2 (t % 4) + {0, 1} of accumulator rows t / 4 and t / 4 + 8: digits 2 p and 2 p + 1
        // (p = (t / 4) % 2) of row 4 sub + t / 8 of x ──
        const uint32_t dw = warp - kFirstDrainWarp, sub = warp & 3u, cq = dw >> 2, q = lane & 3u, dp = (lane >> 2) & 1u;
        const uint32_t r = 4 * sub + (lane >> 3);
        const float dscale = dp ? 65536.0f : 1.0f;  // 256^(2 p)
        const bool live = 64 * cq < tile_rows && 4 * sub < m;  // a narrow tile leaves the last quarters without columns, few rows of x the last quarters of tensor memory without rows
        bool ok = my_tiles != 0;
        if (ok) {  // the (sum of x, 2^(e-26)) pairs arrive with the first stage's digits
            if (lane == 0) ok = mbar_wait(dgfull, 0, failed, status, kStatusFullWaitTimedOut);
            ok = __shfl_sync(0xffffffffu, ok, 0);
        }
        uint32_t it = 0;
        for (uint32_t tl = 0; tl < my_tiles && ok; ++tl) {
            const uint32_t tile = tlane + tl * plan.lanes;
            uint64_t acc[8];
#pragma unroll
            for (uint32_t i = 0; i < 8; ++i) acc[i] = 0ull;
            for (uint32_t i = 0; i < nstage_tile && ok; ++i, ++it) {
                const uint32_t buf = it & 1u;
                if (lane == 0) ok = mbar_wait(dfull + buf, (it >> 1) & 1, failed, status, kStatusMmaWaitTimedOut);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                tc_fence_after_sync();
                if (live) {
                    const float4* slot = reinterpret_cast<const float4*>(szring + (it % kSzSlots) * slot_bytes) + 32 * cq + q;
                    // one load of the warp's 64 columns per group: few, large loads, because each waits its turn behind the
                    // multiplication that is accumulating into tensor memory at that moment
                    uint32_t d[32];
#pragma unroll
                    for (uint32_t p = 0; p < 2; ++p) {
                        tmem_ld_16x256b_x8(tmem_addr(tmem, 32 * sub + 16 * p, buf * kTileMax + 64 * cq), d);
                        // 2^(e-26) of the group and row (0 for what the call does not have) times 256^(2 p); the sum of x goes
                        // with the zero point in the thread of digits 0 and 1
                        const float2 xs = xsinv[(2 * i + p) * 16 + r];
                        const float c = xs.y * dscale, z = dp == 0 ? xs.x : 0.0f;
                        const uint64_t c2 = pack2(c, c), z2 = pack2(z, z);
                        const float4* srow = slot + p * (tile_rows >> 1);
                        tmem_wait_ld_of(d);
#pragma unroll
                        for (uint32_t i8 = 0; i8 < 8; ++i8) {
                            if (64 * cq + 8 * i8 >= tile_rows) continue;  // uniform: the tile ends inside this warp's columns
                            const float4 sz = srow[4 * i8];
                            // |digit sum| < 2^22: D + 256 D' is exact in int32; its conversion rounds to 24 bits like every
                            // float32 operation after it
                            const int v0 = (int)d[4 * i8] + 256 * (int)d[4 * i8 + 2], v1 = (int)d[4 * i8 + 1] + 256 * (int)d[4 * i8 + 3];
                            const uint64_t f = pack2(__int2float_rn(v0), __int2float_rn(v1));
                            acc[i8] = fma2(pack2(sz.z, sz.w), z2, fma2(pack2(sz.x, sz.y), mul2(f, c2), acc[i8]));
                        }
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(dempty + buf);
            }
            if (!ok) break;
            // The two halves of a row of x sit in threads t and t ^ 4: add them, each keeping half of the column blocks
            // (blocks 2 kk + p), in a fixed order.
            float2 out[4];
#pragma unroll
            for (uint32_t kk = 0; kk < 4; ++kk) {
                const float2 a0 = unpack2(acc[2 * kk]), a1 = unpack2(acc[2 * kk + 1]);
                const float2 keep = dp ? a1 : a0, send = dp ? a0 : a1;
                const float ox = __shfl_xor_sync(0xffffffffu, send.x, 4), oy = __shfl_xor_sync(0xffffffffu, send.y, 4);
                // low digits + high digits, whichever thread does the sum
                out[kk].x = dp ? __fadd_rn(ox, keep.x) : __fadd_rn(keep.x, ox);
                out[kk].y = dp ? __fadd_rn(oy, keep.y) : __fadd_rn(keep.y, oy);
            }
#pragma unroll
            for (uint32_t kk = 0; kk < 4; ++kk) {
                const uint32_t col = 64 * cq + 8 * (2 * kk + dp) + 2 * q;  // and col + 1
                const uint32_t feature = tile * tile_rows + col;
#pragma unroll
                for (uint32_t e = 0; e < 2; ++e) {
                    if (col + e >= tile_rows || feature + e >= n || r >= m) continue;
                    const float v = e ? out[kk].y : out[kk].x;
                    if (plan.slices == 1) y[(size_t)r * n + feature + e] = bias ? __fadd_rn(v, bias[feature + e]) : v;
                    else partials[((size_t)slice * m + r) * n + feature + e] = v;  // K is split: added up by slice_sum_kernel
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

// y = the slices' partial sums added in slice order (+ bias): thread = V consecutive outputs (V = 4 when rows are a multiple
// of four outputs long, else 1); every slice's values are requested before the first is used
template <int V>
__global__ void __launch_bounds__(256) slice_sum_kernel(const float* __restrict__ partials, uint32_t slices, uint32_t total, uint32_t n,
                                                        const float* __restrict__ bias, float* __restrict__ y) {
    GQ_GRID_DEP_SYNC();
    const uint32_t idx = (blockIdx.x * 256 + threadIdx.x) * V;
    if (idx >= total) return;
    float part[16][V];
#pragma unroll
    for (uint32_t s = 0; s < 16; ++s) {
        if (V == 4) {
            const float4 v = s < slices ? __ldcg(reinterpret_cast<const float4*>(partials + (size_t)s * total + idx)) : make_float4(0.f, 0.f, 0.f, 0.f);
            part[s][0] = v.x, part[s][V > 1 ? 1 : 0] = v.y, part[s][V > 2 ? 2 : 0] = v.z, part[s][V > 3 ? 3 : 0] = v.w;
        } else {
            part[s][0] = s < slices ? __ldcg(partials + (size_t)s * total + idx) : 0.0f;
        }
    }
    float out[V];
#pragma unroll
    for (int j = 0; j < V; ++j) {
        float tot = part[0][j];
#pragma unroll
        for (uint32_t s = 1; s < 16; ++s)
            if (s < slices) tot = __fadd_rn(tot, part[s][j]);
        out[j] = bias ? __fadd_rn(tot, bias[(idx + j) % n]) : tot;
    }
    if (V == 4) *reinterpret_cast<float4*>(y + idx) = make_float4(out[0], out[V > 1 ? 1 : 0], out[V > 2 ? 2 : 0], out[V > 3 ? 3 : 0]);
    else y[idx] = out[0];
}

// ───────────────────────── the same product with the FEATURES on the lanes ─────────────────────────
// The kernel above keeps the rows of x on the lanes of tensor memory, so a thread of the drain meets a new pair of
// features in every block of eight columns and has to fetch their (scale, zero - 8 scale) from shared memory each time:
// those loads, not the arithmetic, are what its drain costs. Here the operands change places: the packed weight is the
// A operand (M = 128 features: raw bytes as the TMA left them, high nibbles from the four nibble warps), the digit tiles
// of x are the B operand (N = 16 / 32 / 64 digit rows), and an accumulator is [feature][digit row of x]. A kind::i8
// instruction takes 65 cycles for any N up to 128 (128 at N = 256), so eight instructions of N <= 64 per 128 features
// and two groups cost what four of N = 256 cost per 256 features: nothing is lost. A drain thread now owns ONE feature:
// its scale and zero point are two registers per group (read from global memory while it waits for the accumulator),
// the 64 digit sums of the 16 rows of x arrive with four loads from tensor memory, and the accumulator is released
// before the arithmetic starts. Each group has an accumulator of its own (eight slots of 64 columns), so the
// multiplications run up to eight groups ahead of the drain. A CTA owns tiles of 128 features over ALL of K: the digit
// tiles of x stream through the ring beside the weight (two groups = one stage), nothing is split, no partial sums,
// no second kernel.
constexpr int kLThreads = 448;            // warp 0 producer, 1 MMA issuer, 2-5 nibbles, 6-13 drain (two sets of four)
constexpr uint32_t kLFirstDrainWarp = 6;
constexpr uint32_t kLTile = 128;          // features per tile = M of the instruction
constexpr uint32_t kLRaw = kLTile * 128;  // a stage's packed weight: 128 features x two groups
constexpr uint32_t kLSlots = 8;           // accumulators in flight, 64 columns each
constexpr uint32_t kLSets = 2;            // drain sets: set j reads out the tile's groups j, j + 2, ...
constexpr int kLMaxStages = 6;  // (eight measured slower: 16.0 -> 17.3 us on 14336 x 4096 at one row)
constexpr uint32_t kLMaxGroups = 128;     // the (sum of x, 2^(e-26)) pairs of every group stay in shared memory: 128 bytes a group

__global__ void __launch_bounds__(kLThreads, 1)
    gemv_q4_lanes_kernel(const __grid_constant__ CUtensorMap wmap, const uint8_t* __restrict__ xdigits, const float* __restrict__ scale,
                         const float* __restrict__ zero, const float* __restrict__ bias, float* __restrict__ y, float* __restrict__ partials, uint32_t m,
                         uint32_t n, uint32_t groups, uint32_t rows_pad, uint32_t nstages, uint32_t tile_rows, uint32_t kslices, uint32_t gps,
                         uint32_t* status) {
    extern __shared__ uint8_t smem_unaligned[];
    uint8_t* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    const uint32_t dstride = rows_pad * 128u, stage_bytes = kLRaw + 2u * dstride;
    uint8_t* ring = smem;                                                   // nstages x (raw 16 KB | two digit tiles)
    uint8_t* hibuf = ring + (size_t)nstages * stage_bytes;                  // two buffers of a stage's high nibbles
    float2* xsinv = reinterpret_cast<float2*>(hibuf + 2 * kLRaw);           // [groups][16] (sum of x, 2^(e-26))
    float* exchange = reinterpret_cast<float*>(xsinv + (size_t)groups * 16);  // [16 rows][128 features]: set 1's sums on their way to set 0
    uint64_t* full = reinterpret_cast<uint64_t*>(exchange + 16 * kLTile);
    uint64_t* empty = full + kLMaxStages;
    uint64_t* hfull = empty + kLMaxStages;
    uint64_t* hempty = hfull + 2;
    uint64_t* dfull = hempty + 2;
    uint64_t* dempty = dfull + kLSlots;
    uint64_t* xsfull = dempty + kLSlots;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xsfull + 1);
    volatile uint32_t* failed = tmem_slot + 1;

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // A tile is tile_rows <= 128 features (the host sizes it so that the tiles fill whole waves of CTAs); the instruction
    // still multiplies 128 rows, the rest being whatever the stage held before: those lanes are never read out.
    // Where the features alone do not fill the SMs (a narrow shard with a long K), K is cut in `kslices` slices of `gps`
    // groups: CTA c works on slice c % kslices of the tiles c / kslices, + lanes, ...; the slices' sums go to `partials`
    // and are added in slice order afterwards (slice_sum_kernel, or the gather that sends them).
    const uint32_t slice = blockIdx.x % kslices, lane_idx = blockIdx.x / kslices, lanes_n = gridDim.x / kslices;
    const uint32_t gbeg = slice * gps, ng_slice = gbeg < groups ? min(gps, groups - gbeg) : 0u;
    const uint32_t tiles = (n + tile_rows - 1) / tile_rows, chunks = (ng_slice + 1) >> 1;
    const uint32_t my_tiles = (lane_idx < tiles && ng_slice) ? (tiles - lane_idx + lanes_n - 1) / lanes_n : 0u;

    // As above: the kernel ahead in the stream is this call's x_digits_kernel; the weights are settled, the digit tiles
    // are not. The first weight stages are requested before the dependency wait, the digit copies after it.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        for (uint32_t s = 0; s < nstages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1 + kNibbleWarps);  // the multiplications (one commit) and the warps that read the raw bytes
        }
        for (uint32_t h = 0; h < 2; ++h) {
            mbar_init(hfull + h, kNibbleWarps);
            mbar_init(hempty + h, 1);
        }
        for (uint32_t d = 0; d < kLSlots; ++d) {
            mbar_init(dfull + d, 1);
            mbar_init(dempty + d, 4);  // the four warps of the set that reads the slot out
        }
        mbar_init(xsfull, 1);
        *failed = 0;
        mbar_fence_init();
        tma_prefetch_map(&wmap);
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
    __syncthreads();

    uint32_t ps = 0, pround = 0, pt = 0, pc = 0;  // producer position (warp 0, lane 0)
    auto stage_groups = [&](uint32_t c) { return min(2u, ng_slice - 2u * c); };
    auto request_weights = [&]() -> bool {  // the next stage's barrier and raw bytes; false when nothing is left or a wait gave up
        if (pt >= my_tiles) return false;
        if (pround && !mbar_wait(empty + ps, (pround - 1) & 1, failed, status, kStatusEmptyWaitTimedOut)) return false;
        mbar_arrive_expect_tx(full + ps, tile_rows * 128u + stage_groups(pc) * dstride);
        tma_load_2d(ring + (size_t)ps * stage_bytes, &wmap, (int32_t)(gbeg * 64u + pc * 128u), (int32_t)((lane_idx + pt * lanes_n) * tile_rows), full + ps);
        return true;
    };
    auto request_digits = [&]() {  // ... and its digit tiles; then on to the next stage
        bulk_load(ring + (size_t)ps * stage_bytes + kLRaw, xdigits + (size_t)(gbeg + 2 * pc) * dstride, stage_groups(pc) * dstride, full + ps);
        if (++pc == chunks) pc = 0, ++pt;
        if (++ps == nstages) ps = 0, ++pround;
    };
    if (warp == 0 && lane == 0 && my_tiles) {
        // raw bytes of the first stages, then (the digit kernel has finished) their digits and the pairs of every group
        uint32_t ahead = 0;
        {
            uint32_t s0 = ps, r0 = pround, t0 = pt, c0 = pc;
            while (ahead < nstages && request_weights()) {
                ++ahead;
                if (++pc == chunks) pc = 0, ++pt;
                if (++ps == nstages) ps = 0, ++pround;
            }
            ps = s0, pround = r0, pt = t0, pc = c0;
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");
        mbar_arrive_expect_tx(xsfull, groups * 128u);
        bulk_load(xsinv, xdigits + (size_t)groups * dstride, groups * 128u, xsfull);
        for (uint32_t i = 0; i < ahead; ++i) request_digits();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0)
            while (request_weights()) request_digits();
    } else if (warp == 1) {
        if (lane == 0 && my_tiles) {
            // One thread issues everything, and a lone thread runs an instruction every few cycles at best: the loop is kept
            // to ~100 instructions a stage (counters instead of divisions, descriptors as a 32-bit base plus a constant).
            const uint32_t idesc = umma_idesc(2, 0, 1, kLTile, rows_pad);  // s32 accumulate, u8 weights x s8 digits
            // descriptor = (high word: stride between 8-row groups, version, layout) | (low word: address >> 4 | leading offset)
            constexpr uint32_t k128_hi = (1024u >> 4) | (1u << 14) | (2u << 29), plain_hi = (256u >> 4) | (1u << 14);
            constexpr uint32_t k128_lo = 1u << 16, plain_lo = (128u >> 4) << 16;
            auto desc = [](uint32_t hi, uint32_t lo) { return ((uint64_t)hi << 32) | lo; };
            const uint32_t ring_lo = ((smem_u32(ring) & 0x3FFFFu) >> 4) | k128_lo, hi_lo = ((smem_u32(hibuf) & 0x3FFFFu) >> 4) | plain_lo;
            const uint32_t stage_step = stage_bytes >> 4, dstep = dstride >> 4;
            const uint32_t bar_empty = smem_u32(empty), bar_hempty = smem_u32(hempty), bar_dfull = smem_u32(dfull);
            auto commit_at = [](uint32_t bar_addr) {
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
            };
            uint32_t s = 0, sparity = 0, stage_lo = ring_lo, it = 0, gc = 0;
            bool ok = true;
            for (uint32_t t = 0; t < my_tiles && ok; ++t) {
                for (uint32_t c = 0; c < chunks && ok; ++c, ++it) {
                    const uint32_t hb = it & 1u, ng = 2u * c + 2u <= ng_slice ? 2u : 1u;
                    const uint32_t slot0 = gc & (kLSlots - 1), slot1 = (gc + 1) & (kLSlots - 1);
                    if (gc >= kLSlots) {  // the groups' accumulators have been read out
                        ok = mbar_wait(dempty + slot0, ((gc >> 3) - 1) & 1, failed, status, kStatusMmaWaitTimedOut);
                        if (ng == 2) ok = ok && mbar_wait(dempty + slot1, (((gc + 1) >> 3) - 1) & 1, failed, status, kStatusMmaWaitTimedOut);
                    }
                    ok = ok && mbar_wait(full + s, sparity, failed, status, kStatusFullWaitTimedOut) &&
                         mbar_wait(hfull + hb, (it >> 1) & 1, failed, status, kStatusMmaWaitTimedOut);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t dig_lo = stage_lo + (kLRaw >> 4), hib_lo = hi_lo + hb * (kLRaw >> 4);
                    {
                        const uint32_t acc = tmem + slot0 * 64u;
                        umma_i8_ss(acc, desc(k128_hi, stage_lo), desc(k128_hi, dig_lo), idesc, false);           // raw bytes x digits of U
                        umma_i8_ss(acc, desc(k128_hi, stage_lo + 2), desc(k128_hi, dig_lo + 2), idesc, true);
                        umma_i8_ss(acc, desc(plain_hi, hib_lo), desc(k128_hi, dig_lo + 4), idesc, true);          // high nibbles x digits of V
                        umma_i8_ss(acc, desc(plain_hi, hib_lo + (kLTile * 32u >> 4)), desc(k128_hi, dig_lo + 6), idesc, true);
                        commit_at(bar_dfull + 8 * slot0);
                    }
                    if (ng == 2) {
                        const uint32_t acc = tmem + slot1 * 64u, x_lo = dig_lo + dstep;
                        umma_i8_ss(acc, desc(k128_hi, stage_lo + 4), desc(k128_hi, x_lo), idesc, false);
                        umma_i8_ss(acc, desc(k128_hi, stage_lo + 6), desc(k128_hi, x_lo + 2), idesc, true);
                        umma_i8_ss(acc, desc(plain_hi, hib_lo + 2 * (kLTile * 32u >> 4)), desc(k128_hi, x_lo + 4), idesc, true);
                        umma_i8_ss(acc, desc(plain_hi, hib_lo + 3 * (kLTile * 32u >> 4)), desc(k128_hi, x_lo + 6), idesc, true);
                        commit_at(bar_dfull + 8 * slot1);
                    }
                    commit_at(bar_empty + 8 * s);
                    commit_at(bar_hempty + 8 * hb);
                    gc += ng;
                    stage_lo += stage_step;
                    if (++s == nstages) s = 0, sparity ^= 1u, stage_lo = ring_lo;
                }
            }
        }
    } else if (warp >= kFirstNibbleWarp && warp < kLFirstDrainWarp) {
        // per stage: the high nibbles of the thread's feature row (a second set of four warps taking every other stage changed
        // nothing: the stages do not wait for these warps). Every lane waits on the barriers itself (no broadcast
        // of the outcome), positions are counters: the loop around the sixteen loads and stores is what a stage costs here.
        const uint32_t row = tid - kFirstNibbleWarp * 32;  // 0 .. 127
        const uint8_t* src_row = ring + row * 128u;
        uint8_t* dst_row = hibuf + (row >> 3) * 256u + (row & 7u) * 16u;
        const uint32_t sw = row & 7u;
        uint32_t s = 0, sparity = 0;
        bool ok = true;
        {
            for (uint32_t it = 0, total = my_tiles * chunks; it < total && ok; ++it) {
                const uint32_t hb = it & 1u;
                ok = mbar_wait(full + s, sparity, failed, status, kStatusFullWaitTimedOut);
                if (!ok) break;
                uint4 w[8];
                const uint8_t* src = src_row + (size_t)s * stage_bytes;
                if (row < tile_rows) {
#pragma unroll
                    for (uint32_t q = 0; q < 8; ++q) w[q] = *reinterpret_cast<const uint4*>(src + ((q ^ sw) << 4));
                }
#pragma unroll
                for (uint32_t q = 0; q < 8; ++q) {
                    w[q].x = (w[q].x >> 4) & 0x0f0f0f0fu, w[q].y = (w[q].y >> 4) & 0x0f0f0f0fu;
                    w[q].z = (w[q].z >> 4) & 0x0f0f0f0fu, w[q].w = (w[q].w >> 4) & 0x0f0f0f0fu;
                }
                if (it >= 2) {  // the buffer's previous stage has been multiplied
                    ok = mbar_wait(hempty + hb, ((it >> 1) - 1) & 1, failed, status, kStatusMmaWaitTimedOut);
                    if (!ok) break;
                }
                uint8_t* dst = dst_row + hb * kLRaw;
                if (row < tile_rows) {
#pragma unroll
                    for (uint32_t q = 0; q < 8; ++q) *reinterpret_cast<uint4*>(dst + (q >> 1) * kLTile * 32u + (q & 1u) * 128u) = w[q];
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(empty + s);
                    mbar_arrive(hfull + hb);
                }
                if (++s == nstages) s = 0, sparity ^= 1u;
            }
        }
    } else if (warp >= kLFirstDrainWarp) {
        // drain: thread = one feature (a lane of tensor memory); set j takes the tile's groups j, j + 2, ...
        const uint32_t set = (warp - kLFirstDrainWarp) >> 2, quarter = warp & 3u, fl = 32 * quarter + lane;
        bool ok = my_tiles != 0;
        if (ok) {
            if (lane == 0) ok = mbar_wait(xsfull, 0, failed, status, kStatusFullWaitTimedOut);
            ok = __shfl_sync(0xffffffffu, ok, 0);
        }
        for (uint32_t t = 0; t < my_tiles; ++t) {
            const uint32_t feature = (lane_idx + t * lanes_n) * tile_rows + fl;
            const bool have = fl < tile_rows && feature < n;
            const float* srow = scale + (size_t)(have ? feature : 0) * groups;
            const float* zrow = zero + (size_t)(have ? feature : 0) * groups;
            float acc[16];
#pragma unroll
            for (uint32_t r = 0; r < 16; ++r) acc[r] = 0.0f;
            // the scale and zero point of the set's next group are requested a group ahead: a read-out that has fallen behind
            // finds its accumulator ready at once and would otherwise wait out the load's latency every time
            float sv_next = have && set < ng_slice ? __ldg(srow + gbeg + set) : 0.0f, zv_next = have && set < ng_slice ? __ldg(zrow + gbeg + set) : 0.0f;
            for (uint32_t gl = set; gl < ng_slice && ok; gl += kLSets) {
                const uint32_t g = gbeg + gl, gc = t * ng_slice + gl, slot = gc & (kLSlots - 1);
                const float sv = sv_next, zv = zv_next;
                if (have && gl + kLSets < ng_slice) sv_next = __ldg(srow + g + kLSets), zv_next = __ldg(zrow + g + kLSets);
                ok = mbar_wait(dfull + slot, (gc >> 3) & 1, failed, status, kStatusMmaWaitTimedOut);
                if (!ok) break;
                tc_fence_after_sync();
                const float zm = __fmaf_rn(-8.0f, sv, zv);
                const float2* xs = xsinv + (size_t)g * 16;
                uint32_t d[4][16];
#pragma unroll
                for (uint32_t q = 0; q < 4; ++q)
                    if (16 * q < rows_pad) tmem_ld16(tmem_addr(tmem, 32 * quarter, slot * 64 + 16 * q), d[q]);
                tmem_wait_ld();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(dempty + slot);  // the sums are in registers: the slot may be multiplied into again
#pragma unroll
                for (uint32_t q = 0; q < 4; ++q) {
                    if (4 * q >= m) continue;  // uniform
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        // digits 0 .. 3 of row 4 q + i sit in columns 2 i, 2 i + 8, 2 i + 1, 2 i + 9 of the block (digit_row);
                        // |digit sum| < 2^22: D + 256 D' is exact in int32, the two halves meet in one rounded fma
                        const int lo = (int)d[q][2 * i] + 256 * (int)d[q][2 * i + 8], hi = (int)d[q][2 * i + 1] + 256 * (int)d[q][2 * i + 9];
                        const float tsum = __fmaf_rn(__int2float_rn(hi), 65536.0f, __int2float_rn(lo));
                        const float2 p = xs[4 * q + i];  // (sum of x, 2^(e-26)) of the group and row: 0 for rows the call does not have
                        acc[4 * q + i] = __fmaf_rn(zm, p.x, __fmaf_rn(sv, __fmul_rn(tsum, p.y), acc[4 * q + i]));
                    }
                }
            }
            // set 1 hands its sums to set 0, which adds them (set 0 + set 1, a fixed order) and writes y
            if (set == 1) {
#pragma unroll
                for (uint32_t r = 0; r < 16; ++r) exchange[r * kLTile + fl] = acc[r];
            }
            named_barrier_sync(1, 8 * 32);
            if (set == 0 && ok && have) {
                const float bs = bias ? bias[feature] : 0.0f;
#pragma unroll
                for (uint32_t r = 0; r < 16; ++r) {
                    if (r >= m) continue;
                    const float v = __fadd_rn(acc[r], exchange[r * kLTile + fl]);
                    if (kslices == 1) y[(size_t)r * n + feature] = bias ? __fadd_rn(v, bs) : v;
                    else partials[((size_t)slice * m + r) * n + feature] = v;  // K is split: added up (with the bias) afterwards
                }
            }
            named_barrier_sync(2, 8 * 32);  // the exchange buffer is free for the next tile
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

size_t lanes_smem_bytes(uint32_t groups, uint32_t rows_pad, uint32_t nstages) {
    return 1024 + (size_t)nstages * (kLRaw + 2u * rows_pad * 128u) + 2 * kLRaw + (size_t)groups * 128 + 16 * kLTile * 4 +
           (2 * kLMaxStages + 4 + 2 * kLSlots + 1) * 8 + 64;
}

// nanoseconds of one instruction at N columns (M = 64, K = 32 bytes)
double mma_ns(uint32_t ncols) {
    if (ncols <= 64) return 83.0;
    if (ncols <= 128) return 83.0 + (ncols - 64) * (9.0 / 64.0);
    return 92.0 + (ncols - 128) * (41.0 / 128.0);
}

size_t smem_bytes(uint32_t gps, uint32_t tile_rows, uint32_t rows_pad, uint32_t nstages) {
    return 1024 + (size_t)(nstages + 2) * tile_rows * 128 + (size_t)gps * rows_pad * 128 + (size_t)kSzSlots * tile_rows * 16 + (size_t)gps * 128 + kBarrierBytes + 64 +
           8192;  // the instruction reads 8 KB from the last group's digits whatever rows_pad is: keep that inside the allocation
}

// (slices, tile width) that minimise the time of the busiest CTA: per stage eight instructions, or the drain of its 2 x 64
// accumulator rows if that is longer (~4 ns per column); ~0.4 us per tile of results; when K is split, the second kernel.
Plan make_plan(uint64_t m, uint64_t n, uint64_t groups, int sm_count) {
    const uint32_t rows_pad = m <= 4 ? 16u : m <= 8 ? 32u : 64u;
    Plan best{};
    double best_cost = 1e30;
    for (uint32_t ks = 1; ks <= 16 && ks <= (uint32_t)sm_count; ++ks) {
        uint32_t gps = (uint32_t)((groups + ks - 1) / ks);
        gps += gps & 1u;  // whole stages: only the last slice may end in half a stage (the TMA fills what lies beyond K with zeros)
        const uint32_t slices = (uint32_t)((groups + gps - 1) / gps);
        if (slices != ks) continue;  // the same cut as a smaller ks
        const uint32_t lanes_max = (uint32_t)sm_count / slices;
        const uint32_t stages_per_tile = gps / 2;
        if (stages_per_tile > kMaxTileStages) continue;
        for (uint32_t tile_rows = 16; tile_rows <= kTileMax; tile_rows += 16) {
            if (smem_bytes(gps, tile_rows, rows_pad, kMinStages) > kSmemBudget) continue;
            uint32_t nstages = kMinStages;
            while (nstages < (uint32_t)kMaxStages && smem_bytes(gps, tile_rows, rows_pad, nstages + 1) <= kSmemBudget) ++nstages;
            const uint32_t tiles = (uint32_t)((n + tile_rows - 1) / tile_rows);
            const uint32_t lanes = tiles < lanes_max ? tiles : lanes_max;
            const uint32_t rounds = (tiles + lanes - 1) / lanes;
            const double stage_ns = fmax(8.0 * mma_ns(tile_rows), 4.0 * tile_rows);
            double cost = (double)rounds * (stages_per_tile * stage_ns + 400.0) + (nstages < 3 ? 1500.0 : 0.0);
            if (slices > 1) cost += 3000.0 + (double)slices * m * n * 8.0 / 4000.0;
            if (cost < best_cost) best_cost = cost, best = Plan{slices, gps, tile_rows, tiles, lanes, lanes * slices, nstages, rows_pad};
        }
    }
    return best;
}

}  // namespace

static uint64_t digits_region_bytes(uint64_t groups, uint32_t rows_pad) { return (groups * (rows_pad * 128ull + 128ull) + 1023) / 1024 * 1024; }

// How many K slices the features-on-the-lanes kernel cuts a call in (1: none) and the groups per slice: as many slices as
// fit the SMs beside the feature tiles, each of whole stages.
static void lanes_slices(uint64_t n, uint64_t groups, int sm_count, uint32_t* kslices, uint32_t* gps) {
    const uint64_t tiles = (n + kLTile - 1) / kLTile;
    uint64_t ks = tiles * 4 >= (uint64_t)sm_count * 3 ? 1 : (uint64_t)sm_count / tiles;  // three quarters of the SMs busy: leave it
    ks = ks > 8 ? 8 : ks < 1 ? 1 : ks;
    uint64_t per = (groups + ks - 1) / ks;
    per += per & 1;
    if (per < 4) per = groups < 4 ? groups + (groups & 1) : 4;  // two stages a slice at least
    *gps = (uint32_t)per;
    *kslices = (uint32_t)((groups + per - 1) / per);
}

// What AUTO's cost model needs of it: the K slices and the stages (of two groups) the busiest CTA works through.
void gemv_q4_lanes_shape(uint64_t n, uint64_t k, int sm_count, uint32_t* kslices, uint32_t* stages_per_cta) {
    uint32_t ks, gps;
    lanes_slices(n, k / 128, sm_count, &ks, &gps);
    const uint64_t waves = ((n + kLTile - 1) / kLTile * ks + sm_count - 1) / sm_count;
    *kslices = ks, *stages_per_cta = (uint32_t)(waves * ((gps + 1) / 2));
}

// The scratch holds the digit tiles of x and, when K is split, the slices' partial sums.
uint64_t gemv_q4_umma_scratch_bytes(uint64_t m, uint64_t k, uint64_t n, int sm_count) {
    if (m < 1 || m > 16 || k == 0 || k % 128 || n == 0) return 0;
    const Plan p = make_plan(m, n, k / 128, sm_count);
    if (p.grid == 0) return 0;
    uint32_t ls = 1, lg = 0;
    if (k / 128 <= kLMaxGroups) lanes_slices(n, k / 128, sm_count, &ls, &lg);  // (the other kernel's slices, if more)
    const uint64_t slices = p.slices > ls ? p.slices : ls;
    return digits_region_bytes(k / 128, p.rows_pad) + slices * m * n * 4;  // (K not split: room for a copy of y)
}

const float* gemv_q4_umma_partials(const void* scratch, uint64_t m, uint64_t k, uint64_t n, int sm_count) {
    const Plan p = make_plan(m, n, k / 128, sm_count);
    return reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(scratch) + digits_region_bytes(k / 128, p.rows_pad));
}

// Returns false when the shape is not this kernel's: group_size 128, in_features a multiple of 128, 1 to 16 rows of x,
// 16-byte aligned x and weights. `scratch` holds gemv_q4_umma_scratch_bytes bytes. Up to three launches: x -> digit tiles
// (tiny), the linear, and the sum over the K slices.
bool launch_gemv_q4_umma(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                         const float* scale, const float* zero, const float* bias, uint64_t n, uint64_t group, float* y, void* scratch,
                         uint32_t* deferred) {
    if (m < 1 || m > 16 || group != 128 || k == 0 || k % 128 || n == 0 || m * n > 0x7fffffffull || k > (1ull << 24)) return false;
    if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(x)) & 15) != 0) return false;
    const uint64_t groups = k / 128, row_bytes = k / 2;
    const Plan p = make_plan(m, n, groups, sm_count);
    if (p.grid == 0) return false;
    uint8_t* xdigits = reinterpret_cast<uint8_t*>(scratch);
    float* partials = reinterpret_cast<float*>(xdigits + digits_region_bytes(groups, p.rows_pad));
    const CUtensorMap wmap = make_tensor_map_2d(q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, row_bytes, n, row_bytes, 128, p.tile_rows, Swizzle::B128);
    const size_t smem = smem_bytes(p.gps, p.tile_rows, p.rows_pad, p.nstages);
    launch_after(x_digits_kernel, dim3((uint32_t)((groups * (p.rows_pad / 4) + 7) / 8)), dim3(128), 0, s, x, (uint32_t)m, (uint32_t)k, (uint32_t)groups, p.rows_pad,
                 xdigits);
    GQ_CUDA(cudaFuncSetAttribute(gemv_q4_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    launch_after(gemv_q4_umma_kernel, dim3(p.grid), dim3(kThreads), smem, s, wmap, (const uint8_t*)xdigits, scale, zero, p.slices > 1 ? nullptr : bias, y,
                 partials, (uint32_t)m, (uint32_t)k, (uint32_t)n, (uint32_t)groups, p, status);
    if (deferred) *deferred = p.slices > 1 ? p.slices : 0u;
    if (p.slices > 1 && !deferred) {
        if (n % 4 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0)
            launch_after(slice_sum_kernel<4>, dim3((uint32_t)((m * n / 4 + 255) / 256)), dim3(256), 0, s, (const float*)partials, p.slices, (uint32_t)(m * n),
                         (uint32_t)n, bias, y);
        else
            launch_after(slice_sum_kernel<1>, dim3((uint32_t)((m * n + 255) / 256)), dim3(256), 0, s, (const float*)partials, p.slices, (uint32_t)(m * n),
                         (uint32_t)n, bias, y);
    }
    return true;
}

// The features-on-the-lanes kernel: group_size 128, in_features a multiple of 128 up to 16384, 1 to 16 rows of x, 16-byte
// aligned x and weights. `scratch` holds gemv_q4_umma_scratch_bytes bytes. Two launches — x -> digit tiles (tiny), the
// linear — and, where K is cut in slices, the sum over them (left to the caller when `deferred` is given: it receives the
// slice count, 0 for none, and the sums lie where gemv_q4_umma_partials says).
bool launch_gemv_q4_lanes(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                          const float* scale, const float* zero, const float* bias, uint64_t n, uint64_t group, float* y, void* scratch,
                          uint32_t* deferred) {
    if (m < 1 || m > 16 || group != 128 || k == 0 || k % 128 || k / 128 > kLMaxGroups || n == 0 || m * n > 0x7fffffffull) return false;
    if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(x)) & 15) != 0) return false;
    const uint64_t groups = k / 128, row_bytes = k / 2;
    const Plan p = make_plan(m, n, groups, sm_count);  // (for rows_pad: the scratch layout is the other kernel's)
    if (p.grid == 0) return false;
    const uint32_t rows_pad = p.rows_pad;
    uint32_t nstages = kLMaxStages;
    while (nstages > 2 && lanes_smem_bytes((uint32_t)groups, rows_pad, nstages) > kSmemBudget) --nstages;
    if (lanes_smem_bytes((uint32_t)groups, rows_pad, nstages) > kSmemBudget) return false;
    uint8_t* xdigits = reinterpret_cast<uint8_t*>(scratch);
    float* partials = reinterpret_cast<float*>(xdigits + digits_region_bytes(groups, rows_pad));
    uint32_t kslices, gps;
    lanes_slices(n, groups, sm_count, &kslices, &gps);
    // With more than one wave of CTAs the tiles are made equal (28672 features on 148 SMs: 296 tiles of 97, two per CTA,
    // instead of 224 of 128, two for some and one for others). A stage costs about the same whatever its width, so a
    // single wave keeps 128-feature tiles (more, narrower tiles measured slower: 14336 features 16.0 -> 17.0 us).
    const uint64_t waves = ((n + kLTile - 1) / kLTile + sm_count - 1) / sm_count;
    uint64_t tile_rows = waves > 1 ? (n + waves * sm_count - 1) / (waves * sm_count) : kLTile;
    tile_rows = tile_rows < 8 ? 8 : tile_rows > kLTile ? kLTile : tile_rows;
    const CUtensorMap wmap = make_tensor_map_2d(q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, row_bytes, n, row_bytes, 128, (uint32_t)tile_rows, Swizzle::B128);
    const size_t smem = lanes_smem_bytes((uint32_t)groups, rows_pad, nstages);
    const uint64_t tiles = (n + tile_rows - 1) / tile_rows;
    const uint64_t lanes = tiles * kslices <= (uint64_t)sm_count ? tiles : (uint64_t)sm_count / kslices;
    launch_after(x_digits_kernel, dim3((uint32_t)((groups * (rows_pad / 4) + 7) / 8)), dim3(128), 0, s, x, (uint32_t)m, (uint32_t)k, (uint32_t)groups, rows_pad,
                 xdigits);
    GQ_CUDA(cudaFuncSetAttribute(gemv_q4_lanes_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    launch_after(gemv_q4_lanes_kernel, dim3((uint32_t)(lanes * kslices)), dim3(kLThreads), smem, s, wmap, (const uint8_t*)xdigits, scale, zero,
                 kslices > 1 ? nullptr : bias, y, partials, (uint32_t)m, (uint32_t)n, (uint32_t)groups, rows_pad, nstages, (uint32_t)tile_rows, kslices, gps, status);
    if (deferred) *deferred = kslices > 1 ? kslices : 0u;
    if (kslices > 1 && !deferred) {
        if (n % 4 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0)
            launch_after(slice_sum_kernel<4>, dim3((uint32_t)((m * n / 4 + 255) / 256)), dim3(256), 0, s, (const float*)partials, kslices, (uint32_t)(m * n),
                         (uint32_t)n, bias, y);
        else
            launch_after(slice_sum_kernel<1>, dim3((uint32_t)((m * n + 255) / 256)), dim3(256), 0, s, (const float*)partials, kslices, (uint32_t)(m * n),
                         (uint32_t)n, bias, y);
    }
    return true;
}

}  // namespace gq
