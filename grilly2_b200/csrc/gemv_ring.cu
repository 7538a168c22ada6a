// Decode GEMV for int4 group-128 weights and one to four rows of x on the
// warp-level integer tensor instruction (mma.sync m16n8k32, u8 x s8 -> s32),
// organised so that a weight costs few instructions and no CTA-wide barrier
// stands between the launch and the first multiply.
//
// Arithmetic (as gemv_imma.cu): within each group of 128 k, x is held as an
// exact fixed-point integer X = rint(x 2^(30-e)), 2^e > max|x| of the group,
// split into four signed base-256 digits. The digits are the columns of the
// MMA's B operand (four per row of x), sixteen output features are the rows
// of A, and the int4 levels enter as bytes 0..15: per group and feature the
// four digit sums are exact int32, recombined and scaled in float32:
//   y[f] = sum_g  s[f][g] * (sum_k level x) + (zero[f][g] - 8 s[f][g]) * (sum_k x).
// The only approximation is X (2^-31 of the group's max |x|). A non-finite x
// gives NaN outputs.
//
// Ownership: K is split by group over the 16 consumer warps (warp w owns
// groups w, w + 16, ...). A warp converts only its own groups of x, straight
// into the B fragments it keeps in registers for the whole kernel — no
// CTA-wide barrier, and nothing of x is re-read from shared memory in the
// main loop. It then walks the CTA's output features in blocks of 16: per
// block and group two 16-byte shared-memory reads per lane feed four MMAs
// (lane (g, t) reads bytes 16 t .. 16 t + 15 of the group's 64 bytes of features
// 2 g and 2 g + 1; word i of those 16 bytes, split in even and odd nibbles, is
// the A fragment of MMA i, and the B fragments are laid out to match), then
// ~12 instructions fold the int32 sums into two float accumulators. After
// its groups the warp leaves a partial sum per feature in shared memory; the
// last warp to arrive for a block adds the 16 partials in warp order (so the
// result does not depend on timing) and writes y.
//
// Data movement: one producer warp fills a ring of 16-row blocks with 1-D bulk (TMA)
// copies of two weight rows each (MMA rows g and g + 8 are features 2 g and 2 g + 1,
// read by different instructions, and each pair is followed by 16 bytes of padding so
// that one instruction's reads of 8 pairs x 4 chunks spread over all banks; a bulk
// copy costs the copy engine ~40 ns whatever its size, so nothing smaller than
// a row goes that way). The block's scales and zero points come as 2-D TMA
// tiles (16 features x 32 groups, 128-byte swizzle, so that the eight features
// a quarter-warp reads for one group fall in eight different banks). Three or
// more blocks (>= 100 KB) are in flight per SM.
//
// Algorithmic bytes per launch: packed weights + scales + zeros + x + y
// (+ bias). Bound: HBM bandwidth.
#include "gq_internal.h"
#include "tc_common.cuh"

namespace gq {

namespace {

constexpr int kWarps = 16;                  // consumer warps
constexpr int kThreads = (kWarps + 1) * 32; // + the producer warp
constexpr uint32_t kBlockRows = 16;         // output features per MMA and per ring stage
constexpr uint32_t kRowPad = 16;            // bytes added to a row's pitch in shared memory
constexpr int kMaxStages = 8;
constexpr uint32_t kScratchWords = 8 * 4 * 4 * 2;  // per warp and 8-column tile: [column][t][mma][parity] digit words of one group

__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ void st_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// One group of one row of x -> digit words in the warp's scratch, plus 2^(e-30) and the group's sum of x.
// Lane L converts x[128 G + 32 tt + 8 i + 2 b + par], b = 0..3, with tt = L / 8, i = (L / 2) % 4, par = L % 2:
// the four values one packed weight word's even (par = 0) or odd (par = 1) nibbles of chunk tt meet in MMA i.
__device__ __forceinline__ void load_group(const float* __restrict__ xr, uint32_t k, uint32_t G, uint32_t lane, float (&v)[4]) {
    const uint32_t kb = G * 128 + 32 * (lane >> 3) + 8 * ((lane >> 1) & 3u) + (lane & 1u);
#pragma unroll
    for (int b = 0; b < 4; ++b) v[b] = kb + 2 * b < k ? __ldg(xr + kb + 2 * b) : 0.0f;
}
__device__ __forceinline__ void convert_group(const float (&v)[4], uint32_t lane, uint32_t col0, uint32_t* scratch, float& inv, float& xs) {
    const uint32_t tt = lane >> 3, i = (lane >> 1) & 3u, par = lane & 1u;
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    const bool bad = !(fabsf(v[0]) <= 3.402823466e+38f) | !(fabsf(v[1]) <= 3.402823466e+38f) | !(fabsf(v[2]) <= 3.402823466e+38f) |
                     !(fabsf(v[3]) <= 3.402823466e+38f);
    if (bad) amax = __uint_as_float(0x7f800000u);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    uint32_t e = __float_as_uint(amax) >> 23;
    float mult;
    if (e == 255) {
        mult = 0.0f, inv = __uint_as_float(0x7fc00000u);
    } else if (amax == 0.0f) {
        mult = inv = 0.0f;
    } else {
        e = max(e, 32u);
        mult = __uint_as_float((283u - e) << 23);  // 2^(30 - e)
        inv = __uint_as_float((e - 29u) << 23);    // 2^(e - 30)
    }
    uint32_t word[4] = {0u, 0u, 0u, 0u};
    int sum_lo = 0, sum_hi = 0;  // X = lo + 65536 hi with lo a signed 16-bit number: both sums stay far inside int32
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        int X = __float2int_rn(v[b] * mult);
        const int xl = (int)(int16_t)X;
        sum_lo += xl, sum_hi += (X - xl) >> 16;
        const int d0 = (int)(int8_t)X;
        X = (X - d0) >> 8;
        const int d1 = (int)(int8_t)X;
        X = (X - d1) >> 8;
        const int d2 = (int)(int8_t)X;
        const int d3 = (X - d2) >> 8;
        word[0] |= ((uint32_t)d0 & 0xFFu) << (8 * b), word[1] |= ((uint32_t)d1 & 0xFFu) << (8 * b);
        word[2] |= ((uint32_t)d2 & 0xFFu) << (8 * b), word[3] |= ((uint32_t)d3 & 0xFFu) << (8 * b);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, o);
        sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, o);
    }
    xs = __fmaf_rn((float)sum_hi, 65536.0f, (float)sum_lo) * inv;
#pragma unroll
    for (int p = 0; p < 4; ++p) scratch[(((col0 + p) * 4 + tt) * 4 + i) * 2 + par] = word[p];
}

// Shared memory: [stages x (16 padded rows | scale tiles | zero tiles)] [partials: stages x 16 warps x 32] [scratch: 16 warps x 256
// words] [counts: stages] [barriers] [failed].
template <int MR, int GPW, bool PEER>
__global__ void __launch_bounds__(kThreads, 1)
    gemv_q4_ring_kernel(const __grid_constant__ CUtensorMap smap, const __grid_constant__ CUtensorMap zmap, const uint32_t* __restrict__ q,
                        const float* __restrict__ x, const float* __restrict__ bias, float* __restrict__ y, uint32_t k, uint32_t n,
                        uint32_t groups, uint32_t nstages, uint32_t stage_stride, uint32_t* status, bool x_settled, PeerOut peer) {
    extern __shared__ uint8_t smem_unaligned[];
    uint8_t* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);  // swizzle atoms are 1 KB
    const uint32_t row_bytes = k >> 1, pitch = 2 * row_bytes + kRowPad;  // two consecutive features share a copy; 16 bytes of padding follow
    const uint32_t nbox = groups >> 5;                                      // 32 groups of scales (128 bytes) per box row
    const uint32_t sz_off = ((kBlockRows / 2) * pitch + 1023u) & ~1023u;          // a block's scales: nbox boxes of 16 rows x 128 bytes,
    const uint32_t zr_off = sz_off + nbox * 2048u;                          // then its zero points, each box 128-byte swizzled
    float* partials = reinterpret_cast<float*>(smem + (size_t)nstages * stage_stride);
    constexpr int kTiles = (MR + 1) / 2;
    uint32_t* scratch_all = reinterpret_cast<uint32_t*>(partials + (size_t)nstages * kWarps * 32 * kTiles);
    uint32_t* counts = scratch_all + kWarps * kScratchWords * kTiles;
    uint64_t* full = reinterpret_cast<uint64_t*>(counts + kMaxStages);
    uint64_t* empty = full + kMaxStages;
    volatile uint32_t* failed = reinterpret_cast<volatile uint32_t*>(empty + kMaxStages);

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // Output features are dealt out in units of eight rows (a CTA gets floor or ceil of units / CTAs of them) and worked on
    // in 16-row blocks, so that only a CTA's last block can be a short one. A block costs the warp-level tensor instruction
    // the same time whether its 16 rows are all in use or not: dealing the rows out evenly in pairs (every CTA the same
    // bytes, every CTA a short last block) ran 12 % slower on 28672 x 8192 than whole blocks, of which a few CTAs get one
    // more than the others; eight-row units leave those few CTAs half a block more instead of a whole one.
    const uint32_t units_total = (n + 7) / 8;
    const uint32_t u0 = (uint32_t)((uint64_t)units_total * blockIdx.x / gridDim.x), u1 = (uint32_t)((uint64_t)units_total * (blockIdx.x + 1) / gridDim.x);
    const uint32_t row_begin = u0 * 8, row_end = min(u1 * 8, n);
    const uint32_t nrows = row_end - row_begin;
    const uint32_t blocks = (nrows + kBlockRows - 1) / kBlockRows;
    auto block_first = [&](uint32_t rb) { return rb * kBlockRows; };                           // first row of block rb within the CTA
    auto block_rows = [&](uint32_t rb) { return min(kBlockRows, nrows - rb * kBlockRows); };  // its rows

    // The producer warp initialises the barriers itself and requests the first round of blocks at once; the barrier that
    // publishes them to the consumers comes after the consumers' conversion of x, so neither costs the other anything.
    auto request = [&](uint32_t rb) {  // lanes 0-7 bulk-copy a block's weight rows two at a time, lanes 16.. and 24.. fetch its scale and
                                       // zero-point tiles
        const uint32_t s = rb % nstages;
        const uint32_t rows_here = block_rows(rb);
        if (lane == 0) mbar_arrive_expect_tx(full + s, rows_here * row_bytes + 2 * nbox * 2048u);
        __syncwarp();
        uint8_t* dst = smem + (size_t)s * stage_stride;
        const size_t row0 = (size_t)row_begin + block_first(rb);
        if (2 * lane < rows_here)  // features 2 lane and 2 lane + 1 (the last pair of the CTA may be a single row)
            bulk_load(dst + lane * pitch, reinterpret_cast<const uint8_t*>(q) + (row0 + 2 * lane) * row_bytes,
                      min(2u, rows_here - 2 * lane) * row_bytes, full + s);
        else if (lane >= 16 && lane < 16 + nbox)
            tma_load_2d(dst + sz_off + (lane - 16) * 2048u, &smap, (int32_t)((lane - 16) * 32), (int32_t)row0, full + s);
        else if (lane >= 24 && lane < 24 + nbox)
            tma_load_2d(dst + zr_off + (lane - 24) * 2048u, &zmap, (int32_t)((lane - 24) * 32), (int32_t)row0, full + s);
    };
    // Two blocks are requested before anything else happens in the CTA, the rest of the first round right after the arrival below
    // (requesting the whole ring here made the 14336 x 4096 layer slower: the flood delays the few CTAs of the launch ahead that
    // still wait for a seventh block, and with them that launch's end, which this launch's writes wait for).
    const uint32_t first_round = min(min(blocks, nstages), 2u);
    if (warp == kWarps) {
        if (lane < nstages) {
            mbar_init(full + lane, 1);
            mbar_init(empty + lane, kWarps);
            counts[lane] = 0;
        }
        if (lane == 0) *failed = 0;
        __syncwarp();
        if (lane == 0) mbar_fence_init();
        __syncwarp();
        for (uint32_t rb = 0; rb < first_round; ++rb) request(rb);
        // the consumers meet this arrival after their conversion of x (named barrier 4): neither side waits for the other before
        asm volatile("bar.arrive 4, %0;" ::"n"(kThreads) : "memory");
    }

    if (warp == kWarps) {
        // ── producer: refills a stage as soon as every consumer warp has let go of it ──
        for (uint32_t rb = first_round; rb < blocks; ++rb) {
            const uint32_t s = rb % nstages, round = rb / nstages;
            bool ok = true;
            if (round && lane == 0) ok = mbar_wait(empty + s, (round - 1) & 1, failed, status, kStatusEmptyWaitTimedOut);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            request(rb);
        }
        return;
    }

    // ── consumers: B fragments of this warp's groups, once ──
    constexpr int NT = (MR + 1) / 2;               // 8-column tiles of B: two rows of x (4 digits each) per tile
    const uint32_t g8 = lane >> 2, t = lane & 3u;  // MMA row (and B column) index, thread-in-group
    const uint32_t xloc = t >> 1, high = t & 1u;   // this lane's accumulator columns: digits 2 high, 2 high + 1 of row 2 nt + xloc of x
    uint32_t* scratch = scratch_all + warp * (kScratchWords * NT);
    uint32_t bf[GPW][NT][8];
    float coef[GPW][NT], zcoef[GPW][NT];
    constexpr bool kHoist = GPW * MR <= 8;  // registers permitting, every load of x is requested before the first conversion waits for one
    float xv[kHoist ? GPW : 1][MR][4];
    // x may be the previous launch's output: wait for that launch to finish, unless the caller knows that it is not
    // (x_settled); y is only written after a wait in either case. The producer warp did not wait: the weights it fetches
    // are not written by that launch.
    if (!x_settled) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the launch behind may start now (see launch_after)
    }
    if (kHoist) {
#pragma unroll
        for (int gi = 0; gi < GPW; ++gi)
#pragma unroll
            for (int r = 0; r < MR; ++r)
                if (warp + gi * kWarps < groups) load_group(x + (size_t)r * k, k, warp + gi * kWarps, lane, xv[kHoist ? gi : 0][r]);
    }
#pragma unroll
    for (int gi = 0; gi < GPW; ++gi) {
        const uint32_t G = warp + gi * kWarps;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            coef[gi][nt] = zcoef[gi][nt] = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) bf[gi][nt][j] = 0u;
        }
        if (G >= groups) continue;  // uniform over the warp
        float inv[MR], xs[MR];
        if (!kHoist) {
#pragma unroll
            for (int r = 0; r < MR; ++r) load_group(x + (size_t)r * k, k, G, lane, xv[0][r]);
        }
#pragma unroll
        for (int r = 0; r < MR; ++r) convert_group(xv[kHoist ? gi : 0][r], lane, 4 * r, scratch, inv[r], xs[r]);
        __syncwarp();
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint32_t col = nt * 8 + g8;
            if (col < 4 * MR) {
                const uint4 lo = *reinterpret_cast<const uint4*>(scratch + (col * 4 + t) * 8), hi = *reinterpret_cast<const uint4*>(scratch + (col * 4 + t) * 8 + 4);
                bf[gi][nt][0] = lo.x, bf[gi][nt][1] = lo.y, bf[gi][nt][2] = lo.z, bf[gi][nt][3] = lo.w;
                bf[gi][nt][4] = hi.x, bf[gi][nt][5] = hi.y, bf[gi][nt][6] = hi.z, bf[gi][nt][7] = hi.w;
            }
#pragma unroll
            for (int r = 0; r < MR; ++r)
                if ((uint32_t)r == 2 * nt + xloc) {
                    coef[gi][nt] = high ? inv[r] * 65536.0f : inv[r];
                    zcoef[gi][nt] = high ? 0.0f : xs[r];
                }
        }
        __syncwarp();
    }

    // Offsets that do not change from block to block: this lane's 16 bytes of each of its groups within a stage, and
    // its two features' scale / zero-point words within the stage's tiles. (Row r, group G) of a tile lies at
    // r * 128 + ((G % 32 / 4) ^ (r % 8)) * 16 + G % 4 * 4 of box G / 32.
    uint32_t woff[GPW], so0[GPW], so1[GPW];
#pragma unroll
    for (int gi = 0; gi < GPW; ++gi) {
        const uint32_t G = warp + gi * kWarps;
        woff[gi] = g8 * pitch + G * 64 + t * 16;
        const uint32_t r0 = 2 * g8, r1 = r0 + 1, gc = (G & 31u) >> 2, gb = (G >> 5) * 2048u + (G & 3u) * 4u;
        so0[gi] = sz_off + gb + r0 * 128u + ((gc ^ (r0 & 7u)) << 4), so1[gi] = sz_off + gb + r1 * 128u + ((gc ^ (r1 & 7u)) << 4);
    }
    const uint32_t zr_delta = zr_off - sz_off;
    asm volatile("bar.sync 4, %0;" ::"n"(kThreads) : "memory");  // the producer's barriers and counters are ready
    if (x_settled && warp == 0) {  // nothing waited yet: one warp does, after its conversion, and lets the launch behind start
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    const uint32_t smem_base = smem_u32(smem);
    uint32_t step = 0;  // PEER: this call's number, read from the device once the launch ahead is known to be done
    bool have_step = false;
    for (uint32_t rb = 0; rb < blocks; ++rb) {
        const uint32_t s = rb % nstages, round = rb / nstages;
        if (!mbar_wait(full + s, round & 1, failed, status, kStatusFullWaitTimedOut)) break;
        const uint32_t stage = smem_base + s * stage_stride;
        const uint8_t* st_p = smem + (size_t)s * stage_stride;
        float acc0[NT], acc1[NT];  // MMA rows g8 and g8 + 8 are features 2 g8 and 2 g8 + 1 of the block
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc0[nt] = acc1[nt] = 0.0f;
#pragma unroll
        for (int gi = 0; gi < GPW; ++gi) {
            const uint32_t G = warp + gi * kWarps;
            if (G >= groups) continue;
            const uint4 wa = lds128(stage + woff[gi]), wb = lds128(stage + woff[gi] + row_bytes);
            const uint32_t a[4] = {wa.x, wa.y, wa.z, wa.w}, b[4] = {wb.x, wb.y, wb.z, wb.w};
            int c[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t a0 = a[i] & 0x0f0f0f0fu, a1 = b[i] & 0x0f0f0f0fu, a2 = (a[i] >> 4) & 0x0f0f0f0fu, a3 = (b[i] >> 4) & 0x0f0f0f0fu;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_u8s8(c[nt], a0, a1, a2, a3, bf[gi][nt][2 * i], bf[gi][nt][2 * i + 1]);
            }
            const float s0 = *reinterpret_cast<const float*>(st_p + so0[gi]), s1 = *reinterpret_cast<const float*>(st_p + so1[gi]);
            const float z0 = *reinterpret_cast<const float*>(st_p + so0[gi] + zr_delta), z1 = *reinterpret_cast<const float*>(st_p + so1[gi] + zr_delta);
            const float zm0 = __fmaf_rn(-8.0f, s0, z0), zm1 = __fmaf_rn(-8.0f, s1, z1);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float v0 = (float)(c[nt][0] + (c[nt][1] << 8)) * coef[gi][nt], v1 = (float)(c[nt][2] + (c[nt][3] << 8)) * coef[gi][nt];
                acc0[nt] = __fmaf_rn(zm0, zcoef[gi][nt], __fmaf_rn(s0, v0, acc0[nt]));
                acc1[nt] = __fmaf_rn(zm1, zcoef[gi][nt], __fmaf_rn(s1, v1, acc1[nt]));
            }
        }
        // low + high digit pairs; lanes with t even then hold this warp's share of (row 2 nt + xloc of x, features 2 g8, 2 g8 + 1)
        float* part = partials + ((size_t)s * kWarps + warp) * (32 * NT);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            acc0[nt] += __shfl_xor_sync(0xffffffffu, acc0[nt], 1);
            acc1[nt] += __shfl_xor_sync(0xffffffffu, acc1[nt], 1);
            if (!high) part[nt * 32 + xloc * 16 + 2 * g8] = acc0[nt], part[nt * 32 + xloc * 16 + 2 * g8 + 1] = acc1[nt];
        }
        __syncwarp();
        uint32_t last = 0;
        if (lane == 0) {
            __threadfence_block();
            last = atomicAdd(counts + s, 1u) == kWarps - 1;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
            __threadfence_block();
            asm volatile("griddepcontrol.wait;" ::: "memory");  // y (and bias) may be buffers the launch ahead still uses
            const uint32_t f = lane & 15u, j = block_first(rb) + f;
            const bool row_valid = f < block_rows(rb);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t xr = 2 * nt + (lane >> 4);
                const volatile float* p = partials + (size_t)s * kWarps * (32 * NT) + nt * 32 + lane;
                float tot = p[0];
#pragma unroll
                for (int w = 1; w < kWarps; ++w) tot = __fadd_rn(tot, p[w * 32 * NT]);
                if (xr < MR && row_valid) {
                    const float val = bias ? __fadd_rn(tot, bias[row_begin + j]) : tot;
                    if (PEER) {  // this rank's block of columns, sent to every rank's receive buffer: value and step in one word
                        if (!have_step) step = *reinterpret_cast<const volatile uint32_t*>(peer.state) + 1u, have_step = true;
                        const unsigned long long word = ((unsigned long long)step << 32) | __float_as_uint(val);
                        const size_t at = ((size_t)(step & 1u) * peer.m_total + peer.row0 + xr) * peer.n_full + (size_t)peer.rank * n + row_begin + j;
                        for (uint32_t pr = 0; pr < peer.nranks; ++pr) st_sys_u64(peer.ll[pr] + at, word);
                    } else {
                        y[(size_t)xr * n + row_begin + j] = val;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) counts[s] = 0;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);  // everything this warp does with the block is done
    }
    if (PEER) {
        // Receive: every value arrives as one 64-bit word (step << 32 | float bits) in this rank's receive buffer, written by
        // its owner's epilogue above with a single store, so a word whose upper half is this step IS the value: no fence, no
        // counter, no signal. The CTAs share the buffer out, wait (bounded) for their words and write the plain y_full. Two
        // halves of the buffer alternate by step parity: a rank can be at most one step ahead of the slowest (it cannot
        // finish step s + 1 without that rank's step s + 1 words), so the words of step s are never overwritten before
        // they were read. The step word lives on the device, so a captured launch counts on by itself at every replay.
        // (Letting only a few CTAs receive, so that the launch behind gets the other SMs early, measured no faster.)
        const uint32_t receivers = gridDim.x;
        asm volatile("griddepcontrol.wait;" ::: "memory");  // y_full and the step word belong to the launch ahead until it is done
        if (!have_step) step = *reinterpret_cast<const volatile uint32_t*>(peer.state) + 1u;
        const uint32_t ctid = tid, total = MR * peer.n_full;
        const uint32_t e0 = (uint32_t)((uint64_t)total * blockIdx.x / receivers), e1 = (uint32_t)((uint64_t)total * (blockIdx.x + 1) / receivers);
        const unsigned long long* mine = peer.ll[peer.rank] + ((size_t)(step & 1u) * peer.m_total + peer.row0) * peer.n_full;
        const long long start = clock64();
        for (uint32_t i = e0 + ctid; i < e1; i += kWarps * 32) {
            unsigned long long v;
            for (;;) {
                v = ld_sys_u64(mine + i);
                if ((uint32_t)(v >> 32) == step) break;
                if (clock64() - start > peer.wait_cycles) {  // give up, tell the host which rank's words never came
                    atomicCAS(status, 0u, kStatusPeerWaitTimedOut + (i % peer.n_full) / n);
                    break;
                }
            }
            peer.y_full[(size_t)peer.row0 * peer.n_full + i] = __uint_as_float((uint32_t)v);
        }
        named_barrier_sync(3, kWarps * 32);
        if (ctid == 0) {
            __threadfence();
            if (atomicAdd(peer.state + 1, 1u) == receivers - 1) {  // the last receiver: the call is finished
                peer.state[1] = 0;
                peer.state[0] = step;
            }
        }
    }
}

template <int MR, int GPW, bool PEER>
void launch(cudaStream_t s, uint32_t grid, uint64_t smem, const uint32_t* q, const float* x, const float* scale, const float* zero,
            const float* bias, float* y, uint64_t k, uint64_t n, uint64_t groups, uint64_t nstages, uint64_t stage_stride, uint32_t* status,
            bool overlap, bool x_settled, const PeerOut& peer) {
    // scales and zero points as (n x groups) float matrices, fetched in tiles of 16 rows x 32 groups; rows past n read zeros
    const CUtensorMap smap = make_tensor_map_2d(scale, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, groups, n, groups * 4, 32, kBlockRows, Swizzle::B128);
    const CUtensorMap zmap = make_tensor_map_2d(zero, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, groups, n, groups * 4, 32, kBlockRows, Swizzle::B128);
    GQ_CUDA(cudaFuncSetAttribute(gemv_q4_ring_kernel<MR, GPW, PEER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid), cfg.blockDim = dim3(kThreads), cfg.dynamicSmemBytes = smem, cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr, cfg.numAttrs = overlap ? 1 : 0;
    GQ_CUDA(cudaLaunchKernelEx(&cfg, gemv_q4_ring_kernel<MR, GPW, PEER>, smap, zmap, q, x, bias, y, (uint32_t)k, (uint32_t)n, (uint32_t)groups,
                               (uint32_t)nstages, (uint32_t)stage_stride, status, overlap && x_settled, peer));
}

}  // namespace

// Up to four rows of x, group_size 128, K a multiple of 4096 (so that a row of scales is whole 128-byte tile rows) of which two
// 16-row blocks fit shared memory (K <= 8192).
// Returns false when the shape is not this kernel's.
bool launch_gemv_q4_ring(cudaStream_t s, int sm_count, uint32_t* status, const float* x, uint64_t m, uint64_t k, const uint32_t* q,
                         const float* scale, const float* zero, const float* bias, uint64_t n, uint64_t group, float* y,
                         bool overlap_previous, bool x_settled, const PeerOut* peer) {
    if (m < 1 || m > 4 || group != 128 || k == 0 || (k & 4095) || k > 16384 || n == 0 || n > 0x7fffffffull) return false;
    if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(scale) | reinterpret_cast<uintptr_t>(zero)) & 15) != 0) return false;
    const uint64_t groups = k / 128, row_bytes = k / 2;
    const uint64_t gpw = (groups + kWarps - 1) / kWarps;
    const uint64_t blocks_total = (n + kBlockRows - 1) / kBlockRows;
    const uint32_t grid = (uint32_t)(blocks_total < (uint64_t)sm_count ? blocks_total : (uint64_t)sm_count);
    const uint64_t units_max = ((n + 7) / 8 + grid - 1) / grid;  // the most eight-row units a CTA gets
    const uint64_t blocks = (units_max * 8 + kBlockRows - 1) / kBlockRows;  // ... and 16-row blocks
    const uint64_t stage_stride = ((kBlockRows / 2) * (2 * row_bytes + kRowPad) + 1023) / 1024 * 1024 + 2 * (groups / 32) * 2048;
    const uint64_t tiles = (m + 1) / 2;
    if (m > 2 && gpw > 4) return false;  // the B fragments of three or four rows of x must fit the registers
    const uint64_t per_stage = stage_stride + kWarps * 32 * 4 * tiles;
    const uint64_t fixed = 1024 + kWarps * kScratchWords * 4 * tiles + kMaxStages * 4 + 2 * kMaxStages * 8 + 64;
    const uint64_t budget = 226 * 1024;
    if (fixed + 2 * per_stage > budget) return false;
    uint64_t nstages = (budget - fixed) / per_stage;
    if (nstages > kMaxStages) nstages = kMaxStages;
    if (nstages > blocks) nstages = blocks;
    const uint64_t smem = fixed + nstages * per_stage;
#define GQ_RING(MRV, GPWV)                                                                                                              \
    do {                                                                                                                                \
        if (peer)                                                                                                                       \
            launch<MRV, GPWV, true>(s, grid, smem, q, x, scale, zero, bias, y, k, n, groups, nstages, stage_stride, status, overlap_previous, \
                                    x_settled, *peer);                                                                                  \
        else                                                                                                                            \
            launch<MRV, GPWV, false>(s, grid, smem, q, x, scale, zero, bias, y, k, n, groups, nstages, stage_stride, status,            \
                                     overlap_previous, x_settled, PeerOut());                                                           \
    } while (0)
    if (m == 1) {
        if (gpw <= 2) GQ_RING(1, 2);
        else if (gpw <= 4) GQ_RING(1, 4);
        else GQ_RING(1, 8);
    } else if (m == 2) {
        if (gpw <= 2) GQ_RING(2, 2);
        else if (gpw <= 4) GQ_RING(2, 4);
        else GQ_RING(2, 8);
    } else if (m == 3) {
        if (gpw <= 2) GQ_RING(3, 2);
        else GQ_RING(3, 4);
    } else {
        if (gpw <= 2) GQ_RING(4, 2);
        else GQ_RING(4, 4);
    }
#undef GQ_RING
    return true;
}

}  // namespace gq
