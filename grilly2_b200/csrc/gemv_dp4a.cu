// The fast decode GEMV: integer dot products (dp4a) of the packed weights
// against an exact fixed-point copy of x, four signed 8-bit digit planes wide.
//
// Why: the reference's arithmetic (g2-linear-q4.glsl:54-91, g2-linear-q8.glsl:43-75)
// spends one integer->float conversion and one FMA per weight. On a B200 that
// is the bound, not HBM: at 6.5 TB/s an SM must retire 46 int4 levels per
// clock, and at ~5 instructions per level the float kernel (gemv.cu) reaches
// a fifth of the bandwidth. Here a 32-bit word of packed weights is used as a
// vector of four bytes directly:
//
//   x[k] ~= X[k] * 2^(e - 30),  X[k] = rint(x[k] * 2^(30 - e)) an int32,
//           2^e > max|x| over the 16-byte weight vector the element falls in
//   X[k]  = d0 + 256 d1 + 65536 d2 + 2^24 d3,  d0..d2 in [-128, 127], |d3| <= 64
//   sum_k q[k] x[k] ~= 2^(e-30) * (D0 + 256 D1 + 65536 D2 + 2^24 D3),
//   D_i = sum_k q[k] d_i[k]   -- exact int32, four dp4a per four weights
//
// so a weight costs one instruction (plus 3/8 for splitting int4 nibbles into
// bytes) instead of two to five. The only approximation is X: |x - X 2^(e-30)|
// <= 2^-31 of the vector's largest |x|, far below float32 accumulation error,
// and every D_i is exact. The digit sums are recombined and scaled in float32
// once per vector: acc = fma(s * 2^(e-30), T, acc); acc = fma(zero - 8 s,
// sum(x), acc) for int4, acc = fma(2^(e-30), T, acc) for int8, whose row scale
// multiplies the finished sum as in the reference. The result differs from
// the reference-order kernel by float32 rounding only (tests hold it to
// max|y - y_ref| / max|y_ref| <= 1e-5 and to the reference's float64 bound).
//
// Each CTA first converts x into digit planes in shared memory (after issuing
// its first weight loads, so the conversion hides under their latency), then
// every warp streams C weight rows at a time with 128-bit coalesced loads,
// keeping one register copy of x's digits for all C rows.
//
// Non-finite x: a vector holding an Inf or NaN makes its outputs NaN (the
// float kernel would propagate Inf as Inf).
#include "gq_internal.h"

namespace gq {

__device__ __forceinline__ uint4 ldg_stream4(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Power-of-two scales for one block of x whose largest magnitude is amax:
// mult = 2^(30 - e), inv = 2^(e - 30) with 2^e > amax. A zero block gets
// (0, 0); a non-finite one gets (0, NaN) so its outputs are NaN.
__device__ __forceinline__ void block_scales(float amax, float& mult, float& inv) {
    uint32_t b = __float_as_uint(amax) >> 23;  // biased exponent; amax >= 0
    if (b == 255) {
        mult = 0.0f;
        inv = __uint_as_float(0x7fc00000u);
        return;
    }
    if (amax == 0.0f) {
        mult = inv = 0.0f;
        return;
    }
    b = max(b, 32u);  // below 2^-95 the digits just lose bits; such x contributes nothing measurable
    mult = __uint_as_float((283u - b) << 23);  // 2^(30 - (b - 126))
    inv = __uint_as_float((b - 29u) << 23);    // 2^((b - 126) - 30)
}

// The four signed base-256 digits of X, least significant first.
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

// D0 + 256 D1 + 65536 D2 + 2^24 D3 in float32. The pairs fit int32 exactly
// (|D_i| < 2^17 per 32-value vector), so only the last step rounds.
__device__ __forceinline__ float combine_digits(const int (&D)[4]) {
    const int lo = D[0] + (D[1] << 8), hi = D[2] + (D[3] << 8);
    return __fmaf_rn(65536.0f, (float)hi, (float)lo);
}

static constexpr int kWarpsD = 8;

// ── x -> digit planes ────────────────────────────────────────────────────
// int4 layout, per 16-byte weight vector v (32 values, 4 words of 8 nibbles):
// chunk j = 2 * word + half, half 0 = even nibbles (k0,k2,k4,k6), half 1 = odd;
// each chunk is four uint32, one per digit plane. Stored chunk-major,
// xd[(j * vecs + v) * 4 + digit], so a warp reading chunk j of 32 consecutive
// vectors reads 512 contiguous bytes (no bank conflicts).
template <bool XVEC>
__device__ __forceinline__ void prepare_x_q4(const float* __restrict__ xr, uint32_t k, uint32_t vecs, uint32_t* xd,
                                             float* xinv, float* xsum) {
    // one packed word (8 values) per thread; the trip count is the same for a whole warp (shuffles inside)
    for (uint32_t base = 0; base < vecs * 4; base += blockDim.x) {
        const uint32_t wd = base + threadIdx.x;
        const bool live = wd < vecs * 4;
        const uint32_t k0 = wd * 8, v = wd >> 2, word = wd & 3;
        float xv[8];
        if (XVEC) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
                if (live && k0 + 4 * h < k) t = __ldg(reinterpret_cast<const float4*>(xr + k0) + h);
                xv[4 * h] = t.x, xv[4 * h + 1] = t.y, xv[4 * h + 2] = t.z, xv[4 * h + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) xv[j] = (live && k0 + j < k) ? __ldg(xr + k0 + j) : 0.0f;
        }
        float amax = 0.0f;
        bool bad = false;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            amax = fmaxf(amax, fabsf(xv[j]));
            bad |= !(fabsf(xv[j]) <= 3.402823466e+38f);  // Inf or NaN
        }
        if (bad) amax = __uint_as_float(0x7f800000u);
        float sum = ((xv[0] + xv[1]) + (xv[2] + xv[3])) + ((xv[4] + xv[5]) + (xv[6] + xv[7]));
        // the four words of a vector sit in four adjacent lanes
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (!live) continue;
        float mult, inv;
        block_scales(amax, mult, inv);
        int d[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) digits_of(__float2int_rn(xv[j] * mult), d[j]);
        uint4 even, odd;
        even.x = pack4(d[0][0], d[2][0], d[4][0], d[6][0]);
        even.y = pack4(d[0][1], d[2][1], d[4][1], d[6][1]);
        even.z = pack4(d[0][2], d[2][2], d[4][2], d[6][2]);
        even.w = pack4(d[0][3], d[2][3], d[4][3], d[6][3]);
        odd.x = pack4(d[1][0], d[3][0], d[5][0], d[7][0]);
        odd.y = pack4(d[1][1], d[3][1], d[5][1], d[7][1]);
        odd.z = pack4(d[1][2], d[3][2], d[5][2], d[7][2]);
        odd.w = pack4(d[1][3], d[3][3], d[5][3], d[7][3]);
        reinterpret_cast<uint4*>(xd)[(2 * word) * vecs + v] = even;
        reinterpret_cast<uint4*>(xd)[(2 * word + 1) * vecs + v] = odd;
        if (word == 0) {
            xinv[v] = inv;
            xsum[v] = sum;
        }
    }
}

template <int MR, int C, bool XVEC>
__global__ void __launch_bounds__(kWarpsD * 32) gemv_q4_dp4a_kernel(const float* __restrict__ x, const uint4* __restrict__ q,
                                                                     const float* __restrict__ scale,
                                                                     const float* __restrict__ zero,
                                                                     const float* __restrict__ bias, float* __restrict__ y,
                                                                     uint32_t m, uint32_t k, uint32_t n, uint32_t vecs,
                                                                     uint32_t group, uint32_t groups) {
    extern __shared__ __align__(16) uint32_t smem_q4[];
    const uint32_t row_words = 36 * vecs;  // per row of x: 32 vecs digit words, vecs scales, vecs sums (+ pad to 16 B)
    const uint32_t vpg = group >> 5, vpg_shift = __ffs(vpg) - 1;  // vectors per group; a shift when a power of two
    const bool vpg_pow2 = (vpg & (vpg - 1)) == 0;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t col0 = (blockIdx.x * kWarpsD + warp) * C;
    const uint32_t row0 = blockIdx.y * MR;

    // first weight loads go out before x is converted, so the conversion hides under them
    uint4 wq[C];
#pragma unroll
    for (int c = 0; c < C; ++c)
        wq[c] = (lane < vecs && col0 + c < n) ? ldg_stream4(q + (size_t)(col0 + c) * vecs + lane) : make_uint4(0, 0, 0, 0);

#pragma unroll
    for (int r = 0; r < MR; ++r) {
        uint32_t* xd = smem_q4 + r * row_words;
        float* xinv = reinterpret_cast<float*>(xd + 32 * vecs);
        // rows past m read row m-1 again; their results are never stored
        prepare_x_q4<XVEC>(x + (size_t)min(row0 + r, m - 1) * k, k, vecs, xd, xinv, xinv + vecs);
    }
    __syncthreads();
    if (col0 >= n) return;

    float acc[C][MR];
#pragma unroll
    for (int c = 0; c < C; ++c)
#pragma unroll
        for (int r = 0; r < MR; ++r) acc[c][r] = 0.0f;

    for (uint32_t v = lane; v < vecs; v += 32) {
        uint4 wn[C];  // the next iteration's weights
#pragma unroll
        for (int c = 0; c < C; ++c)
            wn[c] = (v + 32 < vecs && col0 + c < n) ? ldg_stream4(q + (size_t)(col0 + c) * vecs + v + 32) : make_uint4(0, 0, 0, 0);
        float sc[C], mn[C];
        const uint32_t g = vpg_pow2 ? v >> vpg_shift : v / vpg;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const bool ok = col0 + c < n;
            sc[c] = ok ? __ldg(scale + (size_t)(col0 + c) * groups + g) : 0.0f;
            const float z = ok ? __ldg(zero + (size_t)(col0 + c) * groups + g) : 0.0f;
            mn[c] = __fsub_rn(z, __fmul_rn(8.0f, sc[c]));  // min = zero - 8 s
        }
        uint32_t ev[C][4], od[C][4];  // even / odd nibbles of each word, as bytes
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const uint32_t w[4] = {wq[c].x, wq[c].y, wq[c].z, wq[c].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                ev[c][i] = w[i] & 0x0F0F0F0Fu;
                od[c][i] = (w[i] >> 4) & 0x0F0F0F0Fu;
            }
        }
#pragma unroll
        for (int r = 0; r < MR; ++r) {
            const uint32_t* xd = smem_q4 + r * row_words;
            const float* xinv = reinterpret_cast<const float*>(xd + 32 * vecs);
            int D[C][4];
#pragma unroll
            for (int c = 0; c < C; ++c) D[c][0] = D[c][1] = D[c][2] = D[c][3] = 0;
#pragma unroll
            for (int word = 0; word < 4; ++word) {
                const uint4 xe = reinterpret_cast<const uint4*>(xd)[(2 * word) * vecs + v];
                const uint4 xo = reinterpret_cast<const uint4*>(xd)[(2 * word + 1) * vecs + v];
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    D[c][0] = dp4a_ss(ev[c][word], xe.x, D[c][0]);
                    D[c][1] = dp4a_ss(ev[c][word], xe.y, D[c][1]);
                    D[c][2] = dp4a_ss(ev[c][word], xe.z, D[c][2]);
                    D[c][3] = dp4a_ss(ev[c][word], xe.w, D[c][3]);
                    D[c][0] = dp4a_ss(od[c][word], xo.x, D[c][0]);
                    D[c][1] = dp4a_ss(od[c][word], xo.y, D[c][1]);
                    D[c][2] = dp4a_ss(od[c][word], xo.z, D[c][2]);
                    D[c][3] = dp4a_ss(od[c][word], xo.w, D[c][3]);
                }
            }
            const float inv = xinv[v], sum = xinv[vecs + v];
#pragma unroll
            for (int c = 0; c < C; ++c) {
                acc[c][r] = __fmaf_rn(__fmul_rn(sc[c], inv), combine_digits(D[c]), acc[c][r]);
                acc[c][r] = __fmaf_rn(mn[c], sum, acc[c][r]);
            }
        }
#pragma unroll
        for (int c = 0; c < C; ++c) wq[c] = wn[c];
    }

#pragma unroll
    for (int c = 0; c < C; ++c)
#pragma unroll
        for (int r = 0; r < MR; ++r) {
            float p = acc[c][r];
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) p += __shfl_xor_sync(0xffffffffu, p, s);
            if (lane == 0 && col0 + c < n && row0 + r < m) {
                if (bias) p = __fadd_rn(p, bias[col0 + c]);
                y[(size_t)(row0 + r) * n + col0 + c] = p;
            }
        }
}

// ── int8 ────────────────────────────────────────────────────────────────
// Layout per 16-byte weight vector v (16 values, 4 words of 4 bytes): chunk
// j = word; each chunk is four uint32, one per digit plane, holding that
// digit of the word's four x values. xd[(j * vecs + v) * 4 + digit].
template <bool XVEC>
__device__ __forceinline__ void prepare_x_q8(const float* __restrict__ xr, uint32_t k, uint32_t vecs, uint32_t* xd,
                                             float* xinv) {
    for (uint32_t base = 0; base < vecs * 4; base += blockDim.x) {  // one packed word (4 values) per thread
        const uint32_t wd = base + threadIdx.x;
        const bool live = wd < vecs * 4;
        const uint32_t k0 = wd * 4, v = wd >> 2, word = wd & 3;
        float xv[4];
        if (XVEC) {
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            if (live && k0 < k) t = __ldg(reinterpret_cast<const float4*>(xr + k0));
            xv[0] = t.x, xv[1] = t.y, xv[2] = t.z, xv[3] = t.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) xv[j] = (live && k0 + j < k) ? __ldg(xr + k0 + j) : 0.0f;
        }
        float amax = 0.0f;
        bool bad = false;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            amax = fmaxf(amax, fabsf(xv[j]));
            bad |= !(fabsf(xv[j]) <= 3.402823466e+38f);
        }
        if (bad) amax = __uint_as_float(0x7f800000u);
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        if (!live) continue;
        float mult, inv;
        block_scales(amax, mult, inv);
        int d[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) digits_of(__float2int_rn(xv[j] * mult), d[j]);
        uint4 out;
        out.x = pack4(d[0][0], d[1][0], d[2][0], d[3][0]);
        out.y = pack4(d[0][1], d[1][1], d[2][1], d[3][1]);
        out.z = pack4(d[0][2], d[1][2], d[2][2], d[3][2]);
        out.w = pack4(d[0][3], d[1][3], d[2][3], d[3][3]);
        reinterpret_cast<uint4*>(xd)[word * vecs + v] = out;
        if (word == 0) xinv[v] = inv;
    }
}

template <int MR, int C, bool XVEC>
__global__ void __launch_bounds__(kWarpsD * 32) gemv_q8_dp4a_kernel(const float* __restrict__ x, const uint4* __restrict__ q,
                                                                     const float* __restrict__ scale,
                                                                     const float* __restrict__ bias, float* __restrict__ y,
                                                                     uint32_t m, uint32_t k, uint32_t n, uint32_t vecs) {
    extern __shared__ __align__(16) uint32_t smem_q8[];
    const uint32_t row_words = 20 * vecs;  // per row of x: 16 vecs digit words, vecs scales (+ pad to 16 B)
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t col0 = (blockIdx.x * kWarpsD + warp) * C;
    const uint32_t row0 = blockIdx.y * MR;

    uint4 wq[C];
#pragma unroll
    for (int c = 0; c < C; ++c)
        wq[c] = (lane < vecs && col0 + c < n) ? ldg_stream4(q + (size_t)(col0 + c) * vecs + lane) : make_uint4(0, 0, 0, 0);

#pragma unroll
    for (int r = 0; r < MR; ++r) {
        uint32_t* xd = smem_q8 + r * row_words;
        prepare_x_q8<XVEC>(x + (size_t)min(row0 + r, m - 1) * k, k, vecs, xd, reinterpret_cast<float*>(xd + 16 * vecs));
    }
    __syncthreads();
    if (col0 >= n) return;

    float acc[C][MR];
#pragma unroll
    for (int c = 0; c < C; ++c)
#pragma unroll
        for (int r = 0; r < MR; ++r) acc[c][r] = 0.0f;

    for (uint32_t v = lane; v < vecs; v += 32) {
        uint4 wn[C];
#pragma unroll
        for (int c = 0; c < C; ++c)
            wn[c] = (v + 32 < vecs && col0 + c < n) ? ldg_stream4(q + (size_t)(col0 + c) * vecs + v + 32) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int r = 0; r < MR; ++r) {
            const uint32_t* xd = smem_q8 + r * row_words;
            int D[C][4];
#pragma unroll
            for (int c = 0; c < C; ++c) D[c][0] = D[c][1] = D[c][2] = D[c][3] = 0;
#pragma unroll
            for (int word = 0; word < 4; ++word) {
                const uint4 xw = reinterpret_cast<const uint4*>(xd)[word * vecs + v];
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    const uint32_t w = word == 0 ? wq[c].x : word == 1 ? wq[c].y : word == 2 ? wq[c].z : wq[c].w;
                    D[c][0] = dp4a_ss(w, xw.x, D[c][0]);
                    D[c][1] = dp4a_ss(w, xw.y, D[c][1]);
                    D[c][2] = dp4a_ss(w, xw.z, D[c][2]);
                    D[c][3] = dp4a_ss(w, xw.w, D[c][3]);
                }
            }
            const float inv = reinterpret_cast<const float*>(xd + 16 * vecs)[v];
#pragma unroll
            for (int c = 0; c < C; ++c) acc[c][r] = __fmaf_rn(inv, combine_digits(D[c]), acc[c][r]);
        }
#pragma unroll
        for (int c = 0; c < C; ++c) wq[c] = wn[c];
    }

#pragma unroll
    for (int c = 0; c < C; ++c)
#pragma unroll
        for (int r = 0; r < MR; ++r) {
            float p = acc[c][r];
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) p += __shfl_xor_sync(0xffffffffu, p, s);
            if (lane == 0 && col0 + c < n && row0 + r < m) {
                float out = __fmul_rn(p, scale[col0 + c]);  // the row scale multiplies the finished sum
                if (bias) out = __fadd_rn(out, bias[col0 + c]);
                y[(size_t)(row0 + r) * n + col0 + c] = out;
            }
        }
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ── one row of x, balanced over the whole GPU ─────────────────────────────
// The decode case proper (a single row of x). One CTA per SM, each owning a
// contiguous range of output features sized to within one feature of the
// others, so the GPU runs a single wave with no tail and x is converted once
// per SM. Inside a CTA each of the 16 warps takes `base` whole features; the
// CTA's remaining (< 16) features are cut into blocks of 32 vectors that are
// dealt round-robin to the warps and summed through shared memory in a fixed
// order, which is also what keeps every warp busy when the layer has few
// output features. Weight vectors for the next step are requested while the
// current ones are multiplied, two steps deep.
static constexpr int kBalWarps = 16;

template <bool IS4>
struct DigitDot;

template <>
struct DigitDot<true> {  // int4: 8 chunks per vector (even/odd nibbles of 4 words)
    static constexpr int kChunks = 8;
    __device__ __forceinline__ static void run(const uint4& w, const uint4 (&xr)[8], int (&D)[4]) {
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 xe = xr[2 * i], xo = xr[2 * i + 1];
            const uint32_t e = ws[i] & 0x0F0F0F0Fu, o = (ws[i] >> 4) & 0x0F0F0F0Fu;
            D[0] = dp4a_ss(e, xe.x, D[0]);
            D[1] = dp4a_ss(e, xe.y, D[1]);
            D[2] = dp4a_ss(e, xe.z, D[2]);
            D[3] = dp4a_ss(e, xe.w, D[3]);
            D[0] = dp4a_ss(o, xo.x, D[0]);
            D[1] = dp4a_ss(o, xo.y, D[1]);
            D[2] = dp4a_ss(o, xo.z, D[2]);
            D[3] = dp4a_ss(o, xo.w, D[3]);
        }
    }
};

template <>
struct DigitDot<false> {  // int8: 4 chunks per vector (one per word)
    static constexpr int kChunks = 4;
    __device__ __forceinline__ static void run(const uint4& w, const uint4 (&xr)[4], int (&D)[4]) {
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 xw = xr[i];
            D[0] = dp4a_ss(ws[i], xw.x, D[0]);
            D[1] = dp4a_ss(ws[i], xw.y, D[1]);
            D[2] = dp4a_ss(ws[i], xw.z, D[2]);
            D[3] = dp4a_ss(ws[i], xw.w, D[3]);
        }
    }
};

template <bool IS4, int C, bool XVEC>
__global__ void __launch_bounds__(kBalWarps * 32, 1)
    gemv_dp4a_balanced_kernel(const float* __restrict__ x, const uint4* __restrict__ q, const float* __restrict__ scale,
                              const float* __restrict__ zero, const float* __restrict__ bias, float* __restrict__ y,
                              uint32_t k, uint32_t n, uint32_t vecs, uint32_t group, uint32_t groups, uint32_t ublocks) {
    extern __shared__ __align__(16) uint32_t smem_bal[];
    constexpr int kWordsPerVec = DigitDot<IS4>::kChunks * 4;
    const uint4* xd4 = reinterpret_cast<const uint4*>(smem_bal);
    float* xinv = reinterpret_cast<float*>(smem_bal + kWordsPerVec * vecs);
    float* xsum = xinv + vecs;                    // int4 only
    float* partial = xsum + (IS4 ? vecs : 0);     // kBalWarps * ublocks floats

    const uint32_t vpg = IS4 ? group >> 5 : 1, vpg_shift = __ffs(vpg) - 1;
    const bool vpg_pow2 = (vpg & (vpg - 1)) == 0;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // this CTA's features [cb, cb + ncols); the first n % gridDim CTAs take one more
    const uint32_t per = n / gridDim.x, extra = n % gridDim.x;
    const uint32_t cb = blockIdx.x * per + min(blockIdx.x, extra), ncols = per + (blockIdx.x < extra ? 1u : 0u);
    const uint32_t base = ncols / kBalWarps, rem = ncols % kBalWarps;
    const uint32_t wcol = cb + warp * base;  // this warp's whole features [wcol, wcol + base)
    const uint32_t steps = ((base + C - 1) / C) * ublocks;  // (chunk of C features) x (block of 32 vectors)

    auto load_step = [&](uint32_t step, uint4 (&w)[C]) {
        const uint32_t c0 = (step / ublocks) * C, v = (step % ublocks) * 32 + lane;
#pragma unroll
        for (int c = 0; c < C; ++c)
            w[c] = (step < steps && c0 + c < base && v < vecs) ? ldg_stream4(q + (size_t)(wcol + c0 + c) * vecs + v)
                                                               : make_uint4(0, 0, 0, 0);
    };

    // the first two steps' weights are requested before x is converted
    uint4 w0[C], w1[C];
    load_step(0, w0);
    load_step(1, w1);

    if (IS4)
        prepare_x_q4<XVEC>(x, k, vecs, smem_bal, xinv, xsum);
    else
        prepare_x_q8<XVEC>(x, k, vecs, smem_bal, xinv);
    __syncthreads();

    float acc[C];
#pragma unroll
    for (int c = 0; c < C; ++c) acc[c] = 0.0f;

    auto finish = [&](uint32_t col, float p) {  // lane 0 of the warp that holds a feature's full sum
        if (IS4) {
            if (bias) p = __fadd_rn(p, bias[col]);
        } else {
            p = __fmul_rn(p, scale[col]);  // the row scale multiplies the finished sum
            if (bias) p = __fadd_rn(p, bias[col]);
        }
        y[col] = p;
    };

    constexpr int kChunks = DigitDot<IS4>::kChunks;
    auto load_x = [&](uint32_t v, uint4 (&xr)[kChunks]) {  // one register copy of x's digits serves C features
#pragma unroll
        for (int j = 0; j < kChunks; ++j) xr[j] = xd4[j * vecs + v];
    };
    auto accumulate = [&](uint32_t col, uint32_t v, const uint4& w, const uint4 (&xr)[kChunks], float& a) {
        int D[4] = {0, 0, 0, 0};
        DigitDot<IS4>::run(w, xr, D);
        const float t = combine_digits(D);
        if (IS4) {
            const size_t gi = (size_t)col * groups + (vpg_pow2 ? v >> vpg_shift : v / vpg);
            const float s = __ldg(scale + gi);
            const float mn = __fsub_rn(__ldg(zero + gi), __fmul_rn(8.0f, s));  // min = zero - 8 s
            a = __fmaf_rn(__fmul_rn(s, xinv[v]), t, a);
            a = __fmaf_rn(mn, xsum[v], a);
        } else {
            a = __fmaf_rn(xinv[v], t, a);
        }
    };

    for (uint32_t step = 0; step < steps; ++step) {
        uint4 w2[C];
        load_step(step + 2, w2);
        const uint32_t c0 = (step / ublocks) * C, ub = step % ublocks, v = ub * 32 + lane;
        if (v < vecs) {
            uint4 xr[kChunks];
            load_x(v, xr);
#pragma unroll
            for (int c = 0; c < C; ++c)
                if (c0 + c < base) accumulate(wcol + c0 + c, v, w0[c], xr, acc[c]);
        }
        if (ub + 1 == ublocks) {  // the chunk's features are complete
#pragma unroll
            for (int c = 0; c < C; ++c) {
                float p = acc[c];
#pragma unroll
                for (int s = 16; s > 0; s >>= 1) p += __shfl_xor_sync(0xffffffffu, p, s);
                if (lane == 0 && c0 + c < base) finish(wcol + c0 + c, p);
                acc[c] = 0.0f;
            }
        }
#pragma unroll
        for (int c = 0; c < C; ++c) w0[c] = w1[c], w1[c] = w2[c];
    }

    // the CTA's leftover features, one (feature, block of 32 vectors) per warp at a time
    const uint32_t lcol = cb + kBalWarps * base;
    for (uint32_t idx = warp; idx < rem * ublocks; idx += kBalWarps) {
        const uint32_t j = idx / ublocks, v = (idx % ublocks) * 32 + lane;
        float a = 0.0f;
        if (v < vecs) {
            uint4 xr[kChunks];
            load_x(v, xr);
            accumulate(lcol + j, v, ldg_stream4(q + (size_t)(lcol + j) * vecs + v), xr, a);
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) a += __shfl_xor_sync(0xffffffffu, a, s);
        if (lane == 0) partial[idx] = a;
    }
    __syncthreads();
    if (threadIdx.x < rem) {
        float p = 0.0f;
        for (uint32_t u = 0; u < ublocks; ++u) p += partial[threadIdx.x * ublocks + u];
        finish(lcol + threadIdx.x, p);
    }
}

// Shared memory the digit planes of `rows` rows of x need. The caller falls
// back to the float kernel when they do not fit.
size_t dp4a_smem_q4(uint64_t k, int rows) { return (k + 31) / 32 * 36 * 4 * rows; }
size_t dp4a_smem_q8(uint64_t k, int rows) { return (k + 15) / 16 * 20 * 4 * rows; }
static constexpr size_t kMaxSmem = 200 * 1024;

template <int MR, int C>
static void run_q4(cudaStream_t s, const float* x, uint64_t m, uint64_t k, const uint32_t* q, const float* scale,
                   const float* zero, const float* bias, uint64_t n, uint64_t group, float* y) {
    const uint32_t vecs = (uint32_t)((k + 31) / 32), groups = (uint32_t)((k + group - 1) / group);
    const size_t smem = dp4a_smem_q4(k, MR);
    dim3 grid((uint32_t)(((n + C - 1) / C + kWarpsD - 1) / kWarpsD), (uint32_t)((m + MR - 1) / MR));
    const bool xvec = aligned16(x) && k % 4 == 0;
    auto kernel = xvec ? gemv_q4_dp4a_kernel<MR, C, true> : gemv_q4_dp4a_kernel<MR, C, false>;
    if (smem > 48 * 1024) GQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<grid, kWarpsD * 32, smem, s>>>(x, reinterpret_cast<const uint4*>(q), scale, zero, bias, y, (uint32_t)m, (uint32_t)k,
                                            (uint32_t)n, vecs, (uint32_t)group, groups);
}

template <int MR, int C>
static void run_q8(cudaStream_t s, const float* x, uint64_t m, uint64_t k, const uint32_t* q, const float* scale,
                   const float* bias, uint64_t n, float* y) {
    const uint32_t vecs = (uint32_t)((k + 15) / 16);
    const size_t smem = dp4a_smem_q8(k, MR);
    dim3 grid((uint32_t)(((n + C - 1) / C + kWarpsD - 1) / kWarpsD), (uint32_t)((m + MR - 1) / MR));
    const bool xvec = aligned16(x) && k % 4 == 0;
    auto kernel = xvec ? gemv_q8_dp4a_kernel<MR, C, true> : gemv_q8_dp4a_kernel<MR, C, false>;
    if (smem > 48 * 1024) GQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<grid, kWarpsD * 32, smem, s>>>(x, reinterpret_cast<const uint4*>(q), scale, bias, y, (uint32_t)m, (uint32_t)k,
                                            (uint32_t)n, vecs);
}

// Returns false when the shape does not fit (the caller then runs the float kernel).
template <bool IS4>
static bool run_balanced(cudaStream_t s, int sm_count, const float* x, uint64_t k, const uint32_t* q, const float* scale,
                         const float* zero, const float* bias, uint64_t n, uint64_t group, float* y) {
    constexpr int C = 4;
    const uint32_t vecs = (uint32_t)(IS4 ? (k + 31) / 32 : (k + 15) / 16);
    const uint32_t ublocks = (vecs + 31) / 32;
    const uint32_t groups = IS4 ? (uint32_t)((k + group - 1) / group) : 0;
    const size_t smem = ((size_t)vecs * (IS4 ? 34 : 17) + (size_t)kBalWarps * ublocks) * 4;
    if (smem > kMaxSmem) return false;
    const uint32_t grid = (uint32_t)(n < (uint64_t)sm_count ? n : (uint64_t)sm_count);
    const bool xvec = aligned16(x) && k % 4 == 0;
    auto kernel = xvec ? gemv_dp4a_balanced_kernel<IS4, C, true> : gemv_dp4a_balanced_kernel<IS4, C, false>;
    if (smem > 48 * 1024) GQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<grid, kBalWarps * 32, smem, s>>>(x, reinterpret_cast<const uint4*>(q), scale, zero, bias, y, (uint32_t)k, (uint32_t)n,
                                              vecs, (uint32_t)group, groups, ublocks);
    return true;
}

bool launch_gemv_q4_dp4a(cudaStream_t s, int sm_count, const float* x, uint64_t m, uint64_t k, const uint32_t* q, const float* scale,
                         const float* zero, const float* bias, uint64_t n, uint64_t group, float* y) {
    if (m == 1 && run_balanced<true>(s, sm_count, x, k, q, scale, zero, bias, n, group, y)) return true;
    if (m >= 3 && dp4a_smem_q4(k, 4) <= kMaxSmem)
        run_q4<4, 2>(s, x, m, k, q, scale, zero, bias, n, group, y);
    else if (m >= 2 && dp4a_smem_q4(k, 2) <= kMaxSmem)
        run_q4<2, 4>(s, x, m, k, q, scale, zero, bias, n, group, y);
    else if (dp4a_smem_q4(k, 1) <= kMaxSmem)
        run_q4<1, 4>(s, x, m, k, q, scale, zero, bias, n, group, y);
    else
        return false;
    return true;
}

bool launch_gemv_q8_dp4a(cudaStream_t s, int sm_count, const float* x, uint64_t m, uint64_t k, const uint32_t* q, const float* scale,
                         const float* bias, uint64_t n, float* y) {
    if (m == 1 && run_balanced<false>(s, sm_count, x, k, q, scale, nullptr, bias, n, 32, y)) return true;
    if (m >= 3 && dp4a_smem_q8(k, 4) <= kMaxSmem)
        run_q8<4, 2>(s, x, m, k, q, scale, bias, n, y);
    else if (m >= 2 && dp4a_smem_q8(k, 2) <= kMaxSmem)
        run_q8<2, 4>(s, x, m, k, q, scale, bias, n, y);
    else if (dp4a_smem_q8(k, 1) <= kMaxSmem)
        run_q8<1, 4>(s, x, m, k, q, scale, bias, n, y);
    else
        return false;
    return true;
}

}  // namespace gq
