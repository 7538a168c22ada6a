/* oracle.c — CPU restatement of grilly2's weight-only quantized linear arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the product path may call this file:
 * it exists so the CUDA kernels can be checked against the reference's
 * arithmetic, and so a CPU baseline can be timed beside them.
 *
 * The reference runs this arithmetic as GLSL compute shaders; each function
 * here follows one shader (cited by its path within the reference project)
 * statement by statement, in the shader's order of floating-point operations:
 *   - div_rn(a, b)   -> IEEE a / b     (crates/grilly-core/shaders/g2-common.glsl:125-137
 *                                       is proven equal to it by
 *                                       crates/grilly-core/tests/div_rn.rs:73-99)
 *   - roundEven(v)   -> rintf(v) under the default rounding mode
 *   - fma(a, b, c)   -> fmaf(a, b, c)  and nowhere else: build with
 *                                       -ffp-contract=off so the compiler
 *                                       fuses nothing on its own
 *   - bitfieldExtract(word, 8j, 8) -> sign-extending byte read
 *
 * Parity pin: the reference cannot be built here (Rust + Vulkan), so this
 * file is pinned against (a) the host formulas the reference's own tests use
 * as their oracle (crates/grilly-infer/tests/quant.rs:40-53,
 * crates/grilly-infer/tests/quant4.rs:41-66, tests/python/test_quantization.py:38-43,172-190),
 * on the reference tests' own shape lists and edge cases, and (b) the
 * reference's numpy int4 quantizer python/grilly/infer/gptq.py:51-65, run in
 * the build container to produce the committed fixtures under tests/golden/.
 *
 * Packed layouts (crates/grilly-infer/src/quant.rs:84-94, quant4.rs:69-81):
 *   int8: row r is words8 = 4*ceil(k/16) little-endian 32-bit words, four
 *         two's-complement int8 each, zero padded to whole 16-byte vectors.
 *   int4: row r is words4 = 4*ceil(k/32) words, eight 4-bit levels each, low
 *         nibble first, zero padded; scale/zero are (rows, ceil(k/group)).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))
#define FLT_EPS_F32 1.1920928955078125e-7f

static inline int64_t words8_of(int64_t k) { return (k + 15) / 16 * 4; }
static inline int64_t words4_of(int64_t k) { return (k + 31) / 32 * 4; }
static inline int64_t imin64(int64_t a, int64_t b) { return a < b ? a : b; }

ORACLE_API int64_t oq_words8(int64_t k) { return words8_of(k); }
ORACLE_API int64_t oq_words4(int64_t k) { return words4_of(k); }

/* ── int8 per-row ─────────────────────────────────────────────────────── */

/* crates/grilly-core/shaders/g2-quantize-q8.glsl:22-53. max is
 * order-independent, so the shader's strided scan + tree is a plain scan. */
ORACLE_API void oq_quantize_q8(const float* w, int64_t rows, int64_t k, uint32_t* q, float* scale) {
    const int64_t words = words8_of(k);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float* wr = w + r * k;
        float m = 0.0f;
        for (int64_t i = 0; i < k; ++i) m = fmaxf(m, fabsf(wr[i]));
        float sc = fmaxf(m / 127.5f, FLT_EPS_F32);
        float inv = 1.0f / sc;
        for (int64_t word = 0; word < words; ++word) {
            uint32_t packed = 0;
            for (int j = 0; j < 4; ++j) {
                int64_t i = word * 4 + j;
                if (i < k) {
                    float v = wr[i] * inv;
                    float rr = rintf(v);
                    rr = fminf(fmaxf(rr, -128.0f), 127.0f);
                    int qv = (int)rr;
                    packed |= ((uint32_t)qv & 0xFFu) << (8 * j);
                }
            }
            q[r * words + word] = packed;
        }
        scale[r] = sc;
    }
}

static inline float q8_at(const uint32_t* qrow, int64_t i) {
    uint32_t word = qrow[i >> 2];
    return (float)(int8_t)((word >> (8 * (i & 3))) & 0xFFu);
}

/* crates/grilly-core/shaders/g2-dequantize-q8.glsl:15-21 */
ORACLE_API void oq_dequantize_q8(const uint32_t* q, const float* scale, int64_t rows, int64_t k, float* w) {
    const int64_t words = words8_of(k);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t i = 0; i < k; ++i) w[r * k + i] = q8_at(q + r * words, i) * scale[r];
}

/* crates/grilly-core/shaders/g2-linear-q8.glsl:33-95 — the decode kernel.
 * 64 lanes per output feature; lane l chains the FMAs of vectors l, l+64, …
 * (16 values each, in order); the 64 partials are then added by the fixed
 * tree partial[t] += partial[t + stride], stride = 32 … 1; the row's scale
 * multiplies the finished sum and the bias is added last. The vec4 and
 * scalar x paths of the shader run the same FMAs in the same order. */
ORACLE_API void oq_linear_q8(const float* x, int64_t m, int64_t k, const uint32_t* q, const float* scale,
                             const float* bias, int64_t n, float* y) {
    const int64_t words = words8_of(k), vecs = words / 4;
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < n; ++c) {
        const uint32_t* qrow = q + c * words;
        for (int64_t r = 0; r < m; ++r) {
            const float* xr = x + r * k;
            float partial[64];
            for (int lane = 0; lane < 64; ++lane) {
                float acc = 0.0f;
                for (int64_t v = lane; v < vecs; v += 64) {
                    int64_t k0 = v * 16, count = imin64(16, k - k0);
                    for (int64_t j = 0; j < count; ++j) acc = fmaf(xr[k0 + j], q8_at(qrow, k0 + j), acc);
                }
                partial[lane] = acc;
            }
            for (int stride = 32; stride > 0; stride >>= 1)
                for (int lane = 0; lane < stride; ++lane) partial[lane] += partial[lane + stride];
            float v = partial[0] * scale[c];
            if (bias) v += bias[c];
            y[r * n + c] = v;
        }
    }
}

/* crates/grilly-core/shaders/g2-linear-q8-tiled.glsl:41-100 — the prefill
 * kernel: every accumulator chains its k FMAs in k order (:78-85), then
 * * scale, + bias (:95-96). */
ORACLE_API void oq_linear_q8_tiled(const float* x, int64_t m, int64_t k, const uint32_t* q, const float* scale,
                                   const float* bias, int64_t n, float* y) {
    const int64_t words = words8_of(k);
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < n; ++c) {
        const uint32_t* qrow = q + c * words;
        for (int64_t r = 0; r < m; ++r) {
            const float* xr = x + r * k;
            float acc = 0.0f;
            for (int64_t i = 0; i < k; ++i) acc = fmaf(xr[i], q8_at(qrow, i), acc);
            float v = acc * scale[c];
            if (bias) v += bias[c];
            y[r * n + c] = v;
        }
    }
}

/* float64 evaluation of scale * sum(x * q) + bias, and of the magnitude
 * scale * sum|x * q| + |bias| the reference's error bound is stated in
 * (crates/grilly-infer/tests/quant.rs:146-160). */
ORACLE_API void oq_linear_q8_f64(const float* x, int64_t m, int64_t k, const uint32_t* q, const float* scale,
                                 const float* bias, int64_t n, double* y, double* mag) {
    const int64_t words = words8_of(k);
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < n; ++c) {
        const uint32_t* qrow = q + c * words;
        for (int64_t r = 0; r < m; ++r) {
            double dot = 0.0, ab = 0.0;
            for (int64_t i = 0; i < k; ++i) {
                double p = (double)x[r * k + i] * (double)q8_at(qrow, i);
                dot += p;
                ab += fabs(p);
            }
            double bv = bias ? (double)bias[c] : 0.0;
            y[r * n + c] = dot * (double)scale[c] + bv;
            if (mag) mag[r * n + c] = ab * (double)scale[c] + fabs(bv);
        }
    }
}

/* ── int4 group-wise ──────────────────────────────────────────────────── */

/* crates/grilly-core/shaders/g2-quantize-q4.glsl:30-70 */
ORACLE_API void oq_quantize_q4(const float* w, int64_t rows, int64_t k, int64_t group, uint32_t* q, float* scale,
                               float* zero) {
    const int64_t words = words4_of(k), groups = (k + group - 1) / group;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float* wr = w + r * k;
        uint32_t* qr = q + r * words;
        memset(qr, 0, (size_t)words * 4);
        for (int64_t g = 0; g < groups; ++g) {
            int64_t start = g * group, end = imin64(k, start + group);
            if (start >= end) {
                scale[r * groups + g] = 1.0f;
                zero[r * groups + g] = 0.0f;
                continue;
            }
            float lo = wr[start], hi = lo;
            for (int64_t i = start + 1; i < end; ++i) {
                lo = fminf(lo, wr[i]);
                hi = fmaxf(hi, wr[i]);
            }
            float s = fmaxf((hi - lo) / 15.0f, FLT_EPS_F32);
            scale[r * groups + g] = s;
            float eight_s = 8.0f * s;
            zero[r * groups + g] = lo + eight_s;
            for (int64_t i = start; i < end; ++i) {
                float d = wr[i] - lo;
                float lv = rintf(d / s);
                lv = fminf(fmaxf(lv, 0.0f), 15.0f);
                qr[i >> 3] |= (uint32_t)(int)lv << ((i & 7) * 4);
            }
        }
    }
}

static inline float q4_at(const uint32_t* qrow, int64_t i) {
    return (float)((qrow[i >> 3] >> ((i & 7) * 4)) & 0xFu);
}

/* crates/grilly-core/shaders/g2-dequantize-q4.glsl:16-24 */
ORACLE_API void oq_dequantize_q4(const uint32_t* q, const float* scale, const float* zero, int64_t rows, int64_t k,
                                 int64_t group, float* w) {
    const int64_t words = words4_of(k), groups = (k + group - 1) / group;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t i = 0; i < k; ++i) {
            float s = scale[r * groups + i / group];
            float eight_s = 8.0f * s;
            float lo = zero[r * groups + i / group] - eight_s;
            w[r * k + i] = fmaf(q4_at(q + r * words, i), s, lo);
        }
}

/* crates/grilly-core/shaders/g2-linear-q4.glsl:43-111. Per 16-byte vector
 * (32 levels, one group): dot chains 32 FMAs from 0, sum adds x — four at a
 * time as (x0+x1)+(x2+x3) when x_vec4 (the shader's vec4 path, taken when
 * x's offset and k are multiples of 4), one at a time otherwise — then
 * acc = fma(s, dot, acc); acc = fma(zero - 8 s, sum, acc). Lanes and tree as
 * in the int8 kernel; bias last. */
ORACLE_API void oq_linear_q4(const float* x, int64_t m, int64_t k, const uint32_t* q, const float* scale,
                             const float* zero, const float* bias, int64_t n, int64_t group, int x_vec4, float* y) {
    const int64_t words = words4_of(k), vecs = words / 4, groups = (k + group - 1) / group;
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < n; ++c) {
        const uint32_t* qrow = q + c * words;
        for (int64_t r = 0; r < m; ++r) {
            const float* xr = x + r * k;
            float partial[64];
            for (int lane = 0; lane < 64; ++lane) {
                float acc = 0.0f;
                for (int64_t v = lane; v < vecs; v += 64) {
                    int64_t k0 = v * 32, g = k0 / group;
                    float s = scale[c * groups + g];
                    float eight_s = 8.0f * s;
                    float lo = zero[c * groups + g] - eight_s;
                    int64_t count = imin64(32, k - k0);
                    float dot = 0.0f, sum = 0.0f;
                    if (x_vec4) {
                        for (int64_t j = 0; 4 * j < count; ++j) {
                            const float* xv = xr + k0 + 4 * j;
                            dot = fmaf(q4_at(qrow, k0 + 4 * j), xv[0], dot);
                            dot = fmaf(q4_at(qrow, k0 + 4 * j + 1), xv[1], dot);
                            dot = fmaf(q4_at(qrow, k0 + 4 * j + 2), xv[2], dot);
                            dot = fmaf(q4_at(qrow, k0 + 4 * j + 3), xv[3], dot);
                            float a = xv[0] + xv[1], b = xv[2] + xv[3];
                            sum += a + b;
                        }
                    } else {
                        for (int64_t j = 0; j < count; ++j) {
                            dot = fmaf(q4_at(qrow, k0 + j), xr[k0 + j], dot);
                            sum += xr[k0 + j];
                        }
                    }
                    acc = fmaf(s, dot, acc);
                    acc = fmaf(lo, sum, acc);
                }
                partial[lane] = acc;
            }
            for (int stride = 32; stride > 0; stride >>= 1)
                for (int lane = 0; lane < stride; ++lane) partial[lane] += partial[lane + stride];
            float v = partial[0];
            if (bias) v += bias[c];
            y[r * n + c] = v;
        }
    }
}

/* float64 evaluation of x @ dequantize(w)^T + bias with the weight taken as
 * level * s + (zero - 8 s) in float64 from the float32 parameters, and the
 * magnitude sum|x * w| + |bias| (crates/grilly-infer/tests/quant4.rs:176-196). */
ORACLE_API void oq_linear_q4_f64(const float* x, int64_t m, int64_t k, const uint32_t* q, const float* scale,
                                 const float* zero, const float* bias, int64_t n, int64_t group, double* y,
                                 double* mag) {
    const int64_t words = words4_of(k), groups = (k + group - 1) / group;
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < n; ++c) {
        const uint32_t* qrow = q + c * words;
        for (int64_t r = 0; r < m; ++r) {
            double dot = 0.0, ab = 0.0;
            for (int64_t i = 0; i < k; ++i) {
                double s = scale[c * groups + i / group], z = zero[c * groups + i / group];
                double wv = (double)q4_at(qrow, i) * s + (z - 8.0 * s);
                double p = (double)x[r * k + i] * wv;
                dot += p;
                ab += fabs(p);
            }
            double bv = bias ? (double)bias[c] : 0.0;
            y[r * n + c] = dot + bv;
            if (mag) mag[r * n + c] = ab + fabs(bv);
        }
    }
}

/* python/grilly/infer/quantization.py:236-244 — Int4Tensor.from_parts' host
 * packer: (rows, k) levels 0..15 -> (rows, words4) words, low nibble first. */
ORACLE_API void oq_pack_levels_q4(const uint8_t* levels, int64_t rows, int64_t k, uint32_t* q) {
    const int64_t words = words4_of(k);
    memset(q, 0, (size_t)(rows * words) * 4);
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t i = 0; i < k; ++i)
            q[r * words + (i >> 3)] |= (uint32_t)(levels[r * k + i] & 0xFu) << ((i & 7) * 4);
}

ORACLE_API int oq_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORACLE_API void oq_set_threads(int n) {
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    omp_set_num_threads(n > 0 ? n : 1);
#else
    (void)n;
#endif
}
