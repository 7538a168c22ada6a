// Device arithmetic shared by the decode-step operators and the GEMV prologues that fuse them.
#pragma once

#include <cstdint>

namespace gq {

// exp as the reference computes it (Cephes expf, g2-common.glsl:21-31), with
// every operation rounded on its own so that the CPU oracle can match it.
__device__ __forceinline__ float exp_cephes(float v) {
    if (v > 88.72283935546875f) return __uint_as_float(0x7f800000u);
    if (v < -103.97207641601562f) return 0.0f;
    const float k = floorf(__fadd_rn(__fmul_rn(v, 1.44269504088896341f), 0.5f));
    float r = __fsub_rn(v, __fmul_rn(k, 0.693359375f));
    r = __fadd_rn(r, __fmul_rn(k, 2.12194440e-4f));
    const float z = __fmul_rn(r, r);
    float p = 1.9875691500e-4f;
    p = __fadd_rn(__fmul_rn(p, r), 1.3981999507e-3f);
    p = __fadd_rn(__fmul_rn(p, r), 8.3334519073e-3f);
    p = __fadd_rn(__fmul_rn(p, r), 4.1665795894e-2f);
    p = __fadd_rn(__fmul_rn(p, r), 1.6666665459e-1f);
    p = __fadd_rn(__fmul_rn(p, r), 5.0000001201e-1f);
    const float yv = __fadd_rn(__fadd_rn(__fmul_rn(p, z), r), 1.0f);
    return ldexpf(yv, (int)k);
}

// (g * sigmoid(g)) * u, sigmoid evaluated on -|g| so that exp never overflows (g2-swiglu.glsl:21-29, g2-common.glsl:163-166).
__device__ __forceinline__ float silu_mul(float g, float u) {
    const float e = exp_cephes(-fabsf(g));
    const float sg = g >= 0.0f ? __fdiv_rn(1.0f, __fadd_rn(1.0f, e)) : __fdiv_rn(e, __fadd_rn(1.0f, e));
    return __fmul_rn(__fmul_rn(g, sg), u);
}

// The same with the hardware's exp2 and reciprocal approximations (about 1e-6 relative): for the GEMV prologue, where every CTA
// evaluates the whole row again and the exact form's ~60 instructions per value would cost more than the launch it saves.
__device__ __forceinline__ float silu_mul_fast(float g, float u) {
    const float e = __expf(-fabsf(g));
    const float r = __fdividef(1.0f, 1.0f + e);
    return g * (g >= 0.0f ? r : e * r) * u;
}

// What a fused GEMV does to its input row before multiplying (one row of x only):
//   kind 1: h = x + residual (residual may be null), h_out = h (if not null), x' = h / sqrt(mean(h^2) + eps) * w
//           — add_rms_norm_kernel's arithmetic, the sum of squares in float64;
//   kind 2: x'[j] = silu(x[j]) * x[k + j] — swiglu_kernel's, to about 1e-6 relative (silu_mul_fast).
struct Prologue {
    const float* res = nullptr;
    const float* w = nullptr;
    float* h_out = nullptr;
    float eps = 0.0f;
};

}  // namespace gq
