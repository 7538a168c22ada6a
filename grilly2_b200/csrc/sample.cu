// Next-token selection on the device, one CTA per row of logits, so that a
// generate loop reads back nothing but token ids: Hugging Face's processors in
// generate()'s order, then the draw.
//   repetition penalty over the tokens so far:  x < 0 ? x * r : x / r
//   greedy: the first index of the maximum
//   sampling: temperature x / t; top_k (drop what is below the k-th largest
//   value, ties with it stay); top_p (in ascending order drop tokens whose
//   cumulative probability is <= 1 - p, the largest always stays); then a draw
//   from the softmax of the rest by the inverse CDF in token order, with one
//   uniform number per row that the caller supplies.
// Replaces crates/grilly-infer/src/sampling.rs + shaders/g2-sample.glsl:1-60
// (same processors, same tie rules; no sort: top_k is a radix select of the
// k-th largest order-preserving key, top_p a binary search over keys for the
// smallest value whose cumulative mass passes (1 - p) Z).
//
// What is new here: the uniform numbers and the history live on the DEVICE and
// are indexed by device counters (a draw counter, a history length), so a
// captured decode step that ends in this kernel replays correctly: every
// replay takes the next uniform number and appends its token to the history.
//
// Structure: after the scores, the candidates — what top_k kept or, without
// top_k, everything not -inf — are compacted in token order into shared memory
// when there are at most kCap of them (Hugging Face's default top_k = 50 always
// is); top_p, the ties and the draw then run on that list. Larger candidate
// sets take the same steps over the whole row in global memory. Every sum is
// compensated (Kahan) per thread and combined in a fixed order: the result
// depends on the inputs and u only.
// Bound: one pass over the row per radix digit; latency, not bytes.
#include "gq_internal.h"

namespace gq {

namespace {

constexpr int kWG = 1024;
constexpr uint32_t kCap = 4096;

__device__ __forceinline__ uint32_t fkey(float f) {  // a < b as floats <=> fkey(a) < fkey(b) as unsigned
    const uint32_t b = __float_as_uint(f);
    return (b >> 31) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float kfloat(uint32_t k) { return __uint_as_float((k >> 31) ? (k & 0x7FFFFFFFu) : ~k); }
__device__ __forceinline__ void kahan(float& sum, float& comp, float v) {
    const float y = __fsub_rn(v, comp), t = __fadd_rn(sum, y);
    comp = __fsub_rn(__fsub_rn(t, sum), y);
    sum = t;
}

struct Shared {
    float red_f[kWG];
    uint32_t red_u[kWG];
    uint32_t bins[256];
    uint32_t pick[2];
    float pick_f;
    uint32_t tie_at;
    uint32_t c_key[kCap];
    uint32_t c_idx[kCap];
    float c_ex[kCap];
};

__device__ float sum_all(Shared& sh, float v) {  // fixed tree: the same result whatever the timing
    const uint32_t tid = threadIdx.x;
    sh.red_f[tid] = v;
    __syncthreads();
    for (uint32_t s = kWG / 2; s > 0; s >>= 1) {
        if (tid < s) sh.red_f[tid] = __fadd_rn(sh.red_f[tid], sh.red_f[tid + s]);
        __syncthreads();
    }
    const float r = sh.red_f[0];
    __syncthreads();
    return r;
}
__device__ uint32_t sum_all_u(Shared& sh, uint32_t v) {
    const uint32_t tid = threadIdx.x;
    sh.red_u[tid] = v;
    __syncthreads();
    for (uint32_t s = kWG / 2; s > 0; s >>= 1) {
        if (tid < s) sh.red_u[tid] += sh.red_u[tid + s];
        __syncthreads();
    }
    const uint32_t r = sh.red_u[0];
    __syncthreads();
    return r;
}
__device__ uint32_t max_all(Shared& sh, uint32_t v) {
    const uint32_t tid = threadIdx.x;
    sh.red_u[tid] = v;
    __syncthreads();
    for (uint32_t s = kWG / 2; s > 0; s >>= 1) {
        if (tid < s) sh.red_u[tid] = max(sh.red_u[tid], sh.red_u[tid + s]);
        __syncthreads();
    }
    const uint32_t r = sh.red_u[0];
    __syncthreads();
    return r;
}

// The key of the need-th largest score (1 <= need <= n): four passes of 8-bit digits from the top.
__device__ uint32_t radix_kth(Shared& sh, const float* scores, uint32_t n, uint32_t need) {
    const uint32_t tid = threadIdx.x;
    uint32_t prefix = 0, mask = 0;
    for (int d = 3; d >= 0; --d) {
        const uint32_t shift = 8u * d;
        if (tid < 256) sh.bins[tid] = 0;
        __syncthreads();
        for (uint32_t i = tid; i < n; i += kWG) {
            const uint32_t k = fkey(scores[i]);
            if ((k & mask) == prefix) atomicAdd(&sh.bins[(k >> shift) & 0xFFu], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t cum = 0;
            sh.pick[0] = 0, sh.pick[1] = need;
            for (int b = 255; b >= 0; --b) {
                const uint32_t c = sh.bins[b];
                if (cum + c >= need) {
                    sh.pick[0] = (uint32_t)b, sh.pick[1] = need - cum;
                    break;
                }
                cum += c;
            }
        }
        __syncthreads();
        prefix |= sh.pick[0] << shift, mask |= 0xFFu << shift, need = sh.pick[1];
        __syncthreads();
    }
    return prefix;
}

struct Params {
    const float* logits;
    const int32_t* history;  // [rows][hist_cap] or null
    uint32_t* hist_len;      // device word (null with no history)
    const float* uniforms;   // [*][rows]
    uint32_t* draws;         // device word: how many draws have been made; this launch uses row `draws` of uniforms
    float* scores;           // [rows][v] scratch
    float* ex;               // [rows][v] scratch
    int32_t* tokens;         // [rows]
    float* probs;            // [rows][v] or null: the filtered distribution
    uint32_t* ticket;        // zero between launches: the last CTA to finish advances the counters
    uint32_t v, rows, hist_cap, uniform_rows, top_k;
    float temperature, penalty, one_minus_p;
    uint32_t do_sample, use_temperature, use_top_p, append;
};

__device__ __forceinline__ bool kept_key(uint32_t k, uint32_t i, uint32_t kcut, uint32_t tie_start) {
    return k > kcut || (k == kcut && i >= tie_start);
}

__global__ void __launch_bounds__(kWG, 1) sample_kernel(Params p) {
    extern __shared__ uint8_t sample_smem[];
    Shared& sh = *reinterpret_cast<Shared*>(sample_smem);
    const uint32_t row = blockIdx.x, tid = threadIdx.x, n = p.v;
    const float* logits = p.logits + (size_t)row * n;
    float* scores = p.scores + (size_t)row * n;
    float* ex = p.ex + (size_t)row * n;
    GQ_GRID_DEP_SYNC();
    const uint32_t hist_len = p.history ? min(*reinterpret_cast<volatile uint32_t*>(p.hist_len), p.hist_cap) : 0u;
    const uint32_t draw = *reinterpret_cast<volatile uint32_t*>(p.draws);
    auto scaled = [&](float x) { return p.use_temperature ? __fdiv_rn(x, p.temperature) : x; };
    int32_t chosen_token = -1;

    // ── scores: penalty, then temperature ──
    for (uint32_t i = tid; i < n; i += kWG) scores[i] = scaled(logits[i]);
    __syncthreads();
    if (p.history && p.penalty != 1.0f) {
        // repeats of a token write the same value, as a gather followed by a scatter does
        for (uint32_t h = tid; h < hist_len; h += kWG) {
            const int32_t tok = p.history[(size_t)row * p.hist_cap + h];
            if (tok >= 0 && (uint32_t)tok < n) {
                const float x = logits[tok];
                scores[tok] = scaled(x < 0.0f ? __fmul_rn(x, p.penalty) : __fdiv_rn(x, p.penalty));
            }
        }
        __syncthreads();
    }

    if (!p.do_sample) {
        // greedy: the first index of the maximum (NaN never wins; an all-NaN row gives index 0 as the comparison falls through)
        unsigned long long best = 0ull;
        for (uint32_t i = tid; i < n; i += kWG) {
            const float s = scores[i];
            const unsigned long long key = ((unsigned long long)(s == s ? fkey(s) : 0u) << 32) | (0xFFFFFFFFu - i);
            best = key > best ? key : best;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        unsigned long long* red = reinterpret_cast<unsigned long long*>(sh.red_f);
        if ((tid & 31) == 0) red[tid >> 5] = best;
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < kWG / 32; ++w) best = red[w] > best ? red[w] : best;
            chosen_token = (int32_t)(0xFFFFFFFFu - (uint32_t)best);
        }
    } else {
        // ── top_k: the key of the k-th largest score; -inf scores have no probability and are never kept ──
        uint32_t kmin = 0;
        if (p.top_k > 0 && p.top_k < n) kmin = radix_kth(sh, scores, n, p.top_k);
        kmin = max(kmin, fkey(__uint_as_float(0xff800000u)) + 1u);
        uint32_t mk = 0;
        for (uint32_t i = tid; i < n; i += kWG) {
            const float s = scores[i];
            if (s == s) mk = max(mk, fkey(s));
        }
        const uint32_t kmax = max_all(sh, mk);
        const float m = kfloat(kmax);
        const uint32_t chunk = (n + kWG - 1) / kWG, start = min(tid * chunk, n), end = min(start + chunk, n);
        bool done = false;

        if (kmax >= kmin) {
            // ── candidates in shared memory when they fit ──
            uint32_t cnt = 0;
            for (uint32_t i = start; i < end; ++i) {
                const float s = scores[i];
                if (s == s && fkey(s) >= kmin) cnt++;
            }
            const uint32_t total = sum_all_u(sh, cnt);
            if (total <= kCap) {
                sh.red_u[tid] = cnt;
                __syncthreads();
                if (tid == 0) {
                    uint32_t acc = 0;
                    for (uint32_t t = 0; t < kWG; ++t) {
                        const uint32_t c = sh.red_u[t];
                        sh.red_u[t] = acc, acc += c;
                    }
                }
                __syncthreads();
                uint32_t at = sh.red_u[tid];
                __syncthreads();
                for (uint32_t i = start; i < end; ++i) {
                    const float s = scores[i];
                    if (s == s && fkey(s) >= kmin) sh.c_key[at] = fkey(s), sh.c_idx[at] = i, sh.c_ex[at] = expf(s - m), at++;
                }
                __syncthreads();
                uint32_t kcut = kmin, tie_start = 0;
                if (p.use_top_p) {
                    float cm = 0.f, cc = 0.f;
                    for (uint32_t j = tid; j < total; j += kWG) kahan(cm, cc, sh.c_ex[j]);
                    const float target = __fmul_rn(p.one_minus_p, sum_all(sh, cm + cc));
                    uint32_t lo = kmin, hi = kmax;
                    while (lo < hi) {  // uniform: every thread sees the same sums
                        const uint32_t mid = lo + (hi - lo) / 2;
                        float part = 0.f, pc = 0.f;
                        for (uint32_t j = tid; j < total; j += kWG)
                            if (sh.c_key[j] <= mid) kahan(part, pc, sh.c_ex[j]);
                        if (sum_all(sh, part + pc) > target) hi = mid;
                        else lo = mid + 1;
                    }
                    kcut = lo;
                    // Ties at the cut: in ascending order each is dropped while the cumulative mass is still <= target: with
                    // `below` the mass under the cut and q each tie's mass that drops floor((target - below) / q), never all.
                    float bm = 0.f, bc = 0.f;
                    uint32_t ties = 0;
                    for (uint32_t j = tid; j < total; j += kWG) {
                        if (sh.c_key[j] < kcut) kahan(bm, bc, sh.c_ex[j]);
                        if (sh.c_key[j] == kcut) ties++;
                    }
                    const float below = sum_all(sh, bm + bc);
                    const uint32_t g = sum_all_u(sh, ties);
                    if (g > 1) {
                        const float q = expf(kfloat(kcut) - m);
                        const uint32_t drop = (uint32_t)fminf(fmaxf(floorf(__fdiv_rn(target - below, q)), 0.0f), (float)(g - 1));
                        if (tid == 0) {
                            uint32_t seen = 0;
                            sh.tie_at = 0;
                            for (uint32_t j = 0; j < total; ++j)
                                if (sh.c_key[j] == kcut) {
                                    if (seen == drop) {
                                        sh.tie_at = sh.c_idx[j];
                                        break;
                                    }
                                    seen++;
                                }
                        }
                        __syncthreads();
                        tie_start = sh.tie_at;
                        __syncthreads();
                    }
                }
                // the draw: inverse CDF in token order over the candidates; a chunk of the list per thread
                const uint32_t cchunk = (total + kWG - 1) / kWG, cs = min(tid * cchunk, total), ce = min(cs + cchunk, total);
                float s1 = 0.f, c1 = 0.f;
                for (uint32_t j = cs; j < ce; ++j)
                    if (kept_key(sh.c_key[j], sh.c_idx[j], kcut, tie_start)) kahan(s1, c1, sh.c_ex[j]);
                sh.red_f[tid] = s1 + c1;
                __syncthreads();
                if (tid == 0) {
                    float tot = 0.f, tc = 0.f;
                    for (uint32_t t = 0; t < kWG; ++t) kahan(tot, tc, sh.red_f[t]);
                    tot += tc;
                    const float u = p.uniforms[(size_t)(draw % p.uniform_rows) * p.rows + row];
                    float target = __fmul_rn(u, tot), before = 0.f, bcomp = 0.f;
                    uint32_t owner = 0xFFFFFFFFu, last = 0xFFFFFFFFu;
                    for (uint32_t t = 0; t < kWG; ++t)
                        if (sh.red_f[t] > 0.f) {
                            last = t;
                            if ((before + bcomp) + sh.red_f[t] > target) {
                                owner = t;
                                break;
                            }
                            kahan(before, bcomp, sh.red_f[t]);
                        }
                    if (owner == 0xFFFFFFFFu && last != 0xFFFFFFFFu) {  // rounding put the target at the very end
                        owner = last, before = 0.f, bcomp = 0.f;
                        for (uint32_t t = 0; t < last; ++t) kahan(before, bcomp, sh.red_f[t]);
                        target = (before + bcomp) + sh.red_f[last];
                    }
                    sh.pick[0] = owner, sh.pick_f = target - (before + bcomp), sh.red_f[0] = tot;
                }
                __syncthreads();
                const uint32_t owner = sh.pick[0];
                const float tot = sh.red_f[0];
                if (tid == owner) {
                    float acc = 0.f, ac = 0.f;
                    uint32_t chosen = 0xFFFFFFFFu, lastkept = 0xFFFFFFFFu;
                    for (uint32_t j = cs; j < ce; ++j)
                        if (kept_key(sh.c_key[j], sh.c_idx[j], kcut, tie_start)) {
                            if (sh.c_ex[j] > 0.f) lastkept = sh.c_idx[j];
                            kahan(acc, ac, sh.c_ex[j]);
                            if (acc + ac > sh.pick_f) {
                                chosen = sh.c_idx[j];
                                break;
                            }
                        }
                    if (chosen == 0xFFFFFFFFu) chosen = lastkept;
                    sh.pick[1] = chosen;
                }
                __syncthreads();
                if (tid == 0) chosen_token = owner == 0xFFFFFFFFu ? -1 : (int32_t)sh.pick[1];
                if (p.probs) {
                    float* pr = p.probs + (size_t)row * n;
                    for (uint32_t i = tid; i < n; i += kWG) pr[i] = 0.f;
                    __syncthreads();
                    for (uint32_t j = tid; j < total; j += kWG)
                        if (kept_key(sh.c_key[j], sh.c_idx[j], kcut, tie_start)) pr[sh.c_idx[j]] = __fdiv_rn(sh.c_ex[j], tot);
                }
                done = true;
            }
        }
        if (!done) {
            // ── the same steps over the whole row ──
            for (uint32_t i = tid; i < n; i += kWG) {
                const float s = scores[i];
                ex[i] = (s == s && fkey(s) >= kmin && kmax >= kmin) ? expf(s - m) : 0.f;
            }
            __syncthreads();
            uint32_t kcut = kmin, tie_start = 0;
            if (p.use_top_p && kmax >= kmin) {
                float z = 0.f, zc = 0.f;
                for (uint32_t i = tid; i < n; i += kWG) kahan(z, zc, ex[i]);
                const float target = __fmul_rn(p.one_minus_p, sum_all(sh, z + zc));
                uint32_t lo = kmin, hi = kmax;
                while (lo < hi) {
                    const uint32_t mid = lo + (hi - lo) / 2;
                    float part = 0.f, pc = 0.f;
                    for (uint32_t i = tid; i < n; i += kWG)
                        if (fkey(scores[i]) <= mid) kahan(part, pc, ex[i]);
                    if (sum_all(sh, part + pc) > target) hi = mid;
                    else lo = mid + 1;
                }
                kcut = lo;
                float bm = 0.f, bc = 0.f;
                uint32_t ties = 0;
                for (uint32_t i = start; i < end; ++i) {
                    const uint32_t k = fkey(scores[i]);
                    if (k >= kmin && k < kcut) kahan(bm, bc, ex[i]);
                    if (k == kcut) ties++;
                }
                const float below = sum_all(sh, bm + bc);
                const uint32_t g = sum_all_u(sh, ties);
                if (g > 1) {
                    const float q = expf(kfloat(kcut) - m);
                    const uint32_t drop = (uint32_t)fminf(fmaxf(floorf(__fdiv_rn(target - below, q)), 0.0f), (float)(g - 1));
                    if (drop > 0) {  // the index of tie number `drop` in index order
                        sh.red_u[tid] = ties;
                        __syncthreads();
                        if (tid == 0) {
                            uint32_t seen = 0;
                            sh.pick[0] = 0, sh.pick[1] = 0;
                            for (uint32_t t = 0; t < kWG; ++t) {
                                if (seen + sh.red_u[t] > drop) {
                                    sh.pick[0] = t, sh.pick[1] = drop - seen;
                                    break;
                                }
                                seen += sh.red_u[t];
                            }
                        }
                        __syncthreads();
                        if (tid == sh.pick[0]) {
                            uint32_t j = 0;
                            for (uint32_t i = start; i < end; ++i)
                                if (fkey(scores[i]) == kcut) {
                                    if (j == sh.pick[1]) {
                                        sh.tie_at = i;
                                        break;
                                    }
                                    j++;
                                }
                        }
                        __syncthreads();
                        tie_start = sh.tie_at;
                        __syncthreads();
                    }
                }
            }
            float cs = 0.f, cc = 0.f;
            for (uint32_t i = start; i < end; ++i)
                if (kept_key(fkey(scores[i]), i, kcut, tie_start)) kahan(cs, cc, ex[i]);
            sh.red_f[tid] = cs + cc;
            __syncthreads();
            if (tid == 0) {
                float tot = 0.f, tc = 0.f;
                for (uint32_t t = 0; t < kWG; ++t) kahan(tot, tc, sh.red_f[t]);
                tot += tc;
                const float u = p.uniforms[(size_t)(draw % p.uniform_rows) * p.rows + row];
                float target = __fmul_rn(u, tot), before = 0.f, bcomp = 0.f;
                uint32_t owner = 0xFFFFFFFFu, last = 0xFFFFFFFFu;
                for (uint32_t t = 0; t < kWG; ++t)
                    if (sh.red_f[t] > 0.f) {
                        last = t;
                        if ((before + bcomp) + sh.red_f[t] > target) {
                            owner = t;
                            break;
                        }
                        kahan(before, bcomp, sh.red_f[t]);
                    }
                if (owner == 0xFFFFFFFFu && last != 0xFFFFFFFFu) {
                    owner = last, before = 0.f, bcomp = 0.f;
                    for (uint32_t t = 0; t < last; ++t) kahan(before, bcomp, sh.red_f[t]);
                    target = (before + bcomp) + sh.red_f[last];
                }
                sh.pick[0] = owner, sh.pick_f = target - (before + bcomp), sh.red_f[0] = tot;
            }
            __syncthreads();
            const uint32_t owner = sh.pick[0];
            const float tot = sh.red_f[0];
            if (tid == owner) {
                float acc = 0.f, ac = 0.f;
                uint32_t chosen = start, lastkept = start;
                bool found = false;
                for (uint32_t i = start; i < end; ++i)
                    if (kept_key(fkey(scores[i]), i, kcut, tie_start)) {
                        const float e = ex[i];
                        if (e > 0.f) lastkept = i;
                        kahan(acc, ac, e);
                        if (acc + ac > sh.pick_f) {
                            chosen = i, found = true;
                            break;
                        }
                    }
                sh.pick[1] = found ? chosen : lastkept;
            }
            __syncthreads();
            if (tid == 0) chosen_token = owner == 0xFFFFFFFFu ? -1 : (int32_t)sh.pick[1];  // nothing to draw from: -1
            if (p.probs) {
                float* pr = p.probs + (size_t)row * n;
                for (uint32_t i = tid; i < n; i += kWG)
                    pr[i] = (owner != 0xFFFFFFFFu && kept_key(fkey(scores[i]), i, kcut, tie_start)) ? __fdiv_rn(ex[i], tot) : 0.f;
            }
        }
    }

    if (tid == 0) {
        p.tokens[row] = chosen_token;
        if (p.history && p.append && hist_len < p.hist_cap) const_cast<int32_t*>(p.history)[(size_t)row * p.hist_cap + hist_len] = chosen_token;
        __threadfence();
        if (atomicAdd(p.ticket, 1u) == gridDim.x - 1) {  // every row has read the counters: advance them for the next step
            *p.ticket = 0;
            if (p.do_sample) *p.draws = draw + 1;
            if (p.history && p.append && hist_len < p.hist_cap) *p.hist_len = hist_len + 1;
        }
    }
}

}  // namespace

uint64_t sample_state_bytes() { return 64; }

void launch_sample(cudaStream_t s, const float* logits, uint64_t rows, uint64_t v, int32_t* history, uint64_t hist_cap, uint32_t* hist_len,
                   bool do_sample, float temperature, uint64_t top_k, float one_minus_p, float penalty, const float* uniforms,
                   uint64_t uniform_rows, uint32_t* draws, float* scores, float* ex, int32_t* tokens, float* probs, bool append, void* state) {
    Params p{};
    p.logits = logits, p.history = history, p.hist_len = hist_len, p.uniforms = uniforms, p.draws = draws, p.scores = scores, p.ex = ex;
    p.tokens = tokens, p.probs = probs, p.ticket = reinterpret_cast<uint32_t*>(state);
    p.v = (uint32_t)v, p.rows = (uint32_t)rows, p.hist_cap = (uint32_t)hist_cap, p.uniform_rows = (uint32_t)(uniform_rows ? uniform_rows : 1);
    p.top_k = do_sample ? (uint32_t)(top_k > 0xffffffffull ? 0xffffffffull : top_k) : 0u;
    p.temperature = temperature, p.penalty = penalty, p.one_minus_p = one_minus_p;
    p.do_sample = do_sample, p.use_temperature = do_sample && temperature != 1.0f, p.use_top_p = do_sample && one_minus_p > 0.0f, p.append = append;
    GQ_CUDA(cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Shared)));
    launch_after(sample_kernel, dim3((uint32_t)rows), dim3(kWG), sizeof(Shared), s, p);
}

}  // namespace gq
