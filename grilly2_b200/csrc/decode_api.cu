// C ABI of the decode-step operators (include/gq.h, "decode step"): argument
// checks against buffer sizes, then the launchers of decode_ops.cu.
#include "gq_internal.h"
#include "math_common.cuh"

using namespace gq;

extern "C" {

int32_t gq_embedding(gq_ctx* ctx, gq_buf table, gq_buf ids, uint64_t rows, uint64_t width, uint64_t vocab, gq_buf out) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_embedding", rows, width, vocab);
        auto tp = (const float*)view(ctx, table, 0, vocab * width, 4, "gq_embedding table");
        auto ip = (const int32_t*)view(ctx, ids, 0, rows, 4, "gq_embedding ids");
        auto op = (float*)view(ctx, out, 0, rows * width, 4, "gq_embedding output");
        if (rows == 0 || width == 0) return;
        launch_embedding(ctx->stream, tp, ip, rows, width, vocab, op);
        after_launch(ctx, "embedding", {table, ids, out}, {out});
    });
}

int32_t gq_add_rms_norm(gq_ctx* ctx, gq_buf x, gq_buf residual, gq_buf weight, uint64_t rows, uint64_t n, float eps, gq_buf y,
                        gq_buf h) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_add_rms_norm", rows, n);
        if (n == 0) fail("gq_add_rms_norm: rows of no elements");
        auto xp = (const float*)view(ctx, x, 0, rows * n, 4, "gq_add_rms_norm input");
        auto rp = residual ? (const float*)view(ctx, residual, 0, rows * n, 4, "gq_add_rms_norm residual") : nullptr;
        auto wp = weight ? (const float*)view(ctx, weight, 0, n, 4, "gq_add_rms_norm weight") : nullptr;
        auto yp = (float*)view(ctx, y, 0, rows * n, 4, "gq_add_rms_norm output");
        auto hp = h ? (float*)view(ctx, h, 0, rows * n, 4, "gq_add_rms_norm sum output") : nullptr;
        if (rows == 0) return;
        launch_add_rms_norm(ctx->stream, xp, rp, wp, rows, n, eps, yp, hp);
        after_launch(ctx, "add_rms_norm", {x, residual, weight, y, h}, {y, h});
    });
}

static void check_heads(const char* op, uint64_t heads, uint64_t kv_heads, uint64_t dim, uint64_t max_len) {
    check_dims(op, heads, kv_heads, dim);
    check_dims(op, max_len, 1);
    if (heads == 0 || kv_heads == 0 || heads % kv_heads) fail("%s: %llu heads do not group over %llu kv heads", op, (unsigned long long)heads, (unsigned long long)kv_heads);
    if (dim != 32 && dim != 64 && dim != 128) fail("%s: head_dim must be 32, 64 or 128, got %llu", op, (unsigned long long)dim);
    if (max_len == 0) fail("%s: a cache of no positions", op);
}

int32_t gq_rope_kv_append(gq_ctx* ctx, gq_buf qkv, gq_buf cos, gq_buf sin, gq_buf lens, uint64_t layer, uint64_t layers, uint64_t heads,
                          uint64_t kv_heads, uint64_t dim, uint64_t max_len, gq_buf q_out, gq_buf kcache, uint64_t k_off, gq_buf vcache,
                          uint64_t v_off) {
    return guarded([&] {
        Locked l(ctx);
        check_heads("gq_rope_kv_append", heads, kv_heads, dim, max_len);
        if (layer >= layers) fail("gq_rope_kv_append: layer %llu of %llu", (unsigned long long)layer, (unsigned long long)layers);
        auto qp = (const float*)view(ctx, qkv, 0, (heads + 2 * kv_heads) * dim, 4, "gq_rope_kv_append qkv");
        auto cp = (const float*)view(ctx, cos, 0, max_len * dim, 4, "gq_rope_kv_append cos");
        auto sp = (const float*)view(ctx, sin, 0, max_len * dim, 4, "gq_rope_kv_append sin");
        auto lp = (const uint32_t*)view(ctx, lens, 0, layers, 4, "gq_rope_kv_append cursor");
        auto op = (float*)view(ctx, q_out, 0, heads * dim, 4, "gq_rope_kv_append q output");
        auto kp = (float*)view(ctx, kcache, k_off, kv_heads * max_len * dim, 4, "gq_rope_kv_append key cache");
        auto vp = (float*)view(ctx, vcache, v_off, kv_heads * max_len * dim, 4, "gq_rope_kv_append value cache");
        launch_rope_kv_append(ctx->stream, qp, cp, sp, lp, (uint32_t)layer, (uint32_t)heads, (uint32_t)kv_heads, (uint32_t)dim,
                              (uint32_t)max_len, op, kp, vp);
        after_launch(ctx, "rope_kv_append", {qkv, cos, sin, lens, q_out, kcache, vcache}, {q_out, kcache, vcache});
    });
}

int32_t gq_kv_advance(gq_ctx* ctx, gq_buf lens, uint64_t layers, uint64_t max_len) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_kv_advance", layers, max_len);
        auto lp = (uint32_t*)view(ctx, lens, 0, layers, 4, "gq_kv_advance cursor");
        if (layers == 0) return;
        launch_kv_advance(ctx->stream, lp, (uint32_t)layers, (uint32_t)max_len);
        after_launch(ctx, "kv_advance", {lens}, {lens});
    });
}

int32_t gq_attn_scratch_bytes(gq_ctx* ctx, uint64_t heads, uint64_t dim, uint64_t max_len, uint64_t* out) {
    return guarded([&] {
        Locked l(ctx);
        if (!out) fail("gq_attn_scratch_bytes: null out pointer");
        check_heads("gq_attn_scratch_bytes", heads, heads, dim, max_len);
        const uint32_t splits = attn_splits((uint32_t)heads, (uint32_t)max_len, ctx->prop.multiProcessorCount);
        *out = attn_scratch_floats((uint32_t)heads, (uint32_t)dim, splits) * 4;
    });
}

int32_t gq_attn_decode(gq_ctx* ctx, gq_buf q, gq_buf kcache, uint64_t k_off, gq_buf vcache, uint64_t v_off, gq_buf lens, uint64_t layer,
                       uint64_t layers, uint64_t heads, uint64_t kv_heads, uint64_t dim, uint64_t max_len, float scale, gq_buf scratch,
                       gq_buf out) {
    return guarded([&] {
        Locked l(ctx);
        check_heads("gq_attn_decode", heads, kv_heads, dim, max_len);
        if (layer >= layers) fail("gq_attn_decode: layer %llu of %llu", (unsigned long long)layer, (unsigned long long)layers);
        const uint32_t splits = attn_splits((uint32_t)heads, (uint32_t)max_len, ctx->prop.multiProcessorCount);
        auto qp = (const float*)view(ctx, q, 0, heads * dim, 4, "gq_attn_decode q");
        auto kp = (float*)view(ctx, kcache, k_off, kv_heads * max_len * dim, 4, "gq_attn_decode key cache");
        auto vp = (float*)view(ctx, vcache, v_off, kv_heads * max_len * dim, 4, "gq_attn_decode value cache");
        auto lp = (const uint32_t*)view(ctx, lens, 0, layers, 4, "gq_attn_decode cursor");
        auto sp = (float*)view(ctx, scratch, 0, attn_scratch_floats((uint32_t)heads, (uint32_t)dim, splits), 4, "gq_attn_decode scratch");
        auto op = (float*)view(ctx, out, 0, heads * dim, 4, "gq_attn_decode output");
        launch_attn_decode(ctx->stream, qp, kp, vp, lp, (uint32_t)layer, (uint32_t)heads, (uint32_t)kv_heads, (uint32_t)dim,
                           (uint32_t)max_len, scale, splits, sp, op);
        after_launch(ctx, "attn_decode", {q, kcache, vcache, lens, scratch, out}, {scratch, out});
    });
}

int32_t gq_attn_decode_rope(gq_ctx* ctx, gq_buf qkv, gq_buf cos, gq_buf sin, gq_buf kcache, uint64_t k_off, gq_buf vcache, uint64_t v_off,
                            gq_buf lens, uint64_t layer, uint64_t layers, uint64_t heads, uint64_t kv_heads, uint64_t dim, uint64_t max_len,
                            float scale, gq_buf scratch, gq_buf out) {
    return guarded([&] {
        Locked l(ctx);
        check_heads("gq_attn_decode_rope", heads, kv_heads, dim, max_len);
        if (layer >= layers) fail("gq_attn_decode_rope: layer %llu of %llu", (unsigned long long)layer, (unsigned long long)layers);
        const uint32_t splits = attn_splits((uint32_t)heads, (uint32_t)max_len, ctx->prop.multiProcessorCount);
        auto qp = (const float*)view(ctx, qkv, 0, (heads + 2 * kv_heads) * dim, 4, "gq_attn_decode_rope qkv");
        auto cp = (const float*)view(ctx, cos, 0, max_len * dim, 4, "gq_attn_decode_rope cos");
        auto sp = (const float*)view(ctx, sin, 0, max_len * dim, 4, "gq_attn_decode_rope sin");
        auto kp = (float*)view(ctx, kcache, k_off, kv_heads * max_len * dim, 4, "gq_attn_decode_rope key cache");
        auto vp = (float*)view(ctx, vcache, v_off, kv_heads * max_len * dim, 4, "gq_attn_decode_rope value cache");
        auto lp = (const uint32_t*)view(ctx, lens, 0, layers, 4, "gq_attn_decode_rope cursor");
        auto scp = (float*)view(ctx, scratch, 0, attn_scratch_floats((uint32_t)heads, (uint32_t)dim, splits), 4, "gq_attn_decode_rope scratch");
        auto op = (float*)view(ctx, out, 0, heads * dim, 4, "gq_attn_decode_rope output");
        if (((uintptr_t)qp | (uintptr_t)cp | (uintptr_t)sp | (uintptr_t)kp | (uintptr_t)vp) & 15) fail("gq_attn_decode_rope: buffers and cache offsets must be 16-byte aligned");
        launch_attn_decode(ctx->stream, qp, kp, vp, lp, (uint32_t)layer, (uint32_t)heads, (uint32_t)kv_heads, (uint32_t)dim,
                           (uint32_t)max_len, scale, splits, scp, op, cp, sp, weights_settled(ctx, {kcache, vcache, lens, cos, sin, scratch}));
        after_launch(ctx, "attn_decode_rope", {qkv, cos, sin, kcache, vcache, lens, scratch, out}, {kcache, vcache, scratch, out});
    });
}

int32_t gq_attn_prefill(gq_ctx* ctx, gq_buf qkv, uint64_t rows, gq_buf cos, gq_buf sin, gq_buf kcache, uint64_t k_off, gq_buf vcache, uint64_t v_off,
                        gq_buf kscale, gq_buf vscale, gq_buf lens, uint64_t layer, uint64_t layers, uint64_t heads, uint64_t kv_heads, uint64_t dim,
                        uint64_t max_len, float scale, gq_buf q_scratch, gq_buf out) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_attn_prefill", rows, heads * dim, max_len);
        check_dims("gq_attn_prefill", kv_heads, layers);
        if (heads == 0 || kv_heads == 0 || heads % kv_heads)
            fail("gq_attn_prefill: %llu heads do not group over %llu kv heads", (unsigned long long)heads, (unsigned long long)kv_heads);
        if (dim != 32 && dim != 64 && dim != 128) fail("gq_attn_prefill: head_dim must be 32, 64 or 128, got %llu", (unsigned long long)dim);
        if (max_len == 0) fail("gq_attn_prefill: a cache of no positions");
        if (layer >= layers) fail("gq_attn_prefill: layer %llu of %llu", (unsigned long long)layer, (unsigned long long)layers);
        if ((kscale == 0) != (vscale == 0)) fail("gq_attn_prefill: an int8 cache needs both scale buffers");
        const bool q8 = kscale != 0;
        if (k_off % dim || v_off % dim) fail("gq_attn_prefill: cache offsets must be whole rows (multiples of head_dim)");
        const uint64_t qsz = heads * dim, kvsz = kv_heads * dim, cache = kv_heads * max_len * dim;
        auto qp = (const float*)view(ctx, qkv, 0, rows * (qsz + 2 * kvsz), 4, "gq_attn_prefill qkv");
        auto cp = (const float*)view(ctx, cos, 0, max_len * dim, 4, "gq_attn_prefill cos");
        auto sp = (const float*)view(ctx, sin, 0, max_len * dim, 4, "gq_attn_prefill sin");
        void* kp = view(ctx, kcache, k_off, cache, q8 ? 1 : 4, "gq_attn_prefill key cache");
        void* vp = view(ctx, vcache, v_off, cache, q8 ? 1 : 4, "gq_attn_prefill value cache");
        auto ksp = q8 ? (float*)view(ctx, kscale, k_off / dim, kv_heads * max_len, 4, "gq_attn_prefill key scales") : nullptr;
        auto vsp = q8 ? (float*)view(ctx, vscale, v_off / dim, kv_heads * max_len, 4, "gq_attn_prefill value scales") : nullptr;
        auto lp = (const uint32_t*)view(ctx, lens, 0, layers, 4, "gq_attn_prefill cursor");
        auto qs = (float*)view(ctx, q_scratch, 0, rows * qsz, 4, "gq_attn_prefill rotated queries");
        auto op = (float*)view(ctx, out, 0, rows * qsz, 4, "gq_attn_prefill output");
        if (ranges_overlap(op, rows * qsz * 4, qs, rows * qsz * 4)) fail("gq_attn_prefill: the output must not be the rotated-query scratch");
        if (rows == 0) return;
        launch_rope_append_rows(ctx->stream, qp, cp, sp, lp, (uint32_t)layer, (uint32_t)rows, (uint32_t)heads, (uint32_t)kv_heads, (uint32_t)dim,
                                (uint32_t)max_len, qs, kp, vp, ksp, vsp, q8);
        launch_attn_prefill(ctx->stream, qs, kp, vp, ksp, vsp, lp, (uint32_t)layer, (uint32_t)rows, (uint32_t)heads, (uint32_t)kv_heads, (uint32_t)dim,
                            (uint32_t)max_len, scale, op, q8);
        ctx->stats.launches++;
        after_launch(ctx, "attn_prefill", {qkv, cos, sin, kcache, vcache, kscale, vscale, lens, q_scratch, out}, {});
    });
}

int32_t gq_kv_advance_by(gq_ctx* ctx, gq_buf lens, uint64_t layers, uint64_t max_len, uint64_t count) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_kv_advance_by", layers, max_len, count);
        auto lp = (uint32_t*)view(ctx, lens, 0, layers, 4, "gq_kv_advance_by cursor");
        if (layers == 0 || count == 0) return;
        launch_kv_advance_by(ctx->stream, lp, (uint32_t)layers, (uint32_t)max_len, (uint32_t)count);
        after_launch(ctx, "kv_advance_by", {lens}, {});
    });
}

int32_t gq_swiglu(gq_ctx* ctx, gq_buf gate_up, uint64_t rows, uint64_t width, gq_buf out) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_swiglu", rows, 2 * width);
        auto gp = (const float*)view(ctx, gate_up, 0, rows * 2 * width, 4, "gq_swiglu input");
        auto op = (float*)view(ctx, out, 0, rows * width, 4, "gq_swiglu output");
        if (rows == 0 || width == 0) return;
        launch_swiglu(ctx->stream, gp, rows, width, op);
        after_launch(ctx, "swiglu", {gate_up, out}, {out});
    });
}

int32_t gq_argmax_rows(gq_ctx* ctx, gq_buf v, uint64_t rows, uint64_t n, gq_buf out) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_argmax_rows", rows, n);
        if (n == 0) fail("gq_argmax_rows: rows of no elements");
        auto vp = (const float*)view(ctx, v, 0, rows * n, 4, "gq_argmax_rows input");
        auto op = (int32_t*)view(ctx, out, 0, rows, 4, "gq_argmax_rows output");
        if (rows == 0) return;
        launch_argmax_rows(ctx->stream, vp, rows, n, op, ctx->argmax_state);
        after_launch(ctx, "argmax_rows", {v, out}, {out});
    });
}

int32_t gq_sample(gq_ctx* ctx, gq_buf logits, uint64_t rows, uint64_t vocab, gq_buf history, uint64_t hist_cap, gq_buf hist_len, uint32_t append,
                  uint32_t do_sample, double temperature, uint64_t top_k, double top_p, double repetition_penalty, gq_buf uniforms,
                  uint64_t uniform_rows, gq_buf draws, gq_buf scratch, gq_buf tokens, gq_buf probs) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_sample", rows, vocab, hist_cap);
        if (vocab == 0) fail("gq_sample: expected (batch, vocab) with vocab > 0");
        // Hugging Face's checks, with its messages (crates/grilly-infer/src/sampling.rs:70-96)
        if (!(repetition_penalty > 0.0)) fail("`penalty` has to be a strictly positive float, but is %g", repetition_penalty);
        if (do_sample) {
            if (!(temperature > 0.0))
                fail("`temperature` (=%g) has to be a strictly positive float, otherwise your next token scores will be invalid. If you're "
                     "looking for greedy decoding strategies, set `do_sample=False`.", temperature);
            if (!(top_p >= 0.0 && top_p <= 1.0)) fail("`top_p` has to be a float > 0 and < 1, but is %g", top_p);
        }
        auto lp = (const float*)view(ctx, logits, 0, rows * vocab, 4, "gq_sample logits");
        auto hp = history ? (int32_t*)view(ctx, history, 0, rows * hist_cap, 4, "gq_sample history") : nullptr;
        auto hl = history ? (uint32_t*)view(ctx, hist_len, 0, 1, 4, "gq_sample history length") : nullptr;
        auto up = do_sample ? (const float*)view(ctx, uniforms, 0, uniform_rows * rows, 4, "gq_sample uniforms") : nullptr;
        if (do_sample && uniform_rows == 0) fail("gq_sample: sampling needs at least one row of uniform numbers");
        auto dp = (uint32_t*)view(ctx, draws, 0, 1, 4, "gq_sample draw counter");
        auto sp = (float*)view(ctx, scratch, 0, 2 * rows * vocab, 4, "gq_sample scratch");
        auto tp = (int32_t*)view(ctx, tokens, 0, rows, 4, "gq_sample tokens");
        auto pp = probs ? (float*)view(ctx, probs, 0, rows * vocab, 4, "gq_sample probabilities") : nullptr;
        if (rows == 0) return;
        launch_sample(ctx->stream, lp, rows, vocab, hp, hist_cap, hl, do_sample != 0, (float)temperature, top_k, (float)(1.0 - top_p),
                      (float)repetition_penalty, up, uniform_rows, dp, sp, sp + rows * vocab, tp, pp, append != 0, ctx->sample_state);
        after_launch(ctx, "sample", {logits, history, hist_len, uniforms, draws, scratch, tokens, probs}, {});
    });
}

int32_t gq_int8_linear_norm(gq_ctx* ctx, gq_buf x, gq_buf residual, gq_buf norm_weight, float eps, gq_buf h_out, uint64_t k, gq_buf q,
                            gq_buf scale, gq_buf bias, uint64_t b_off, uint64_t n, gq_buf y) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_int8_linear_norm", 1, k, n);
        if (k == 0 || n == 0) fail("gq_int8_linear_norm: an empty layer");
        Prologue pro;
        auto xp = (const float*)view(ctx, x, 0, k, 4, "gq_int8_linear_norm input");
        pro.res = residual ? (const float*)view(ctx, residual, 0, k, 4, "gq_int8_linear_norm residual") : nullptr;
        pro.w = (const float*)view(ctx, norm_weight, 0, k, 4, "gq_int8_linear_norm norm weight");
        pro.h_out = h_out ? (float*)view(ctx, h_out, 0, k, 4, "gq_int8_linear_norm sum output") : nullptr;
        pro.eps = eps;
        auto qp = (const uint32_t*)view(ctx, q, 0, n * 4 * ((k + 15) / 16), 4, "gq_int8_linear_norm q");
        auto sp = (const float*)view(ctx, scale, 0, n, 4, "gq_int8_linear_norm scale");
        auto bp = bias ? (const float*)view(ctx, bias, b_off, n, 4, "gq_int8_linear_norm bias") : nullptr;
        auto yp = (float*)view(ctx, y, 0, n, 4, "gq_int8_linear_norm output");
        // Every CTA re-reads x and residual for the row's norm while CTA 0 already stores h_out: in place would be a race.
        if (ranges_overlap(pro.h_out, k * 4, xp, k * 4) || ranges_overlap(pro.h_out, k * 4, pro.res, k * 4))
            fail("gq_int8_linear_norm: h_out must not overlap x or residual (every CTA reads them while one writes h_out); "
                 "use gq_add_rms_norm, which is safe in place, or a separate buffer");
        if (ranges_overlap(yp, n * 4, xp, k * 4) || ranges_overlap(yp, n * 4, pro.res, k * 4) || ranges_overlap(yp, n * 4, pro.h_out, k * 4) ||
            ranges_overlap(yp, n * 4, pro.w, k * 4))
            fail("gq_int8_linear_norm: the output must not overlap x, residual, the norm weight or h_out");
        if (!launch_gemv_q8_imma_fused(ctx->stream, ctx->prop.multiProcessorCount, ctx->status_dev, xp, k, qp, sp, bp, n, yp, 1, pro,
                                       weights_settled(ctx, {q, scale})))
            fail("gq_int8_linear_norm: in_features = %llu must be a multiple of 4 that fits shared memory, and the buffers 16-byte aligned", (unsigned long long)k);
        after_launch(ctx, "gemv_q8_imma_norm", {x, residual, norm_weight, h_out, q, scale, bias, y}, {y, h_out});
    });
}

int32_t gq_int8_linear_swiglu(gq_ctx* ctx, gq_buf gate_up, uint64_t k, gq_buf q, gq_buf scale, gq_buf bias, uint64_t b_off, uint64_t n,
                              gq_buf y) {
    return guarded([&] {
        Locked l(ctx);
        check_dims("gq_int8_linear_swiglu", 1, 2 * k, n);
        if (k == 0 || n == 0) fail("gq_int8_linear_swiglu: an empty layer");
        auto xp = (const float*)view(ctx, gate_up, 0, 2 * k, 4, "gq_int8_linear_swiglu input");
        auto qp = (const uint32_t*)view(ctx, q, 0, n * 4 * ((k + 15) / 16), 4, "gq_int8_linear_swiglu q");
        auto sp = (const float*)view(ctx, scale, 0, n, 4, "gq_int8_linear_swiglu scale");
        auto bp = bias ? (const float*)view(ctx, bias, b_off, n, 4, "gq_int8_linear_swiglu bias") : nullptr;
        auto yp = (float*)view(ctx, y, 0, n, 4, "gq_int8_linear_swiglu output");
        if (ranges_overlap(yp, n * 4, xp, 2 * k * 4)) fail("gq_int8_linear_swiglu: the output must not overlap gate_up");
        if (!launch_gemv_q8_imma_fused(ctx->stream, ctx->prop.multiProcessorCount, ctx->status_dev, xp, k, qp, sp, bp, n, yp, 2, Prologue(),
                                       weights_settled(ctx, {q, scale})))
            fail("gq_int8_linear_swiglu: in_features = %llu must be a multiple of 4 that fits shared memory, and the input 16-byte aligned", (unsigned long long)k);
        after_launch(ctx, "gemv_q8_imma_swiglu", {gate_up, q, scale, bias, y}, {y});
    });
}

}  // extern "C"
