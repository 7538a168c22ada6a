/* gq.h — C ABI of the B200 (sm_100a) backend for grilly2's weight-only
 * quantized linear path: int8 per-row and int4 group-wise weights, their
 * packers, the dequant-fused linear, and capture/replay as CUDA graphs.
 *
 * It takes the place, for these operators only, of the reference's Vulkan
 * shim: crates/grilly-sys/shim/gc_shim.h:78-126 (gc_create … gc_submit) and
 * the per-operator "signatures" (binding order + push-constant words) that
 * crates/grilly-infer/src/quant.rs:18-46 and quant4.rs:26-46 declare for
 * gc_dispatch. The conventions are that shim's (gc_shim.h:1-16):
 *
 *  - every function returns GQ_OK or GQ_ERR; on GQ_ERR the message is
 *    available from gq_last_error() on the same thread until the next
 *    failing call on that thread. No C++ exception crosses this boundary,
 *    and misuse (bad handle, wrong size, bad shape) is reported, never a
 *    device fault: every operator checks its operands against the sizes of
 *    the buffers it was given before it launches anything.
 *  - the context is opaque; buffers are 64-bit handles, 0 is never valid.
 *    The caller owns the context and every handle it creates and releases
 *    handles before gq_destroy. Allocations stay on this side.
 *  - tensors are contiguous row-major float32 / 32-bit words located by an
 *    ELEMENT offset into a whole buffer, as the reference's kernels receive
 *    them (crates/grilly-core/src/kernel.rs:26-36), so an input may start at
 *    any element; aligned fast paths are chosen inside.
 *  - all work is asynchronous on the context's one CUDA stream, in call
 *    order. gq_download and gq_synchronize wait for it. There is no batch to
 *    open or submit.
 *  - every call on a context is serialised on that context's mutex.
 *
 * Packed weight layouts are the reference's, bit for bit
 * (crates/grilly-infer/src/quant.rs:84-94, quant4.rs:69-81), so a weight
 * packed by either side is readable by the other:
 *   int8: q[rows][words8] int32 words, words8 = 4*ceil(k/16); four
 *         two's-complement int8 per word, little-endian; rows zero padded to
 *         whole 16-byte vectors; scale[rows] float32.
 *   int4: q[rows][words4] int32 words, words4 = 4*ceil(k/32); eight 4-bit
 *         levels per word, low nibble first; zero padded;
 *         scale[rows][groups], zero[rows][groups] float32,
 *         groups = ceil(k/group).
 */
#ifndef GQ_H
#define GQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(GQ_BUILD) && defined(__GNUC__)
#pragma GCC visibility push(default) /* the library hides everything else */
#endif

typedef struct gq_ctx gq_ctx;
typedef struct gq_graph gq_graph;
typedef struct gq_comm gq_comm;
typedef uint64_t gq_buf; /* 0 is never a valid handle */

#define GQ_OK 0
#define GQ_ERR 1

/* Memory classes; the values are gc_shim.h:33-41's. */
#define GQ_MEM_DEVICE 0            /* pooled device memory (activations, outputs) */
#define GQ_MEM_DEVICE_PERSISTENT 3 /* exactly the size asked for, never pooled, counted in
                                      persistent_bytes / persistent_peak: weights and quantized data */

/* Which kernel a linear runs. AUTO picks by shape (see gq_int8_linear). */
#define GQ_KERNEL_AUTO 0
#define GQ_KERNEL_GEMV 1   /* dequant-fused float32 GEMV in the reference shader's summation order:
                              bit-identical to the reference's arithmetic, bounded by the FP32 pipes */
#define GQ_KERNEL_TENSOR 2 /* tcgen05 tensor-core GEMM (tf32), dequantised in shared memory */
#define GQ_KERNEL_DP4A 3   /* GEMV on integer dot products (dp4a) against exact fixed-point digit planes of x,
                              within float32 rounding of GQ_KERNEL_GEMV; any group size, up to 16 rows */
#define GQ_KERNEL_UMMA 5   /* decode linear on tcgen05 (kind::i8, accumulators in tensor memory), weights fed to the
                              tensor core by TMA exactly as they lie in HBM. int8: one or two rows of x. int4 (group_size
                              128, in_features a multiple of 128): 1 to 16 rows of x in ONE pass over the weight */
#define GQ_KERNEL_IMMA 4   /* the same arithmetic on the warp-level int8 tensor instruction: the fast path for
                              one or two rows of x (int4: group_size a multiple of 128) */
#define GQ_KERNEL_RING 6   /* int4 group-128 decode on the warp-level int8 tensor instruction with K split by group over the
                              warps (digits of x in registers, weights through a deep ring of bulk copies): in_features 4096
                              or 8192, up to four rows of x per launch and up to 16 in passes: what AUTO picks there */

#define GQ_KERNEL_TENSOR_I8 7 /* int8 only: the prefill GEMM in exact integer arithmetic on tcgen05 (kind::i8): x as three
                                 signed base-256 digit planes of a per-row fixed-point integer (error 2^-23 of the row's
                                 largest |x| per element), the packed weight fed to the tensor core as it lies in HBM, digits
                                 joined as a 64-bit integer in the epilogue. Tiles of 256 features x 80 rows of x for prefill,
                                 128 features x 16 / 32 / 64 rows for decode batches, so a few rows cost one pass over the
                                 weight. What AUTO picks from three rows of x on (inside a capture in which the context's
                                 scratch would have to grow it falls back to dp4a, from 64 rows to GQ_KERNEL_TENSOR) */

#define GQ_KERNEL_UMMA_LANES 8 /* int4 only (group_size 128, in_features a multiple of 128 up to 16384, 1 to 16 rows of x): the
                                  tcgen05 decode kernel with the operands exchanged, the output features on the lanes of
                                  tensor memory, so that a read-out thread owns one feature and its scale; tiles of up
                                  to 128 features over all of K (over a slice of K where the features alone do not fill
                                  the SMs). What AUTO runs for 5 to 16 rows of x on weights of 4 MB and more, and in
                                  passes of 16 rows beyond that */

typedef struct gq_caps { /* replaces gc_caps, gc_shim.h:43-50 */
    char device_name[256];
    uint32_t cc_major, cc_minor;
    uint32_t sm_count;
    uint32_t max_shared_per_block;
    uint64_t total_memory;
    uint64_t l2_bytes;
} gq_caps;

typedef struct gq_stats { /* replaces gc_submit_stats, gc_shim.h:61-76 */
    uint64_t launches;            /* kernels launched by operators (eager and while capturing) */
    uint64_t graph_launches;      /* gq_graph_replay calls */
    uint64_t graph_nodes_replayed;/* kernel nodes those replays ran */
    uint64_t captures;            /* graphs instantiated */
    uint64_t syncs;               /* host waits (download, synchronize) */
    uint64_t wait_ns_total;       /* host time spent in those waits */
    uint64_t wait_ns_last;
    uint64_t buffer_allocations;  /* fresh device allocations (pool misses and persistent) */
    uint64_t buffers_outstanding; /* handles alive */
    uint64_t pool_reuses;         /* GQ_MEM_DEVICE requests served from the pool */
    uint64_t persistent_buffers;  /* GQ_MEM_DEVICE_PERSISTENT buffers alive */
    uint64_t persistent_bytes;    /* and their total size */
    uint64_t persistent_peak;     /* the most persistent bytes alive at once */
    uint64_t uploads, downloads;
} gq_stats;

/* gc_shim.h:78 */
const char* gq_last_error(void);

/* gc_shim.h:80-82. `device` is the CUDA ordinal. Refuses anything that is not
 * compute capability 10.x: the kernels are built for sm_100a only. */
int32_t gq_create(int32_t device, gq_ctx** out);
void gq_destroy(gq_ctx* ctx);
int32_t gq_caps_get(gq_ctx* ctx, gq_caps* out);

/* gc_shim.h:96-98 */
int32_t gq_buffer_create(gq_ctx* ctx, uint64_t bytes, uint32_t mem, gq_buf* out);
int32_t gq_buffer_release(gq_ctx* ctx, gq_buf buf);
int32_t gq_buffer_size(gq_ctx* ctx, gq_buf buf, uint64_t* out);
/* No counterpart in the shim (Vulkan buffers have no address): register
 * device memory the caller owns (a framework tensor, say) so operators can
 * use it without a copy. Releasing the handle does not free the memory. */
int32_t gq_buffer_wrap(gq_ctx* ctx, void* device_ptr, uint64_t bytes, gq_buf* out);
/* The device address behind a handle, for callers that run their own kernels
 * on the context's stream. */
int32_t gq_buffer_ptr(gq_ctx* ctx, gq_buf buf, void** out);
/* The context's cudaStream_t, as a void*. */
int32_t gq_stream(gq_ctx* ctx, void** out);

/* gc_shim.h:100-107. Both return after the copy has completed. Refused while
 * a capture is open, with the reference's messages
 * (crates/grilly-core/src/device.rs:591-597, 620-628). */
int32_t gq_upload(gq_ctx* ctx, gq_buf dst, uint64_t offset, const void* src, uint64_t bytes);
int32_t gq_download(gq_ctx* ctx, gq_buf src, uint64_t offset, void* dst, uint64_t bytes);
/* Asynchronous forms for pinned host memory (gq_host_alloc): the copy is
 * ordered on the stream and the host pointer must stay valid until the next
 * gq_synchronize. These may be captured. */
int32_t gq_upload_async(gq_ctx* ctx, gq_buf dst, uint64_t offset, const void* pinned_src, uint64_t bytes);
int32_t gq_download_async(gq_ctx* ctx, gq_buf src, uint64_t offset, void* pinned_dst, uint64_t bytes);
int32_t gq_host_alloc(gq_ctx* ctx, uint64_t bytes, void** out);
int32_t gq_host_free(gq_ctx* ctx, void* ptr);

/* gc_shim.h:117-121 (byte offsets; multiples of 4) */
int32_t gq_copy(gq_ctx* ctx, gq_buf src, uint64_t src_offset, gq_buf dst, uint64_t dst_offset, uint64_t bytes);
int32_t gq_fill(gq_ctx* ctx, gq_buf dst, uint64_t offset, uint64_t bytes, uint32_t word);
/* gc_submit's wait, gc_shim.h:122 */
int32_t gq_synchronize(gq_ctx* ctx);
/* gc_shim.h:123-125 */
int32_t gq_stats_get(gq_ctx* ctx, gq_stats* out);
int32_t gq_persistent_peak_reset(gq_ctx* ctx);

/* ── int8 per-row ──────────────────────────────────────────────────────
 * Offsets named *_off are in ELEMENTS of the tensor's type. */

/* QUANTIZE{w,q,scale; rows,k,words,w_off} — crates/grilly-infer/src/quant.rs:18-24,98-141
 * and shaders/g2-quantize-q8.glsl:22-53. w is (rows, k) float32 at w_off;
 * q must hold rows*words8 words, scale rows floats. */
int32_t gq_int8_quantize(gq_ctx* ctx, gq_buf w, uint64_t w_off, uint64_t rows, uint64_t k, gq_buf q, gq_buf scale);

/* The same packer writing rows [row0, row0 + rows) of a LARGER weight of total_rows rows (q: total_rows * words8 words,
 * scale: total_rows floats): the parts of a fused projection (q | k | v, gate | up) are quantized straight into the fused
 * weight, one call per part, instead of being quantized apart and copied together, so the parts never exist twice on the
 * device. No counterpart in the reference, which names this as its next step (docs/inference.md:900-904;
 * python/grilly/infer/models/llama.py:108-131 builds the fused weight with Int8Weight::cat). Bit for bit what quantizing
 * the parts and gq_copy-ing them together gives, because the parameters are per row. */
int32_t gq_int8_quantize_rows(gq_ctx* ctx, gq_buf w, uint64_t w_off, uint64_t rows, uint64_t k, gq_buf q, gq_buf scale, uint64_t row0,
                              uint64_t total_rows);

/* LINEAR / LINEAR_TILED{x,q,scale,bias,y; m,k,n,vecs,x_off,b_off,has_bias,x_vec4}
 * — quant.rs:25-39,233-304, g2-linear-q8.glsl:33-95, g2-linear-q8-tiled.glsl:41-100.
 * y[m][n] = (sum_k x[m][k] * q[n][k]) * scale[n] (+ bias[n]); bias == 0 means none.
 * AUTO: the streaming IMMA kernel for one or two rows of x; from three rows on (at three rows on weights of 8 MB and
 * more) the integer tensor-core GEMM GQ_KERNEL_TENSOR_I8, with tiles sized to the row count (it holds three digit planes
 * of x in the context's scratch: inside a capture in which the scratch would have to grow, dp4a, or from 64 rows the tf32
 * GEMM when the shape meets its alignment rules, k % 4 == 0 and x_off % 4 == 0); dp4a elsewhere. y must not overlap x
 * (refused). */
int32_t gq_int8_linear(gq_ctx* ctx, gq_buf x, uint64_t x_off, uint64_t m, uint64_t k, gq_buf q, gq_buf scale,
                       gq_buf bias, uint64_t b_off, uint64_t n, gq_buf y, int32_t kernel);

/* The backward of the linear with its weight frozen — LinearInt8Backward, quant.rs:326-349:
 * grad_x[m][k] = sum_n grad[m][n] * (q[n][k] * scale[n]); grad_bias[n] = sum_m grad[m][n].
 * grad at element offset g_off; grad_x / grad_bias == 0 means "not needed". The dequantized weight is never written
 * to memory (the reference materialises it for the duration of the call). float32 products accumulated in float32:
 * within the reference's bound for this operator, (n + 2) 2^-24 sum|grad w| of float64. Outputs must not overlap grad. */
int32_t gq_int8_linear_backward(gq_ctx* ctx, gq_buf grad, uint64_t g_off, uint64_t m, gq_buf q, gq_buf scale, uint64_t n, uint64_t k,
                                gq_buf grad_x, gq_buf grad_bias);

/* DEQUANTIZE{q,scale,w; rows,k,words} — quant.rs:40-46,307-322, g2-dequantize-q8.glsl:15-21 */
int32_t gq_int8_dequantize(gq_ctx* ctx, gq_buf q, gq_buf scale, uint64_t rows, uint64_t k, gq_buf w);

/* ── int4 group-wise ─────────────────────────────────────────────────── */

/* QUANTIZE{w,q,scale,zero; rows,k,group,words,groups,w_off} — quant4.rs:26-32,85-154,
 * g2-quantize-q4.glsl:30-70. group must be a positive multiple of 32. */
int32_t gq_int4_quantize(gq_ctx* ctx, gq_buf w, uint64_t w_off, uint64_t rows, uint64_t k, uint64_t group, gq_buf q,
                         gq_buf scale, gq_buf zero);

/* As gq_int8_quantize_rows, for int4: rows [row0, row0 + rows) of a weight of total_rows rows. */
int32_t gq_int4_quantize_rows(gq_ctx* ctx, gq_buf w, uint64_t w_off, uint64_t rows, uint64_t k, uint64_t group, gq_buf q, gq_buf scale,
                              gq_buf zero, uint64_t row0, uint64_t total_rows);

/* LINEAR{x,q,scale,zero,bias,y; m,k,n,vecs,group,groups,x_off,b_off,has_bias,x_vec4}
 * — quant4.rs:33-39,371-442, g2-linear-q4.glsl:43-111.
 * AUTO (group_size 128): one to four rows of x on the warp-level ring kernel where it applies (in_features 4096 or
 * 8192), more rows — and three or more rows of other in_features that are multiples of 128 — on a tcgen05 kernel
 * (GQ_KERNEL_UMMA_LANES up to in_features 16384, GQ_KERNEL_UMMA beyond), which reads the weight once for up to 16 rows,
 * when the weight is large enough to pay for its start-up (4 MB); more than 16 rows in passes of 16 through the same
 * kernel; the IMMA and dp4a kernels elsewhere. y must not overlap x (refused). */
int32_t gq_int4_linear(gq_ctx* ctx, gq_buf x, uint64_t x_off, uint64_t m, uint64_t k, gq_buf q, gq_buf scale,
                       gq_buf zero, gq_buf bias, uint64_t b_off, uint64_t n, uint64_t group, gq_buf y,
                       int32_t kernel);

/* DEQUANTIZE{q,scale,zero,w; rows,k,group,words,groups} — quant4.rs:40-46,343-366,
 * g2-dequantize-q4.glsl:16-24 */
int32_t gq_int4_dequantize(gq_ctx* ctx, gq_buf q, gq_buf scale, gq_buf zero, uint64_t rows, uint64_t k,
                           uint64_t group, gq_buf w);

/* As gq_int8_linear_backward for an int4 weight — LinearInt4Backward, quant4.rs:447-480:
 * grad_x[m][k] = sum_n grad[m][n] * (level[n][k] * scale[n][g] + (zero[n][g] - 8 scale[n][g])), g = k / group. */
int32_t gq_int4_linear_backward(gq_ctx* ctx, gq_buf grad, uint64_t g_off, uint64_t m, gq_buf q, gq_buf scale, gq_buf zero, uint64_t n,
                                uint64_t k, uint64_t group, gq_buf grad_x, gq_buf grad_bias);

/* ── GPTQ on the device ──────────────────────────────────────────────────
 * The reference runs both in numpy on the host (python/grilly/infer/gptq.py:87-181, the column loop;
 * python/grilly/infer/calibration.py:97-123, the Hessian capture): 263 s per model, docs/inference.md:357-359. */

/* hessian[k][k] += 2 X^T X for the calibration rows X (rows, k) at x_off: GPTQ's H. float32, symmetric. */
int32_t gq_gptq_hessian_add(gq_ctx* ctx, gq_buf x, uint64_t x_off, uint64_t rows, uint64_t k, gq_buf hessian);
/* The column loop of gptq.py:150-178 on `work`, a float32 COPY of the weight (rows, k) that the call consumes:
 * column by column each value is rounded to its int4 level with the group's parameters taken from the weights as
 * they stand when the loop reaches the group, and the rounding error, divided by upper[j][j], is pushed into the
 * columns not yet quantized along row j of `upper` — the (k, k) upper factor U, U^T U = H^-1 after damping, which
 * the caller computes once per layer (gptq.py:68-84). Writes the packed levels, scales and zero points in the
 * int4 layout (an Int4Weight). errors: scratch of rows * 128 floats. group_size 32, 64 or 128 (a group must lie
 * inside a block of 128 columns); act_order / static_groups are not implemented. With a diagonal `upper` the
 * result is gq_int4_quantize's, bit for bit. */
int32_t gq_gptq_quantize(gq_ctx* ctx, gq_buf work, uint64_t rows, uint64_t k, uint64_t group, gq_buf upper, gq_buf errors, gq_buf q, gq_buf scale,
                         gq_buf zero);

/* ── capture / replay — crates/grilly-core/src/graph.rs:43-164,
 * device.rs:365-416, as CUDA graphs. Capture is context-wide: capture from
 * the thread that replays, with nothing else running on the context
 * (graph.rs:23-26). Buffers an operator touches while capturing are retained
 * by the graph until gq_graph_destroy, so a replay never writes memory that
 * has been handed to someone else (kernel.rs:99-117). */
int32_t gq_begin_capture(gq_ctx* ctx);
int32_t gq_end_capture(gq_ctx* ctx, gq_graph** out); /* GQ_ERR "nothing was captured" for an empty capture */
int32_t gq_capturing(gq_ctx* ctx, uint32_t* out);
int32_t gq_graph_replay(gq_ctx* ctx, gq_graph* graph);
int32_t gq_graph_nodes(gq_graph* graph, uint64_t* out); /* operator launches the graph holds */
void gq_graph_destroy(gq_ctx* ctx, gq_graph* graph);

/* ── the rest of a decode step (the int8 full-step configuration) ───────
 * The operators between the quantized linears of a Llama/Qwen2-shaped decode
 * step, one new token, batch 1. What a step must know about where it is — the
 * token id, the cache cursor, which is also q's and k's rotary position — is
 * read from device memory, so a captured step replays correctly. float32
 * tensors at offset 0 unless an offset is given. */

/* out[r][:] = table[ids[r]][:] — python/grilly/infer/models/llama.py:348 (g2-index.glsl:22-38). ids int32. */
int32_t gq_embedding(gq_ctx* ctx, gq_buf table, gq_buf ids, uint64_t rows, uint64_t width, uint64_t vocab, gq_buf out);
/* h = x (+ residual); y = h / sqrt(mean(h^2) + eps) * weight — crates/grilly-infer/src/ops.rs rms_norm /
 * add_rms_norm, g2-rms-norm.glsl:54-74. residual, weight and h may be 0 (absent). */
int32_t gq_add_rms_norm(gq_ctx* ctx, gq_buf x, gq_buf residual, gq_buf weight, uint64_t rows, uint64_t n, float eps, gq_buf y,
                        gq_buf h);
/* One token's fused q|k|v row: rotary on q and k at position lens[layer] (cos/sin tables [max_len][dim]), q
 * to q_out, k and v appended to the layer's cache [kv_heads][max_len][dim] at that position —
 * crates/grilly-infer/src/ops.rs:120-133 (rope), kv_cache.rs:378-432 (append_rotary), g2-rope.glsl:24-40,
 * g2-kv-write.glsl:43-72. A full cache takes nothing more. lens: uint32 per layer. */
int32_t gq_rope_kv_append(gq_ctx* ctx, gq_buf qkv, gq_buf cos, gq_buf sin, gq_buf lens, uint64_t layer, uint64_t layers, uint64_t heads,
                          uint64_t kv_heads, uint64_t dim, uint64_t max_len, gq_buf q_out, gq_buf kcache, uint64_t k_off, gq_buf vcache,
                          uint64_t v_off);
/* lens[l] = min(lens[l] + 1, max_len) for all layers, once per step — g2-kv-advance.glsl:18-21. */
int32_t gq_kv_advance(gq_ctx* ctx, gq_buf lens, uint64_t layers, uint64_t max_len);
/* Grouped-query attention of the new token over the cache's first lens[layer] + 1 positions, split over
 * the length and merged in one launch — kv_cache.rs:454-568, g2-attn-decode{,-split,-merge}.glsl.
 * `scratch` holds gq_attn_scratch_bytes bytes, zeroed once before the first call; calls sharing a scratch
 * buffer must not overlap on the GPU. */
int32_t gq_attn_scratch_bytes(gq_ctx* ctx, uint64_t heads, uint64_t dim, uint64_t max_len, uint64_t* out);
int32_t gq_attn_decode(gq_ctx* ctx, gq_buf q, gq_buf kcache, uint64_t k_off, gq_buf vcache, uint64_t v_off, gq_buf lens, uint64_t layer,
                       uint64_t layers, uint64_t heads, uint64_t kv_heads, uint64_t dim, uint64_t max_len, float scale, gq_buf scratch,
                       gq_buf out);
/* gq_rope_kv_append and gq_attn_decode in one launch: `qkv` is the raw q | k | v row; every CTA rotates its head of q at the
 * cursor's position, the new token's rotated key and its value are used where that position is attended to and are appended to
 * the cache by one CTA per KV head. No counterpart in the reference (two launches there). Buffers 16-byte aligned. */
int32_t gq_attn_decode_rope(gq_ctx* ctx, gq_buf qkv, gq_buf cos, gq_buf sin, gq_buf kcache, uint64_t k_off, gq_buf vcache, uint64_t v_off,
                            gq_buf lens, uint64_t layer, uint64_t layers, uint64_t heads, uint64_t kv_heads, uint64_t dim, uint64_t max_len,
                            float scale, gq_buf scratch, gq_buf out);
/* Fused forms for one decode token (one row): the operator before a linear runs inside the linear's conversion of x,
 * saving a launch and a round trip of the row. No counterpart in the reference, which launches them one by one.
 * gq_int8_linear_norm:   h = x + residual (residual 0: h = x); h_out = h (if not 0); y = W . (h / sqrt(mean(h^2) + eps) * w) + bias
 *                        — gq_add_rms_norm then gq_int8_linear.
 * gq_int8_linear_swiglu: y = W . (silu(gate_up[0:k]) * gate_up[k:2k]) + bias — gq_swiglu then gq_int8_linear, with the
 *                        hardware's exp2 and reciprocal (about 1e-6 relative to the separate operators).
 * k = in_features of the layer, a multiple of 4; x, residual, w, h_out and gate_up at offset 0. Outputs must not overlap
 * inputs: h_out may not be x or residual (every CTA reads them for the row's norm while one stores h_out; gq_add_rms_norm is
 * the in-place form), y may not overlap any input. Refused with GQ_ERR. */
int32_t gq_int8_linear_norm(gq_ctx* ctx, gq_buf x, gq_buf residual, gq_buf norm_weight, float eps, gq_buf h_out, uint64_t k, gq_buf q,
                            gq_buf scale, gq_buf bias, uint64_t b_off, uint64_t n, gq_buf y);
int32_t gq_int8_linear_swiglu(gq_ctx* ctx, gq_buf gate_up, uint64_t k, gq_buf q, gq_buf scale, gq_buf bias, uint64_t b_off, uint64_t n,
                              gq_buf y);
/* gq_attn_decode with the scratch in a fixed 2 MiB array of the library's own device memory: takes no scratch
 * buffer and allocates nothing, on the first call or later. No counterpart in the reference (its scratch is
 * a pooled buffer, kv_cache.rs:502-528). The first call on a device does the set-up (an address look-up):
 * make it before a stream capture begins. Refuses shapes whose 1024 + heads * splits * (dim + 2) floats exceed
 * the array (the per-head counters lie in its first 1024 words whatever the shape, so calls of different shapes may
 * follow one another). Every call on a device shares the array, so calls that overlap on the GPU race; calls on one
 * context are stream-ordered and do not. */
int32_t gq_attn_decode_static(gq_ctx* ctx, gq_buf q, gq_buf kcache, uint64_t k_off, gq_buf vcache, uint64_t v_off, gq_buf lens,
                              uint64_t layer, uint64_t layers, uint64_t heads, uint64_t kv_heads, uint64_t dim, uint64_t max_len,
                              float scale, gq_buf out);
/* Prompt processing for `rows` new tokens at once — the prefill branch of python/grilly/infer/models/llama.py:168-179
 * (rope on q and k, causal scaled_dot_product_attention with grouped queries, cache.append) in two launches: the rows'
 * q are rotated into q_scratch, their k (rotated) and v are appended at cache positions lens[layer] + t, and every
 * query attends causally over positions 0 .. lens[layer] + t. The positions come from the DEVICE cursor, so the rows
 * may continue a non-empty cache (chunked prefill) and the call may be captured; rows == 1 is a decode step's
 * attention. The cursor is not advanced: gq_kv_advance_by does that once per step, after the last layer.
 * With kscale / vscale (float32 [layers * kv_heads * max_len], one per cached row) the cache buffers hold int8
 * codes [kv_heads][max_len][dim] (k_off / v_off in bytes then): every appended row is stored as rint(v / s),
 * s = max|v| / 127, and dequantized as it is read — a quarter of the bytes per decoded token. The reference's cache
 * is exact float32 (crates/grilly-infer/src/kv_cache.rs:1-19): the int8 form has no counterpart there. */
int32_t gq_attn_prefill(gq_ctx* ctx, gq_buf qkv, uint64_t rows, gq_buf cos, gq_buf sin, gq_buf kcache, uint64_t k_off, gq_buf vcache, uint64_t v_off,
                        gq_buf kscale, gq_buf vscale, gq_buf lens, uint64_t layer, uint64_t layers, uint64_t heads, uint64_t kv_heads, uint64_t dim,
                        uint64_t max_len, float scale, gq_buf q_scratch, gq_buf out);
/* lens[l] = min(lens[l] + count, max_len) for all layers — g2-kv-advance.glsl:18-21 for a whole prompt chunk. */
int32_t gq_kv_advance_by(gq_ctx* ctx, gq_buf lens, uint64_t layers, uint64_t max_len, uint64_t count);
/* out[r][j] = silu(gate_up[r][j]) * gate_up[r][width + j] — ops.rs:148-212, g2-swiglu.glsl:21-29. */
int32_t gq_swiglu(gq_ctx* ctx, gq_buf gate_up, uint64_t rows, uint64_t width, gq_buf out);
/* The next token of every row, chosen on the device — crates/grilly-infer/src/sampling.rs:1-60,
 * shaders/g2-sample.glsl: Hugging Face's processors in generate()'s order (repetition penalty over `history`,
 * then with do_sample temperature, top_k (0 = off), top_p (1 = off)) and a draw from what is left by the inverse
 * CDF in token order; without do_sample the first index of the largest penalized score. tokens: int32 per row,
 * -1 where nothing can be drawn (every score -inf). probs (0 = none) receives the filtered distribution.
 * Where the reference passes each row's uniform number and the history length from the host, here they are read
 * from device memory so that a captured step replays: `uniforms` holds uniform_rows x rows floats in [0, 1) and the
 * launch uses row (*draws % uniform_rows), adding one to the uint32 word `draws` when do_sample; `history`
 * (0 = none) is int32 [rows][hist_cap] of which the uint32 word `hist_len` says how many are set, and with
 * `append` the chosen token is written at that place and the word advanced (a full history takes nothing more).
 * scratch: 2 * rows * vocab floats. */
int32_t gq_sample(gq_ctx* ctx, gq_buf logits, uint64_t rows, uint64_t vocab, gq_buf history, uint64_t hist_cap, gq_buf hist_len, uint32_t append,
                  uint32_t do_sample, double temperature, uint64_t top_k, double top_p, double repetition_penalty, gq_buf uniforms,
                  uint64_t uniform_rows, gq_buf draws, gq_buf scratch, gq_buf tokens, gq_buf probs);
/* The whole decode step (one token, batch 1, int8 weights, float32 cache) as ONE persistent kernel: what
 * python/grilly/infer/models/llama.py:353-366 issues as ~270 dispatches, and gq_embedding ... gq_argmax_rows above as
 * ~125 launches, runs as phases of a single cooperative launch separated by grid-wide barriers, each CTA's share of
 * every weight prefetched into shared memory phases ahead. Same results as the operator-by-operator step to float32
 * rounding (the linears use the fixed-point arithmetic of the fast GEMV). The plan names the model's buffers (it
 * retains them until it is destroyed) and owns its activations; a step reads the token from device memory, writes the
 * logits and the greedy next token, appends to the cache at the device cursor and advances it: capture it and replay.
 * Shapes: hidden, heads * dim and inter multiples of 16; hidden <= 4096, the other two <= 8192; dim 32, 64 or 128;
 * kv_heads * 16 <= the SM count. Every wait inside is bounded by the context's wait limit (gq_set_wait_limit_us). */
typedef struct gq_decode_layer {
    gq_buf input_norm;                    /* float32 [hidden] */
    gq_buf qkv_q, qkv_scale, qkv_bias;    /* int8 codes [(heads + 2 kv_heads) dim][hidden], scales, bias (0 = none) */
    gq_buf o_q, o_scale;                  /* [hidden][heads dim] */
    gq_buf post_norm;                     /* float32 [hidden] */
    gq_buf gate_up_q, gate_up_scale;      /* gate rows then up rows: [2 inter][hidden] */
    gq_buf down_q, down_scale;            /* [hidden][inter] */
} gq_decode_layer;
typedef struct gq_decode_desc {
    uint64_t hidden, heads, kv_heads, dim, inter, vocab, layers, max_len;
    float eps, attn_scale;
    gq_buf embed, final_norm, head_q, head_scale; /* float32 table [vocab][hidden]; the (tied) head's int8 codes and scales */
    gq_buf cos, sin;                              /* [max_len][dim] */
    gq_buf kcache, vcache, lens;                  /* float32 [layers][kv_heads][max_len][dim]; uint32 [layers] */
    const gq_decode_layer* layer;                 /* [layers] */
} gq_decode_desc;
typedef struct gq_decode_plan gq_decode_plan;
int32_t gq_decode_plan_create(gq_ctx* ctx, const gq_decode_desc* desc, gq_decode_plan** out);
int32_t gq_decode_plan_step(gq_ctx* ctx, gq_decode_plan* plan, gq_buf token, gq_buf logits, gq_buf next_token);
void gq_decode_plan_destroy(gq_ctx* ctx, gq_decode_plan* plan);
/* out[r] = index of the maximum of row r (int32; the first on ties) — g2-argreduce-rows.glsl:42-77. */
int32_t gq_argmax_rows(gq_ctx* ctx, gq_buf v, uint64_t rows, uint64_t n, gq_buf out);

/* ── multi-GPU: column-sharded linears over the GPUs of one box ──────────
 * No counterpart in the reference, which runs on a single device. One process
 * (and one context) per GPU. Rank r owns output features [r n/W, (r+1) n/W):
 * it quantizes and multiplies its own rows with the functions above, then the
 * blocks of y are gathered so that every rank holds y[m][n]. */

/* NCCL communicator. Rank 0 makes a 128-byte id (gq_comm_unique_id), the
 * caller carries it to the other ranks, every rank calls gq_comm_create. */
#define GQ_COMM_ID_BYTES 128
int32_t gq_comm_unique_id(void* out, uint64_t bytes);
int32_t gq_comm_create(gq_ctx* ctx, int32_t nranks, int32_t rank, const void* unique_id, gq_comm** out);
void gq_comm_destroy(gq_ctx* ctx, gq_comm* comm);
/* dst[r][rank * n_shard + c] = src(rank)[r][c] for every rank (ncclAllGather per row, one group), on the
 * context's stream; may be captured. src holds m * n_shard floats, dst m * n_shard * nranks. */
int32_t gq_all_gather_columns(gq_ctx* ctx, gq_comm* comm, gq_buf src, gq_buf dst, uint64_t m, uint64_t n_shard);

/* Peer-mapped memory (CUDA IPC) for the put-and-signal gather below. Export
 * fills 64 bytes the caller carries to the other processes of the box; open
 * maps that memory here and returns a handle (releasing it unmaps). Only
 * buffers made by gq_buffer_create can be exported. */
#define GQ_IPC_HANDLE_BYTES 64
int32_t gq_buffer_ipc_export(gq_ctx* ctx, gq_buf buf, void* out, uint64_t bytes);
int32_t gq_buffer_ipc_open(gq_ctx* ctx, const void* handle, uint64_t buffer_bytes, gq_buf* out);

/* This library's own gather over NVLink. Every value of y travels as ONE 64-bit word, step << 32 | the
 * float's bits, written with a single plain store into every rank's RECEIVE buffer (peer_recv[i] = a handle to
 * rank i's receive buffer: its own for i == rank, an ipc-opened one otherwise; GQ_PEER_RECV_BYTES(m, n_full)
 * bytes, zeroed once before the first call). A word whose upper half is the current step has arrived: no
 * fence, counter or signal is involved. The kernel then waits, at most the context's wait limit
 * (gq_set_wait_limit_us, default ~2 s), for all words of this step and writes this rank's plain
 * y_full[m][n_full] (a local buffer). `state` is two uint32 words of this rank, zeroed once: the step number
 * lives on the device, so a captured call keeps counting when replayed. The receive buffer has two halves that
 * the device alternates by step parity, which is all the protection needed: a rank can be at most one step
 * ahead of the slowest. Every rank must make the same sequence of calls on one set of buffers. A wait that
 * gives up is reported by the next host wait (GQ_ERR naming the rank whose words never came); the context
 * stays usable. */
#define GQ_PEER_RECV_BYTES(m, n_full) (2ull * (uint64_t)(m) * (uint64_t)(n_full) * 8ull)
int32_t gq_peer_gather(gq_ctx* ctx, gq_buf src, uint64_t m, uint64_t n_shard, int32_t rank, int32_t nranks,
                       const gq_buf* peer_recv, gq_buf state, gq_buf y_full);
/* gq_int4_linear and the gather in ONE kernel: the GEMV's epilogue sends this rank's block of columns straight to every
 * rank's receive buffer (plain peer stores of value-and-step words, as above) and the CTAs then share out the receiving of the
 * whole y into y_full. Same buffers and protocol as gq_peer_gather, so calls of both kinds may be mixed on one set.
 * Shapes: the ring kernel's (group_size 128, in_features 4096 or 8192); up to 16 rows of x, four per pass. Where
 * gq_int4_linear's AUTO would pick the tcgen05 decode kernel (five and more rows on a shard of 4 MB and more; any
 * in_features that is a multiple of 128), that kernel runs instead and the gather adds up its K slices' partial sums
 * (and the bias) as it sends them: one pass over the weight, one launch less than linear-then-gather. */
int32_t gq_int4_linear_gather(gq_ctx* ctx, gq_buf x, uint64_t x_off, uint64_t m, uint64_t k, gq_buf q, gq_buf scale, gq_buf zero, gq_buf bias,
                              uint64_t b_off, uint64_t n_shard, uint64_t group, int32_t rank, int32_t nranks, const gq_buf* peer_recv,
                              gq_buf state, gq_buf y_full);
/* How long a kernel waits for another GPU's data before it gives up (0 restores the default, ~2 s). Failure
 * detection in the reference's convention: misuse and failure are reported, never thrown
 * (crates/grilly-sys/tests/gpu.rs:272-329); the reference itself has no multi-GPU wait. */
int32_t gq_set_wait_limit_us(gq_ctx* ctx, uint64_t microseconds);

#if defined(GQ_BUILD) && defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif

#endif /* GQ_H */
