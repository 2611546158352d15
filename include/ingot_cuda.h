/*
 * ingot_cuda.h — C ABI of libingot_cuda.so, the sm_100a (B200) implementation
 * of ingot's decode hot path: block-quantised weights (GGUF Q4_0, Q8_0, Q4_K,
 * Q6_K, plus F32/F16/BF16), fused dequantise-and-dot GEMV, gate/up + GLU,
 * expert-routed GEMV, top-k routing, expert combine, and the dequant-GEMM.
 *
 * The boundary it replaces is the reference's Rust `Gpu` type ("the only
 * unsafe boundary", src/metal.rs:1) together with the operator layer in
 * src/metal_generic.rs and the data model in src/gguf.rs / src/weights.rs.
 * Each entry point cites the reference function it stands in for.  All
 * pointers are plain host or device addresses; there are no C++ or framework
 * types in any signature.
 *
 * Conventions (identical to the reference's kernel parameter block `p[]`,
 * kernels/generic.metal:294-297, src/metal_generic.rs:195-202):
 *   cols    K, the contiguous dimension of a weight row (Tensor.dims[0])
 *   rows    N, output rows of one matrix (Tensor.dims[1])
 *   stride  bytes of one weight row = cols / block * block_bytes
 *   kind    GGML type id: 0 F32, 1 F16, 2 Q4_0, 8 Q8_0, 12 Q4_K, 14 Q6_K, 30 BF16
 *   expert  index into experts stacked as [expert][rows][stride]
 *   x       activations [tokens][cols]; y outputs [tokens][rows], float32
 *   x_kind  type of x: 0 (float32, what the reference uses) or 30 (bfloat16)
 * Operators take DEVICE pointers and are asynchronous on the handle's stream;
 * the *_host conveniences take HOST pointers and block.
 *
 * Threading: a handle is owned by one host thread, like the reference's
 * !Send/!Sync `Gpu` (src/metal.rs:193-208).
 *
 * Errors: every call returns an ingot_status.  A device failure is sticky:
 * later calls on the handle return INGOT_DEVICE ("requires reload"), matching
 * src/metal.rs:663-671,1349-1353.
 */
#ifndef INGOT_CUDA_H
#define INGOT_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define INGOT_API __attribute__((visibility("default")))
#else
#define INGOT_API
#endif

typedef int32_t ingot_status;
enum {
    INGOT_OK = 0,
    INGOT_INVALID = 1,      /* io::ErrorKind::InvalidData: shape/layout/bounds (src/lib.rs:39-41) */
    INGOT_UNSUPPORTED = 2,  /* "no kernel for this type": Ok(None)/false in src/metal_generic.rs */
    INGOT_DEVICE = 3,       /* io::Error::other: CUDA failure; sticky */
    INGOT_EOF = 4,          /* io::ErrorKind::UnexpectedEof (src/gguf.rs:359-362) */
    INGOT_INTERRUPTED = 5,  /* io::ErrorKind::Interrupted (src/generic.rs:52-54) */
    INGOT_TIMEOUT = 6       /* a bounded device-side wait ran out */
};

enum {
    INGOT_KIND_F32 = 0, INGOT_KIND_F16 = 1, INGOT_KIND_Q4_0 = 2, INGOT_KIND_Q8_0 = 8,
    INGOT_KIND_Q4_K = 12, INGOT_KIND_Q6_K = 14, INGOT_KIND_BF16 = 30
};

/* x_kind of activation rows already packed by ingot_pack_x / ingot_pack_digits */
enum { INGOT_X_PACKED = 256, INGOT_X_DIGITS = 258, INGOT_X_PACKED_HI = 259 };

typedef struct ingot_gpu ingot_gpu;      /* opaque; the reference's `Gpu` */
typedef struct ingot_graph ingot_graph;  /* opaque; a recorded `Command` */

/* ---- data model --------------------------------------------------------- */

/* geometry(kind) -> (block elements, block bytes): src/gguf.rs:470-491.
 * INGOT_UNSUPPORTED for a type outside this path. */
INGOT_API ingot_status ingot_geometry(uint32_t kind, uint32_t *block, uint32_t *bytes);

/* Row stride and total bytes of a tensor of `cols` x `rows` x `count`
 * (stride/bytes derivation in src/gguf.rs:152-161); INGOT_INVALID when cols is
 * not a whole number of blocks or a product overflows. */
INGOT_API ingot_status ingot_tensor_layout(uint32_t kind, uint64_t cols, uint64_t rows, uint64_t count,
                                           uint64_t *stride, uint64_t *bytes);

/* ---- handle ------------------------------------------------------------- */

/* Gpu::new (src/metal.rs:238-533): binds CUDA device `device`, creates the
 * stream and the device status word.  INGOT_DEVICE when the device is not an
 * sm_100 part or CUDA fails. */
INGOT_API ingot_status ingot_gpu_create(int32_t device, ingot_gpu **out);
INGOT_API void ingot_gpu_destroy(ingot_gpu *gpu);

/* Text of the last error on this handle (never NULL). */
INGOT_API const char *ingot_last_error(const ingot_gpu *gpu);

/* Runs later operators on a caller-owned cudaStream_t (NULL restores the
 * handle's own stream).  The Command <-> stream correspondence:
 * src/metal.rs:659-673. */
INGOT_API ingot_status ingot_gpu_set_stream(ingot_gpu *gpu, void *cuda_stream);

/* Gpu::independent_projections, src/metal.rs:1371-1396: between begin and end only
 * operators that do not consume each other's results may be issued (no buffer
 * upload, read or synchronize either); they run concurrently — on B200 the launches
 * rotate over the handle's stream and three side streams forked from it — and
 * everything issued after end is ordered after all of them.  Works inside a
 * recorded command. */
INGOT_API ingot_status ingot_independent_begin(ingot_gpu *gpu);
INGOT_API ingot_status ingot_independent_end(ingot_gpu *gpu);

/* Options: INGOT_OPT_PDL (default 1) launches kernels with programmatic
 * dependent launch so a kernel's weight prefetch overlaps its predecessor's
 * tail; INGOT_OPT_FORCE_PLAIN (default 0) routes every GEMV through the plain
 * one-warp-per-row kernel (a test hook); INGOT_OPT_NO_MMA (default 0) keeps the
 * streaming GEMV on the fp32 CUDA-core kernel instead of the one whose inner
 * products run on the tensor cores (a test and comparison hook);
 * INGOT_OPT_TCGEN05_GEMV sends one-token GEMVs over Q4_K weights to the kernel
 * that multiplies on the tcgen05 int8 tensor cores (rows unpacked into tensor
 * memory, activations as base-256 digits); INGOT_OPT_EP_WORLD (default 1) is the
 * number of devices the experts are split over (ingot_ep_localize): routed launches
 * then expect about pairs / value live pairs and give each more CTAs;
 * INGOT_OPT_GROUP_SCOPE (default 1) launches the one-token projections of an
 * independent scope as one grid at the scope's end (0: each on its own stream);
 * INGOT_OPT_WIDE_ROWS (default 0) makes the fused-norm projections build their
 * activation rows with 30 bits of fixed point per 32 columns even when they round
 * to bfloat16 (default then: 15 bits, which leave the small neighbours of an
 * outlier hundreds of times their size fewer bits than bfloat16 carries), at the
 * price of twice the tensor-core instructions. */
enum { INGOT_OPT_PDL = 1, INGOT_OPT_FORCE_PLAIN = 2, INGOT_OPT_NO_MMA = 3, INGOT_OPT_TCGEN05_GEMV = 4, INGOT_OPT_EP_WORLD = 5,
       INGOT_OPT_GROUP_SCOPE = 6, INGOT_OPT_WIDE_ROWS = 7 };
INGOT_API ingot_status ingot_gpu_set_option(ingot_gpu *gpu, int32_t option, int32_t value);

/* Command::wait / Gpu::complete (src/metal.rs:1224-1235): blocks until the
 * stream drains, then reports CUDA errors and the device status word
 * (INGOT_TIMEOUT, INGOT_INVALID for an out-of-range expert id or a non-finite
 * router logit). */
INGOT_API ingot_status ingot_synchronize(ingot_gpu *gpu);

/* ---- buffers (Gpu::bytes / floats / zeros / output / read_f32:
 *      src/metal.rs:1251-1333, 649-658) ---------------------------------- */

INGOT_API ingot_status ingot_buffer_alloc(ingot_gpu *gpu, size_t bytes, void **device_ptr);
INGOT_API ingot_status ingot_buffer_free(ingot_gpu *gpu, void *device_ptr);

/* Gpu::output and Gpu::configure_workspace (src/metal.rs:1278-1337): float32 output buffers from a
 * size-keyed pool.  With no budget set (0, the default) ingot_output_alloc is a plain allocation.
 * With a budget, a released buffer waits on the idle list of its exact length and the next
 * request of that length takes it (a reuse); a request of a new length allocates, charged in
 * 16 KiB pages, after giving up only as much idle capacity as it needs, largest buffers first;
 * INGOT_INVALID "workspace live allocation exceeds budget" when leased buffers alone exceed it.
 * A released buffer may still be read by work already enqueued on the handle's stream: its next
 * holder's work is enqueued behind that.  ingot_workspace_statistics = workspace_statistics
 * (src/metal.rs:1338-1342): cumulative allocations, reuses, managed bytes now, peak. */
INGOT_API ingot_status ingot_gpu_configure_workspace(ingot_gpu *gpu, size_t limit_bytes);
INGOT_API ingot_status ingot_output_alloc(ingot_gpu *gpu, size_t count_f32, float **device_ptr);
INGOT_API ingot_status ingot_output_release(ingot_gpu *gpu, float *device_ptr);
INGOT_API ingot_status ingot_workspace_statistics(const ingot_gpu *gpu, uint64_t *allocations, uint64_t *reuses,
                                                  size_t *managed_bytes, size_t *peak_bytes);
/* host -> device, asynchronous on the handle's stream when `host` is pinned */
INGOT_API ingot_status ingot_buffer_upload(ingot_gpu *gpu, void *device_ptr, const void *host, size_t bytes);
/* device -> host; returns after the copy has completed */
INGOT_API ingot_status ingot_buffer_read(ingot_gpu *gpu, void *host, const void *device_ptr, size_t bytes);
INGOT_API ingot_status ingot_buffer_zero(ingot_gpu *gpu, void *device_ptr, size_t bytes);
/* Page-locked host memory for uploads/readbacks. */
INGOT_API ingot_status ingot_host_alloc(ingot_gpu *gpu, size_t bytes, void **host_ptr);
INGOT_API ingot_status ingot_host_free(ingot_gpu *gpu, void *host_ptr);

/* Gpu::load_weight (src/metal.rs:546-582) for a discrete GPU: validates the
 * tensor layout (kind, cols, rows, count, stride) against `bytes`, allocates
 * HBM and copies the GGUF bytes unchanged.  Replaces the no-copy mmap. */
INGOT_API ingot_status ingot_weight_upload(ingot_gpu *gpu, const void *host, uint32_t kind, uint64_t cols,
                                           uint64_t rows, uint64_t count, size_t bytes, void **device_ptr);

/* ---- operators on device buffers ---------------------------------------- */

/* read_rows (kernels/qwen.metal:35): y[r][j] = weight_at(row r, j) for
 * `rows` rows (all stacked experts); bit-exact. */
INGOT_API ingot_status ingot_dequant_rows(ingot_gpu *gpu, const void *w, uint32_t cols, uint64_t rows,
                                          uint32_t stride, uint32_t kind, float *y);

/* Gpu::matmul (src/metal.rs:877-1107) / Gpu::generic_project
 * (src/metal_generic.rs:175-228) / Gpu::matvec (src/metal.rs:846-875):
 * y[t][r] = sum_j W[expert][r][j] x[t][j] for `count` tokens.  count <= 4 runs the
 * GEMV (fp32 products of exactly dequantised weights); count > 4 runs ingot_gemm where
 * it applies (binary16 operand staging, as the reference does), else GEMV groups of four. */
INGOT_API ingot_status ingot_matmul(ingot_gpu *gpu, const void *w, uint32_t cols, uint32_t rows, uint32_t stride,
                                    uint32_t kind, uint32_t expert, const void *x, uint32_t x_kind,
                                    uint32_t count, float *y);

/* Gpu::generic_project for count > 4 (src/metal_generic.rs:182-206; kernels gemm_q4k / gemm_q6k,
 * kernels/generic.metal:315-388): Y[t][r] = sum_j W[expert][r][j] x[t][j] on the tensor cores
 * (tcgen05), weights and activations rounded to binary16 before the product like the reference's
 * staging, fp32 accumulation.  Q4_K and Q6_K with cols % 256 == 0; INGOT_UNSUPPORTED otherwise.
 * ingot_matmul takes this path by itself for count > 4.  Uses the handle's scratch for the
 * binary16 copy of x (count * cols * 2 bytes, grown on demand; not while recording). */
INGOT_API ingot_status ingot_gemm(ingot_gpu *gpu, const void *w, uint32_t cols, uint32_t rows, uint32_t stride,
                                  uint32_t kind, uint32_t expert, const void *x, uint32_t x_kind, uint32_t count,
                                  float *y);

/* Gpu::generic_gate_up (src/metal_generic.rs:231-261): y[t][r] =
 * glu(gate x, up x); gelu != 0 selects tanh-GeLU, else SiLU. */
INGOT_API ingot_status ingot_gate_up(ingot_gpu *gpu, const void *gate, const void *up, uint32_t cols,
                                     uint32_t rows, uint32_t stride, uint32_t kind, const void *x,
                                     uint32_t x_kind, uint32_t count, uint32_t gelu, float *y);

/* Gpu::generic_routed (src/metal_generic.rs:298-329) and the generic-format
 * project_routed_batch (kernels/qwen.metal:93-112): for each pair p,
 * y[p] = W[ids[p]] x[per_pair ? p : p / top].  `experts` bounds ids. */
INGOT_API ingot_status ingot_routed(ingot_gpu *gpu, const void *w, uint32_t cols, uint32_t rows, uint32_t stride,
                                    uint32_t kind, uint32_t experts, const void *x, uint32_t x_kind,
                                    const uint32_t *ids, uint32_t per_pair, uint32_t top, uint32_t pairs,
                                    float *y);

/* Gpu::generic_routed_gate_up (src/metal_generic.rs:264-296):
 * y[p] = silu(gate[ids[p]] x[p / top]) * (up[ids[p]] x[p / top]). */
INGOT_API ingot_status ingot_routed_gate_up(ingot_gpu *gpu, const void *gate, const void *up, uint32_t cols,
                                            uint32_t rows, uint32_t stride, uint32_t kind, uint32_t experts,
                                            const void *x, uint32_t x_kind, const uint32_t *ids, uint32_t top,
                                            uint32_t pairs, float *y);

/* route_topk (kernels/generic.metal:479-494; CPU route(): src/lib.rs:43-60):
 * ids[t][k], weights[t][k] for k < top; ties go to the lowest expert id.
 * experts <= 512.  top == 0 or top > experts is INGOT_INVALID; a non-finite
 * logit is reported by ingot_synchronize as INGOT_INVALID. */
INGOT_API ingot_status ingot_route_topk(ingot_gpu *gpu, const float *logits, uint32_t experts, uint32_t top,
                                        uint32_t tokens, uint32_t *ids, float *weights);

/* moe_sum (kernels/generic.metal:17): y[t][j] = sum_e routed[t*top+e][j] *
 * weights[t*top+e], in route order.  width % 4 == 0. */
INGOT_API ingot_status ingot_moe_sum(ingot_gpu *gpu, const float *routed, const float *weights, uint32_t width,
                                     uint32_t top, uint32_t tokens, float *y);

/* Gpu::activation (src/metal.rs:1172-1197; swiglu kernels/moe.metal:405-410,
 * gelu_mul kernels/generic_arch.metal:7-10). */
INGOT_API ingot_status ingot_activation(ingot_gpu *gpu, const float *gate, const float *up, uint64_t n,
                                        uint32_t gelu, float *y);

/* Architecture glue of the generic path (kernels/generic_arch.metal:2-17; Gemma and Phi-3 graphs in
 * src/generic.rs), one element per thread:
 *   scale_rows     y[i] = x[i] * scale                                  (:2-3)
 *   softcap_rows   y[i] = cap * tanh(x[i] / cap), final logit soft-cap  (:4-5)
 *   swiglu_fused   y[t][j] = silu(x[t][j]) * x[t][ff + j] over fused gate|up rows of width 2 ff (:11-15)
 *   copy_columns   y[r][j] = x[r * stride + offset + j], j < width      (:16-17) */
INGOT_API ingot_status ingot_scale_rows(ingot_gpu *gpu, const float *x, uint64_t n, float scale, float *y);
INGOT_API ingot_status ingot_softcap_rows(ingot_gpu *gpu, const float *x, uint64_t n, float cap, float *y);
INGOT_API ingot_status ingot_swiglu_fused(ingot_gpu *gpu, const float *x, uint32_t tokens, uint32_t ff, float *y);
INGOT_API ingot_status ingot_copy_columns(ingot_gpu *gpu, const float *x, uint32_t rows, uint32_t width,
                                          uint32_t offset, uint32_t stride, float *y);

/* Gpu::merge (src/metal.rs:1199-1223; combine kernels/moe.metal:412-422):
 * y[j] = sum_e routed[e][j] * weights[e] + shared[j] * sigmoid(shared_logit[0]). */
INGOT_API ingot_status ingot_merge(ingot_gpu *gpu, const float *routed, const float *shared,
                                   const float *weights, const float *shared_logit, uint32_t width,
                                   uint32_t top, float *y);

/* Gpu::add_rms (src/metal_generic.rs; kernel kernels/generic.metal:390-404):
 * per row s = a + b (when add), y = s * rsqrt(mean(s^2) + eps) * w.  `w`, `s`,
 * `y`, `y_bf16` may be NULL; y_bf16 receives y rounded to bfloat16. */
INGOT_API ingot_status ingot_add_rms(ingot_gpu *gpu, const float *a, const float *b, const float *w, float *s,
                                     float *y, void *y_bf16, uint32_t width, uint32_t rows, float eps,
                                     uint32_t add);

/* add_rms that also writes y in the packed order of ingot_pack_x (`y_packed`, rows of
 * ingot_packed_x_bytes(width); width a multiple of 64), so the projections that
 * follow need no separate packing pass.  pack_from_bf16 != 0 packs the bfloat16
 * rounding of y (what packing `y_bf16` would give); pack_from_bf16 = 3 packs that
 * rounding as high-part rows (ingot_pack_x_hi; rows of ingot_packed_hi_bytes). */
INGOT_API ingot_status ingot_add_rms_packed(ingot_gpu *gpu, const float *a, const float *b, const float *w, float *s,
                                            float *y, void *y_bf16, void *y_packed, uint32_t pack_from_bf16,
                                            uint32_t width, uint32_t rows, float eps, uint32_t add);

/* add_rms fused into the one-token projection that consumes it: x = rms_norm(a + b) * w (w
 * may be NULL; b is ignored unless add), rounded to bfloat16 when round_bf16, then y = W x
 * (or glu(gate x, up x)).  Every CTA of the GEMV computes the normalised row for itself, so
 * the step loses a launch and a round trip through memory; `s` (may be NULL) receives a + b
 * and must not alias a or b.  INGOT_UNSUPPORTED when the weight type has no tensor-core GEMV
 * (Q4_0, Q8_0, Q4_K, Q6_K with 16-byte aligned rows have one): call ingot_add_rms and the
 * plain projection instead.  No counterpart in the reference, whose add_rms
 * (kernels/generic.metal:390-404) is always a separate dispatch. */
INGOT_API ingot_status ingot_matmul_normed(ingot_gpu *gpu, const void *w, uint32_t cols, uint32_t rows, uint32_t stride,
                                           uint32_t kind, uint32_t expert, const float *a, const float *b,
                                           const float *norm_w, float *s, float eps, uint32_t add,
                                           uint32_t round_bf16, float *y);
INGOT_API ingot_status ingot_gate_up_normed(ingot_gpu *gpu, const void *gate, const void *up, uint32_t cols,
                                            uint32_t rows, uint32_t stride, uint32_t kind, const float *a,
                                            const float *b, const float *norm_w, float *s, float eps, uint32_t add,
                                            uint32_t round_bf16, uint32_t gelu, float *y);

/* ---- the rest of a generic decode step (graph: Generic::hidden, src/generic.rs:664-749) ---- */

/* embedding_batch (kernels/qwen.metal:139): y[t][j] = weight_at(row ids[t] of w, j) for `count`
 * tokens; w is `rows` (the vocabulary) x width in any type of this path; bit-exact.  A token
 * id >= rows is reported by ingot_synchronize as INGOT_INVALID (its row is zeros). */
INGOT_API ingot_status ingot_embedding_batch(ingot_gpu *gpu, const void *w, const uint32_t *ids, uint32_t width,
                                             uint32_t rows, uint32_t stride, uint32_t kind, uint32_t count, float *y);

/* The integer and float parameters of qk_rope_cache (kernels/generic.metal:405-410: head dim
 * <= 512, heads, kv heads, rotated dims, position, base, NeoX pairing, frequency factors,
 * QK norm, eps, unweighted value norm, q scale). */
typedef struct ingot_rope_params {
    uint32_t head_dim, heads, kv_heads, rotated, position;
    float base;
    uint32_t neox, use_factors, qk_norm;
    float eps;
    uint32_t value_norm;
    float q_scale;
} ingot_rope_params;

/* qk_rope_cache (kernels/generic.metal:405-438): per head row of `tokens` tokens, optional QK
 * RMS norm (weights q_norm, k_norm), rotary embedding of the first `rotated` dimensions at
 * position + t (interleaved pairs, or NeoX halves), q times q_scale to q_out [t][heads][D];
 * k and v (v optionally RMS-normalised without a weight) into the float32 caches at row
 * position + t, [row][kv_heads][D]. */
INGOT_API ingot_status ingot_qk_rope_cache(ingot_gpu *gpu, const float *q, const float *k, const float *v,
                                           const float *q_norm, const float *k_norm, const float *factors,
                                           float *q_out, float *k_cache, float *v_cache,
                                           const ingot_rope_params *params, uint32_t tokens);

/* attention_decode_<D> (kernels/generic.metal:440-474): causal attention of 1..4 query tokens
 * (the first at `position`) over the float32 caches, softmax scale 1/sqrt(D), grouped-query
 * heads, sliding window (0: none).  D in {64, 96, 128, 256, 512}, else INGOT_UNSUPPORTED. */
INGOT_API ingot_status ingot_attention_decode(ingot_gpu *gpu, const float *q, const float *k_cache,
                                              const float *v_cache, float *out, uint32_t head_dim, uint32_t heads,
                                              uint32_t kv_heads, uint32_t position, uint32_t window, uint32_t tokens);

/* flash_prefill_<D> (kernels/generic.metal:19-136, driven by Generic::flash, src/generic.rs:421-470):
 * causal attention of `rows` query rows — the first at `position`, position + rows <= length —
 * over the float32 caches, same scale, grouped-query heads and sliding window as above; what the
 * reference runs for more than four tokens.  Here one CTA per (row, head) with an online softmax
 * (the decode kernel over more rows): the same result, without the reference kernel's tiling of
 * eight query rows per threadgroup. */
INGOT_API ingot_status ingot_attention_prefill(ingot_gpu *gpu, const float *q, const float *k_cache,
                                               const float *v_cache, float *out, uint32_t head_dim,
                                               uint32_t heads, uint32_t kv_heads, uint32_t length,
                                               uint32_t position, uint32_t rows, uint32_t window);

/* greedy_select (kernels/qwen.metal:384-410) in its two stages, as Gpu::finish_greedy issues them
 * (src/metal.rs:1507-1548): out[r] = (token of the largest logit of row r — equal values, signed
 * zeros included, go to the smaller token id; `mapping` (may be NULL) renames column i —, 1 when
 * the row holds a non-finite logit).  scratch: rows * ceil(vocab / 1024) * 3 words. */
INGOT_API ingot_status ingot_greedy_select(ingot_gpu *gpu, const float *logits, const uint32_t *mapping, uint32_t rows,
                                           uint32_t vocab, uint32_t *scratch, uint32_t *out);

/* The packed MoE path at prefill width (Generic::moe_packed, src/generic.rs:578-660, with quant_expert_gemm and
 * indexed_gate_up, kernels/qwen.metal:895-1081): after ingot_expert_layout, ingot_gather_rows puts the
 * activation rows into packed order (y[pos] = x[packed[pos] / top]); ingot_expert_gemm_gate_up and
 * ingot_expert_gemm then run every expert's pairs — a contiguous run of packed rows — through the dense
 * operators (the tcgen05 GEMM for more than four pairs, the GEMV otherwise), driven by the (count, first)
 * table, which they read back to the host first (they wait for the stream; not inside a recording);
 * ingot_combine_packed finishes.  For a few pairs per expert ingot_expert_gate_up / ingot_expert_project
 * (below) stream each expert once without leaving the device. */
INGOT_API ingot_status ingot_gather_rows(ingot_gpu *gpu, const float *x, const uint32_t *packed, uint32_t pairs,
                                         uint32_t top, uint32_t width, float *y);
INGOT_API ingot_status ingot_expert_gemm(ingot_gpu *gpu, const void *w, uint32_t cols, uint32_t rows, uint32_t stride,
                                         uint32_t kind, uint32_t experts, const float *x_packed, const uint32_t *layout,
                                         uint32_t pairs, float *y_packed);
INGOT_API ingot_status ingot_expert_gemm_gate_up(ingot_gpu *gpu, const void *gate, const void *up, uint32_t cols,
                                                 uint32_t rows, uint32_t stride, uint32_t kind, uint32_t experts,
                                                 const float *x_packed, const uint32_t *layout, uint32_t pairs,
                                                 uint32_t gelu, float *y_packed);

/* expert_layout + expert_pairs (kernels/prefill.metal:7-35): stable
 * expert-major grouping of `pairs` ids.  layout [experts][2] = (count, first),
 * tiles [tile_capacity][4] = (expert, first, n <= 32, mode), packed[pos] =
 * pair index, inverse[pair] = pos. */
INGOT_API ingot_status ingot_expert_layout(ingot_gpu *gpu, const uint32_t *ids, uint32_t pairs,
                                           uint32_t experts, uint32_t tile_capacity, uint32_t *layout,
                                           uint32_t *tiles, uint32_t *packed, uint32_t *inverse);

/* The per-expert projections of the packed MoE path (Generic::moe_packed, src/generic.rs:578-660):
 * quant_expert_gather / quant_expert_packed (kernels/qwen.metal:953-999) and quant_expert_gate_up
 * (:1002-1081).  `tiles` and `pairs` are the tables of ingot_expert_layout; every tile's expert is
 * streamed once per four of its pairs.  x holds float32 rows: with gather, packed position q reads
 * row pairs[q] / top (the token's activations); without, row q (activations already in packed order,
 * the down projection).  y_packed[q][rows] is in packed order; ingot_combine_packed brings it back.
 * INGOT_UNSUPPORTED when the weight type or alignment has no grouped kernel (project pair by pair
 * with ingot_routed / ingot_routed_gate_up instead). */
INGOT_API ingot_status ingot_expert_project(ingot_gpu *gpu, const void *w, uint32_t cols, uint32_t rows, uint32_t stride,
                                            uint32_t kind, uint32_t experts, const float *x, const uint32_t *tiles,
                                            const uint32_t *pairs, uint32_t tile_capacity, uint32_t top, uint32_t n_pairs,
                                            uint32_t gather, float *y_packed);
INGOT_API ingot_status ingot_expert_gate_up(ingot_gpu *gpu, const void *gate, const void *up, uint32_t cols, uint32_t rows,
                                            uint32_t stride, uint32_t kind, uint32_t experts, const float *x,
                                            const uint32_t *tiles, const uint32_t *pairs, uint32_t tile_capacity,
                                            uint32_t top, uint32_t n_pairs, float *y_packed);

/* combine_packed without the shared expert (kernels/prefill.metal:39). */
INGOT_API ingot_status ingot_combine_packed(ingot_gpu *gpu, const float *routed, const float *weights,
                                            const uint32_t *inverse, uint32_t width, uint32_t top,
                                            uint32_t tokens, float *y);

/* Expert-parallel sharding of a routing result (no counterpart in the reference,
 * which keeps every expert on one device).  Pairs whose expert id lies in
 * [first_expert, first_expert + local_experts) keep their weight and get the local
 * id; the others get id 0xffffffff and weight 0.  ingot_routed / ingot_routed_gate_up
 * write zero rows for id 0xffffffff, so ingot_moe_sum then yields this device's partial
 * sum and an all-reduce over the devices the full one. */
INGOT_API ingot_status ingot_ep_localize(ingot_gpu *gpu, const uint32_t *ids, const float *weights, uint32_t pairs,
                                         uint32_t first_expert, uint32_t local_experts, uint32_t *ids_out,
                                         float *weights_out);

/* float32 -> bfloat16 (round to nearest even) for activations. */
INGOT_API ingot_status ingot_convert_bf16(ingot_gpu *gpu, const float *x, uint64_t n, void *y_bf16);

/* Activations in the order the tensor-core GEMV consumes them.  No counterpart in
 * the reference (its kernels read float32 x directly); on B200 packing once and
 * handing the same packed row to every projection that reads it (q, k, v; gate
 * and up) removes the conversion from each GEMV.  A packed row holds, for `cols`
 * (a multiple of 64) activations: binary16 (high, low) halves, the fp32 sum of
 * every 16 columns, and a power-of-two scale.  Pass it with x_kind =
 * INGOT_X_PACKED to ingot_matmul (count 1), ingot_gate_up (count 1), ingot_routed
 * and ingot_routed_gate_up; row r of `packed` starts at r * ingot_packed_x_bytes. */
INGOT_API ingot_status ingot_packed_x_bytes(uint32_t cols, uint64_t *bytes);
INGOT_API ingot_status ingot_pack_x(ingot_gpu *gpu, const void *x, uint32_t x_kind, uint32_t rows, uint32_t cols,
                                    void *packed);

/* High-part rows, for bfloat16 activations only: a bfloat16 value is exact in binary16
 * (up to underflow below 2^-24 of the row's scale), so the low parts of ingot_pack_x are
 * all zero and are left out: half the bytes, and with one part per token the eight
 * columns of the tensor-core operand hold EIGHT TOKENS.  Pass `count` rows (1 to any
 * number; they go through eight, or as many as fit in shared memory, at a time) with
 * x_kind = INGOT_X_PACKED_HI to ingot_matmul / ingot_gate_up: the weights are streamed
 * once per group of tokens (Q4_K, Q6_K with cols a multiple of 2048; one token: every
 * tensor-core GEMV type).  Rows of ingot_packed_hi_bytes(cols).  No counterpart in the
 * reference. */
INGOT_API ingot_status ingot_packed_hi_bytes(uint32_t cols, uint64_t *bytes);
INGOT_API ingot_status ingot_pack_x_hi(ingot_gpu *gpu, const void *x_bf16, uint32_t rows, uint32_t cols, void *packed);

/* Activations as the operand of the tcgen05 int8 GEMV (INGOT_OPT_TCGEN05_GEMV): every
 * value is round(x * S), S the power of two that puts the row's largest magnitude in
 * [2^21, 2^22), written as three signed base-256 digits in the shared-memory layout of
 * an N = 8 tensor-core operand, followed by the fp32 sum of every 16 columns and 1/S.
 * cols a multiple of 256; rows of ingot_packed_digits_bytes(cols); pass them with
 * x_kind = INGOT_X_DIGITS (one token).  No counterpart in the reference. */
INGOT_API ingot_status ingot_packed_digits_bytes(uint32_t cols, uint64_t *bytes);
INGOT_API ingot_status ingot_pack_digits(ingot_gpu *gpu, const void *x, uint32_t x_kind, uint32_t rows, uint32_t cols,
                                         void *packed);

/* No counterpart in the reference.  y = W[expert] x for ONE float32 activation row, for
 * callers that must not allocate: it takes no handle and calls neither cudaMalloc nor
 * cudaFree nor any allocating routine.  The scratch of the tensor-core GEMV and its error
 * word live in file-scope __device__ arrays of the library (about 70 KB per GPU, held
 * until the process exits), so cols is limited to 16384 (INGOT_INVALID beyond that;
 * ingot_matvec_static_error() gives the text).  The scratch array receives the packed copy
 * of x when x is only 4-byte aligned; a 16-byte aligned x is packed inside the kernel, in
 * shared memory, and only the error word is touched.  Served:
 * kinds 2, 8, 12, 14 with cols % 64 == 0 and 16-byte aligned rows (INGOT_UNSUPPORTED
 * otherwise).  The first call on a device looks up the arrays' device addresses
 * (cudaGetSymbolAddress) — make that first call outside any stream capture.  Work is
 * enqueued on `cuda_stream` of the CURRENT device; wait != 0 also waits for it and
 * reports a device-side time-out.  Every call uses the same scratch: two calls that
 * overlap on the GPU (different streams, no ordering) race — serialise them.  First calls
 * on a device from several host threads are serialised by the library (a lock around the
 * address look-up). */
INGOT_API ingot_status ingot_matvec_static(const void *w, uint32_t cols, uint32_t rows, uint32_t stride,
                                           uint32_t kind, uint32_t expert, const float *x, float *y,
                                           void *cuda_stream, int32_t wait);
INGOT_API const char *ingot_matvec_static_error(void);

/* ---- command recording (Command: src/metal.rs:659-673; a whole decode step
 *      is one command buffer, src/generic.rs:701-704) ---------------------- */

/* Starts recording the operators issued on this handle into a CUDA graph. */
INGOT_API ingot_status ingot_command_begin(ingot_gpu *gpu);
/* Ends recording; the graph can be replayed any number of times. */
INGOT_API ingot_status ingot_command_end(ingot_gpu *gpu, ingot_graph **out);
INGOT_API ingot_status ingot_command_submit(ingot_gpu *gpu, ingot_graph *graph);
INGOT_API void ingot_command_destroy(ingot_graph *graph);

/* ---- tensor-parallel groups: output rows sharded over the GPUs of one node -------------
 * No counterpart in the reference, whose Gpu owns one device (src/metal.rs:193-208).  Rank r of
 * `world` owns rows [r N / world, (r + 1) N / world) of every matrix (block quantisation runs
 * along K, so a row split keeps the GGUF layout).  Every rank has a WINDOW of device memory that
 * the other ranks can write: the activation vectors that have to be whole on every rank live
 * there, at the same offset on every rank, and each has a TAGGED TWIN behind the window: one
 * 8-byte word {value, tag} per element, the tag naming the step and the slot.  A fused-norm
 * projection marked with ingot_tp_signal_next stores its rows as plain floats where it was told
 * AND as tagged words, each with one 8-byte store, into the twin of every rank (over NVLink for
 * the peers).  A projection marked with ingot_tp_wait_next reads the awaited inputs from their
 * twins and polls each word until it carries this step's tag — with a time limit, reported as
 * INGOT_TIMEOUT by ingot_synchronize.  A word arrives whole or not at all, so the exchange needs
 * no fence, flag or counter, and no collective launch sits between two projections: it is the
 * epilogue of one kernel and the prologue of the next.  Every slot is signalled by exactly one
 * projection per step; ingot_group_step (once per step, first) advances the step counter.  The
 * plain copy of an exchanged vector holds only the own rows until ingot_group_wait fills it.
 *
 * One process per GPU: ingot_group_create returns 64 bytes (a CUDA IPC handle); gather the
 * handles of all ranks by any means (MPI, torch.distributed, a file) and pass the world x 64
 * bytes to ingot_group_connect.  One process driving several GPUs: create the groups, then
 * ingot_group_connect_local(groups, world).  A rank's kernels never wait for kernels of the
 * same GPU: do not put two ranks of a group on one device. */
typedef struct ingot_group ingot_group;
INGOT_API ingot_status ingot_group_create(ingot_gpu *gpu, uint32_t rank, uint32_t world, size_t window_bytes,
                                          uint32_t slots, ingot_group **out, void *handle64);
INGOT_API ingot_status ingot_group_connect(ingot_group *group, const void *handles);
INGOT_API ingot_status ingot_group_connect_local(ingot_group **groups, uint32_t world);
/* Base address of rank `rank`'s window as this process sees it (the own window: a device pointer
 * to allocate the shared activation vectors in; window_bytes of it are the caller's). */
INGOT_API ingot_status ingot_group_window(const ingot_group *group, uint32_t rank, void **base);
INGOT_API ingot_status ingot_group_step(ingot_group *group);
/* Enqueues a kernel that waits (time-limited) for every rank's rows of `slot` in this step and
 * copies them out of the twin into the plain vector `whole` (n floats, inside the own window):
 * what a reader outside the fused projections (attention, the sampler, the host) needs. */
INGOT_API ingot_status ingot_group_wait(ingot_group *group, uint32_t slot, float *whole, uint32_t n);
/* The next ingot_matmul_normed / ingot_gate_up_normed on the group's handle: its output (which
 * must lie inside the own window) also goes, tagged with `slot`, to the twin on every rank. */
INGOT_API ingot_status ingot_tp_signal_next(ingot_group *group, uint32_t slot);
/* The next fused-norm projection reads the vectors of slot_a and, unless 0xffffffff, slot_b from
 * their twins; each must be one of its two normalised inputs (the whole vector, in the window). */
INGOT_API ingot_status ingot_tp_wait_next(ingot_group *group, uint32_t slot_a, uint32_t slot_b);

/* ---- expert-parallel token exchange (a group whose ranks each own experts / world experts) ----
 * No counterpart in the reference, which keeps every expert on its one device
 * (src/weights.rs:55-58; dataflow of the layer: Generic::moe, src/generic.rs:508-574).  Every
 * rank routes its OWN tokens (ingot_route_topk); then, per layer:
 *   ingot_ep_dispatch  each pair's activation row and {local expert id, pair index} go into region
 *                      `rank` of the owner's receive area (plain stores over NVLink), unused places
 *                      of the region are marked skipped, one tagged word per owner closes the region
 *   ingot_ep_receive   waits (time-limited) for the regions of all ranks and writes ids_out[world x
 *                      cap] (local expert id or 0xffffffff) for ingot_routed_gate_up / ingot_routed
 *                      over the world x cap places (x = rx_rows, one row per place, top = 1)
 *   ingot_ep_return    each live place's output row (row `place` of `rows`, or row inverse[place] when
 *                      the places ran through the expert grouping: ingot_expert_layout accepts the
 *                      skipped places of ids_out and gives them no position) goes to the home rank's
 *                      ret_rows at the pair's index, one tagged word per home rank closes it
 *   ingot_ep_combine   waits (time-limited) for all owners, then y[t] = sum_k w[t][k] ret_rows[t top + k]
 *                      in route order — what ingot_moe_sum computes on one device, bit for bit.
 * The five areas lie inside the own window at the same offsets on every rank: rx_rows
 * [world][cap][hidden] floats, rx_meta [world][cap] words, rx_ready [world] 8-byte words, ret_rows
 * [cap][hidden] floats, ret_ready [world] 8-byte words; cap >= tokens x top of every rank, at
 * most 4096.  `slot` names the exchange within the step (two per layer: dispatch, return); a
 * wait that runs out is INGOT_TIMEOUT at the next ingot_synchronize. */
typedef struct ingot_ep_buffers {
    float *rx_rows;
    uint32_t *rx_meta;
    uint64_t *rx_ready;
    float *ret_rows;
    uint64_t *ret_ready;
} ingot_ep_buffers;
INGOT_API ingot_status ingot_ep_dispatch(ingot_group *group, uint32_t slot, const ingot_ep_buffers *bufs, const float *x,
                                         const uint32_t *ids, uint32_t tokens, uint32_t top, uint32_t hidden, uint32_t cap,
                                         uint32_t experts_per_rank);
INGOT_API ingot_status ingot_ep_receive(ingot_group *group, uint32_t slot, const ingot_ep_buffers *bufs, uint32_t hidden, uint32_t cap,
                                        uint32_t *ids_out);
INGOT_API ingot_status ingot_ep_return(ingot_group *group, uint32_t slot, const ingot_ep_buffers *bufs, const float *rows,
                                       const uint32_t *inverse, uint32_t hidden, uint32_t cap);
INGOT_API ingot_status ingot_ep_combine(ingot_group *group, uint32_t slot, const ingot_ep_buffers *bufs, const float *weights,
                                        uint32_t hidden, uint32_t top, uint32_t tokens, uint32_t cap, float *y);
INGOT_API void ingot_group_destroy(ingot_group *group);

/* ---- chains: a whole decode step as ONE kernel -----------------------------
 * The reference encodes a token's operators into one command buffer
 * (src/generic.rs:701-704) and Metal runs them back to back.  On B200 a chain of short,
 * dependent GEMV launches leaves HBM idle between them, so the projections of a step can
 * be recorded into a chain instead: between ingot_chain_begin and ingot_chain_end,
 * ingot_matmul_normed and ingot_gate_up_normed are collected, not launched (independent
 * scopes may be opened and closed; any other operator is INGOT_INVALID).  ingot_chain_end
 * works out from the buffer addresses which projection waits for which, lets projections
 * with the same normalised input (q, k, v) share it, and builds the list on the device.
 * ingot_chain_submit enqueues ONE cooperative kernel (one CTA per SM, all resident): a
 * producer warp per CTA streams the weights of projection after projection without
 * pause, the other warps wait — with a time limit, reported as INGOT_TIMEOUT by
 * ingot_synchronize — for the projections theirs depends on.  Results are those of the
 * same calls issued one by one.  INGOT_UNSUPPORTED when a recorded projection has no
 * fused tensor-core form or the types mix K-quants with Q4_0/Q8_0.  The buffers and
 * weights of the recorded calls must stay alive and in place while the chain is used. */
typedef struct ingot_chain ingot_chain;
INGOT_API ingot_status ingot_chain_begin(ingot_gpu *gpu);
INGOT_API ingot_status ingot_chain_end(ingot_gpu *gpu, ingot_chain **out);
INGOT_API ingot_status ingot_chain_submit(ingot_gpu *gpu, ingot_chain *chain);
/* Counts of a built chain (any pointer may be NULL): recorded projections, projections that
 * wait for another one, and the shared-memory ring (stages, bytes per stage). */
INGOT_API ingot_status ingot_chain_info(const ingot_chain *chain, uint32_t *projections, uint32_t *waits,
                                        uint32_t *stages, uint32_t *stage_bytes);
INGOT_API void ingot_chain_destroy(ingot_chain *chain);

/* ---- GGUF v3 files (src/gguf.rs) -------------------------------------------
 * Gguf::open (src/gguf.rs:205-271) with the directory rules of :121-202: little-endian
 * version 3; metadata types 0..12, arrays not nested, no duplicate key; general.alignment
 * (default 32) a power of two; tensors of rank 1..4 with no zero dimension, dims[0] a whole
 * number of blocks (geometry(): :470-491, every type the reference lists), aligned offsets,
 * no duplicate, none beyond the file, no overlap; split models through their primary shard.
 * Any violation is INGOT_INVALID; a positional read the file can no longer satisfy is
 * INGOT_EOF (io::ErrorKind::UnexpectedEof).  These functions take no GPU handle and keep
 * their error text per thread (ingot_gguf_last_error). */
typedef struct ingot_gguf ingot_gguf;

/* Tensor (src/gguf.rs:18-25): dims[0] = cols (contiguous), dims[1] = rows, dims[2] = experts;
 * offset = absolute byte offset in file `shard`; stride = bytes of one row; bytes = all rows. */
typedef struct ingot_tensor_info {
    uint64_t dims[4];
    uint32_t rank, kind;
    uint64_t offset;
    uint32_t shard, reserved;
    uint64_t stride, bytes;
} ingot_tensor_info;

INGOT_API ingot_status ingot_gguf_open(const char *path, ingot_gguf **out);
INGOT_API void ingot_gguf_close(ingot_gguf *gguf);
INGOT_API const char *ingot_gguf_last_error(void);
INGOT_API const char *ingot_gguf_architecture(const ingot_gguf *gguf);
INGOT_API uint64_t ingot_gguf_tensor_count(const ingot_gguf *gguf);
/* Gguf::bytes_read: bytes delivered by successful positional reads. */
INGOT_API uint64_t ingot_gguf_bytes_read(const ingot_gguf *gguf);
INGOT_API ingot_status ingot_gguf_tensor_at(const ingot_gguf *gguf, uint64_t index, const char **name,
                                            ingot_tensor_info *info);
/* Gguf::tensor (:338-342): "missing tensor" is INGOT_INVALID. */
INGOT_API ingot_status ingot_gguf_tensor(const ingot_gguf *gguf, const char *name, ingot_tensor_info *info);
/* Gguf::integer / float / string / array accessors (:273-337); a missing key or a value of another
 * type is INGOT_INVALID.  Returned strings live as long as the handle. */
INGOT_API ingot_status ingot_gguf_integer(const ingot_gguf *gguf, const char *key, uint64_t *value);
INGOT_API ingot_status ingot_gguf_float(const ingot_gguf *gguf, const char *key, float *value);
INGOT_API ingot_status ingot_gguf_string(const ingot_gguf *gguf, const char *key, const char **value);
INGOT_API ingot_status ingot_gguf_array_length(const ingot_gguf *gguf, const char *key, uint64_t *length);
INGOT_API ingot_status ingot_gguf_array_integer(const ingot_gguf *gguf, const char *key, uint64_t index, uint64_t *value);
INGOT_API ingot_status ingot_gguf_array_string(const ingot_gguf *gguf, const char *key, uint64_t index, const char **value);
/* Gguf::read_range (:361-366): `len` bytes at `offset` inside the tensor. */
INGOT_API ingot_status ingot_gguf_read_range(ingot_gguf *gguf, const ingot_tensor_info *tensor, uint64_t offset, void *dst,
                                             uint64_t len);
/* Gguf::rows (:417-447): rows[i] of the tensor, in caller order (repeats allowed), `n` x stride bytes. */
INGOT_API ingot_status ingot_gguf_rows(ingot_gguf *gguf, const char *name, const uint64_t *rows, uint64_t n, void *dst);
/* Gguf::matrix (:448-476): the listed experts of a tensor whose dims equal `shape`. */
INGOT_API ingot_status ingot_gguf_matrix(ingot_gguf *gguf, const char *name, const uint64_t *shape, uint32_t rank,
                                         const uint64_t *experts, uint64_t n_experts, void *dst);
/* Weight::load (src/weights.rs:22-32) + Gpu::load_weight (src/metal.rs:546-582): checks the shape,
 * reads the tensor through a pinned staging buffer and uploads it (a discrete GPU cannot map the
 * file in place).  *device is released with ingot_buffer_free. */
INGOT_API ingot_status ingot_weight_load(ingot_gpu *gpu, ingot_gguf *gguf, const char *name, const uint64_t *shape,
                                         uint32_t rank, void **device, ingot_tensor_info *info);

/* ---- host-vector conveniences (the reference's public parity hooks) ------ */

/* Gpu::dequant(&Matrix) (src/metal.rs:1581-1601) with validate_matrix
 * (src/metal.rs:1602-1621): data is `count` experts of rows x stride bytes. */
INGOT_API ingot_status ingot_dequant_host(ingot_gpu *gpu, const void *data, size_t data_bytes, uint64_t cols,
                                          uint64_t rows, uint64_t count, uint32_t kind, uint64_t stride,
                                          float *out);

/* Gpu::ffn (src/metal.rs:1634-1661) on device buffers: `count` stacked experts' SwiGLU FFN of the same
 * input x[width]: gate and up are [count][inner][width], down is [count][width][inner], all of
 * `kind`; scratch holds 3 x inner x count floats; expert_ids = 0 .. count - 1 on the device;
 * out[count][width]. */
INGOT_API ingot_status ingot_ffn(ingot_gpu *gpu, const void *gate, const void *up, const void *down, uint32_t width,
                                 uint32_t inner, uint32_t count, uint32_t kind, const float *x, float *scratch,
                                 const uint32_t *expert_ids, float *out);

/* Gpu::moe(&[Matrix; 3], &[Matrix; 3], &Matrix, &[f32], &[f32]) (src/metal.rs:1663-1713) with host
 * vectors: routed = the selected experts' gate, up, down stacked (count = weights), shared = the
 * shared expert's three (count 1), shared_gate [1][width];
 * out[j] = sum_e weights[e] routed_e[j] + sigmoid(shared_gate . x) shared[j].  Shape and
 * finiteness errors are INGOT_INVALID with the reference's messages. */
typedef struct ingot_host_matrix {
    const void *data;
    size_t bytes;
    uint64_t cols, rows, count;
    uint32_t kind;
    uint64_t stride;
} ingot_host_matrix;
INGOT_API ingot_status ingot_moe_host(ingot_gpu *gpu, const ingot_host_matrix routed[3], const ingot_host_matrix shared[3],
                                      const ingot_host_matrix *shared_gate, const float *input, size_t width,
                                      const float *weights, size_t n_weights, float *out);

/* Gpu::project(&Matrix, &[f32]) (src/metal.rs:1622-1632): count must be 1,
 * input finite and of length cols. */
INGOT_API ingot_status ingot_project_host(ingot_gpu *gpu, const void *data, size_t data_bytes, uint64_t cols,
                                          uint64_t rows, uint64_t count, uint32_t kind, uint64_t stride,
                                          const float *input, size_t input_len, float *out);

#ifdef __cplusplus
}
#endif
#endif /* INGOT_CUDA_H */
