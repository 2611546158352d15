// Internal launch interface between the C ABI (abi.cu) and the kernel files.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace ingot {

// A kernel's dynamic shared-memory limit is a per-device attribute: set it once per (kernel
// instantiation, device) — one static DeviceOnce per instantiation, a bit per device ordinal — and
// safely from several host threads (setting it twice is harmless, skipping it is not).
struct DeviceOnce {
    std::atomic<uint64_t> mask{0};
    template <typename K>
    cudaError_t smem(K kernel, int bytes) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        const uint64_t bit = 1ull << (dev & 63);
        if (mask.load(std::memory_order_acquire) & bit) return cudaSuccess;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e == cudaSuccess) mask.fetch_or(bit, std::memory_order_release);
        return e;
    }
};

// Codes kernels write to the device status word (0 = ok).
enum : int {
    KERNEL_OK = 0,
    KERNEL_ERR_PRODUCER_TIMEOUT = 1,   // ring stage never freed
    KERNEL_ERR_CONSUMER_TIMEOUT = 2,   // bulk copy never landed
    KERNEL_ERR_EXPERT_RANGE = 3,       // routed id >= number of experts
    KERNEL_ERR_ROUTER_INPUT = 4,       // non-finite router logit
    KERNEL_ERR_GEMM_TIMEOUT = 5,       // prefill GEMM pipeline wait ran out
    KERNEL_ERR_CHAIN_TIMEOUT = 6,      // a projection of a chain kernel never saw the one it depends on finish
    KERNEL_ERR_PEER_TIMEOUT = 7        // a row-sharded projection never saw every rank's shard of its input arrive
};

// Tensor-parallel links of one projection (all null / zero on a single GPU).
static constexpr uint32_t TP_MAX_RANKS = 8;
struct TpLink {
    // A vector that is assembled from every rank's rows has a tagged twin in each rank's window: one 8-byte word
    // {value, tag} per element, stored whole (so a reader sees either the old word or the new one), the tag naming the
    // step and the projection that wrote it.  A reader polls the words themselves: no fence, flag or arrival count.
    uint64_t *out[TP_MAX_RANKS];            // this output's tagged twin on every rank, the own one included
    uint32_t n_out;
    uint32_t out_tag;                       // this step's tag of the output = step * tag_mul + out_tag
    const uint64_t *in[2];                  // tagged twins of the two normalised inputs (null: a plain vector)
    uint32_t in_tag[2];
    uint32_t tag_mul;
    const uint32_t *step;                   // own step counter (1 in the first step)
};

// Expert-parallel exchange areas of one rank's window as every rank sees them (index = rank).
static constexpr uint32_t EP_MAX_PAIRS = 4096;
struct EpLink {
    float *rx_rows[TP_MAX_RANKS];           // [world][cap][hidden]: region s holds the rows rank s sent
    uint32_t *rx_meta[TP_MAX_RANKS];        // [world][cap]: local expert id | pair index << 16, or ROUTE_SKIP
    uint64_t *rx_ready[TP_MAX_RANKS];       // [world] tagged: region s is complete (low half: its live places)
    float *ret_rows[TP_MAX_RANKS];          // [cap][hidden]: the outputs of the rank's own pairs, by pair index
    uint64_t *ret_ready[TP_MAX_RANKS];      // [world] tagged: owner s has returned everything it had
    uint32_t *launch_count;                 // own device: CTAs of this kind of launch so far (the last one of a launch signals)
    const uint32_t *step;
    uint32_t tag_mul, tag_add, world, rank;
};

struct LaunchCtx {
    cudaStream_t stream;
    int *status;          // device status word
    uint32_t sm_count;
    bool pdl;             // launch with programmatic stream serialization
    bool force_plain;     // test hook: skip the streaming kernels
    bool no_mma;          // test hook: use the fp32 CUDA-core streaming kernel instead of the MMA one
    void *workspace;      // device scratch of the handle (packed activations)
    size_t workspace_bytes;
    uint32_t ep_world;    // experts are split over this many devices: about pairs / ep_world routed pairs are live
    bool use_tc;          // one-token Q4_K GEMVs go to the tcgen05 int8 kernel
    void *tc_scratch;     // its tile counters (TC_COUNTER_BYTES, zero between launches) and partial rows
    size_t tc_scratch_bytes;
};
static constexpr size_t TC_COUNTER_BYTES = 64u * 1024u;

// y = W x for `count` tokens (dense) or `pairs` (token, expert) pairs (routed,
// ids != null).  nmat == 2 fuses two matrices and stores glu(gate, up).
struct GemvCall {
    const uint8_t *w[2];
    const void *x;
    float *y;
    const uint32_t *ids;
    uint32_t cols, rows, stride, kind;
    uint32_t expert;       // dense
    uint32_t count;        // dense tokens
    uint32_t pairs, top, per_pair, n_experts;   // routed
    uint32_t x_bf16;
    uint32_t x_packed;     // x is already packed: 1 = packed_x_bytes(cols) rows (launch_pack_x), 3 = digit rows (launch_pack_digits), 4 = high-part rows (launch_pack_x_hi)
    uint32_t nmat, glu;    // glu: 1 silu, 2 tanh-gelu
    // fused input normalisation (tensor-core GEMV, dense, one token): x = rms_norm(norm_a + norm_b) * norm_w,
    // optionally rounded to bfloat16; norm_s receives norm_a + norm_b.  x is ignored when norm_a is set.
    const float *norm_a, *norm_b, *norm_w;
    float *norm_s;
    float norm_eps;
    uint32_t norm_round_bf16;
    uint32_t norm_wide;    // four-digit rows even when rounding to bfloat16
    TpLink tp;
};
cudaError_t launch_gemv(const GemvCall &c, const LaunchCtx &ctx);
// The tensor-core-assisted streaming GEMV; false when the call is not one it handles.
bool try_launch_gemv_mma(const GemvCall &c, const LaunchCtx &ctx, cudaError_t &err);
// Two or more float32 rows against one dense matrix: one pass over the weights per four rows, each row's bits those of the one-token kernel.
bool try_launch_gemv_rows(const GemvCall &c, const LaunchCtx &ctx, cudaError_t &err);
// Several independent one-token projections as one grid (2..4 calls that gemv_mma_group_eligible accepts).
bool gemv_mma_group_eligible(const GemvCall &c, const LaunchCtx &ctx);
// Loads the kernels a tensor-parallel group's projections use onto the current device (before the first step).
cudaError_t preload_exchange_kernels();
bool try_launch_gemv_mma_group(const GemvCall *calls, uint32_t n, const LaunchCtx &ctx, cudaError_t &err);
// A recorded sequence of one-token fused-norm projections run by one persistent kernel: built once
// (device copies of the projection list and its completion counters), launched any number of times.
struct ChainLaunch {
    void *ops_dev = nullptr;
    uint32_t *done_dev = nullptr;
    void *maps_dev = nullptr;          // tensor maps of the recorded matrices (one tiled copy per stage)
    void *trace_dev = nullptr;         // debugging (INGOT_CHAIN_TRACE=1): per-projection times of CTA 0, printed when the chain is freed
    uint32_t n_ops = 0, ctas = 0, smem_bytes = 0, xm = 0, family = 0;
    uint32_t slots = 0, slot_bytes = 0, waits = 0, occ = 1, warps = 8;
};
bool chain_call_eligible(const GemvCall &c);
// cudaErrorNotSupported (with `why`) when the calls cannot run as one chain.
cudaError_t chain_build(const GemvCall *calls, uint32_t n, const LaunchCtx &ctx, ChainLaunch &out, const char *&why);
cudaError_t chain_launch(const ChainLaunch &c, const LaunchCtx &ctx);
void chain_free(ChainLaunch &c);
// Routed projections grouped by expert: the tiles and pairs tables of launch_expert_layout; x float32 rows; results in
// packed positions.  False when the call is not one the kernel handles.
bool try_launch_gemv_tiles(const GemvCall &c, const uint32_t *tiles, const uint32_t *pairs, uint32_t tile_capacity, bool gather,
                           const LaunchCtx &ctx, cudaError_t &err);
// The tcgen05 int8 GEMV (one token, Q4_K); false when the call is not one it handles.
bool try_launch_gemv_tc(const GemvCall &c, const LaunchCtx &ctx, cudaError_t &err);
// Packs `rows` activation rows (f32 or bf16) as base-256 digits for it.
cudaError_t launch_pack_digits(const void *x, uint32_t bf16, uint32_t rows, uint32_t cols, void *packed, const LaunchCtx &ctx);
// The tensor-core GEMV for 2..8 tokens whose activations are high-part rows (x_packed == 4); false when not handled.
bool try_launch_gemv_mt(const GemvCall &c, const LaunchCtx &ctx, cudaError_t &err);
// Packs `rows` bfloat16 activation rows as high-part rows (packed_hi_bytes(cols) each).
cudaError_t launch_pack_x_hi(const void *x_bf16, uint32_t rows, uint32_t cols, void *packed, const LaunchCtx &ctx);
// Packs `rows` activation rows (f32 or bf16) for the tensor-core GEMV.
cudaError_t launch_pack_x(const void *x, uint32_t bf16, uint32_t rows, uint32_t cols, void *packed, const LaunchCtx &ctx);

// out[r][j] = weight_at(row r, j) for rows*cols elements.
cudaError_t launch_dequant(const uint8_t *w, uint32_t cols, uint64_t rows, uint32_t stride, uint32_t kind,
                           float *out, const LaunchCtx &ctx);

cudaError_t launch_route_topk(const float *logits, uint32_t experts, uint32_t top, uint32_t tokens, uint32_t *ids,
                              float *weights, const LaunchCtx &ctx);
cudaError_t launch_moe_sum(const float *routed, const float *w, uint32_t width, uint32_t top, uint32_t tokens,
                           float *y, const LaunchCtx &ctx);
// y[pos] = x[pairs[pos] / top]: activation rows in the expert grouping's packed order
cudaError_t launch_gather_rows(const float *x, const uint32_t *pairs, uint32_t n, uint32_t top, uint32_t width, float *y, const LaunchCtx &ctx);
// scale (0), soft-cap (1), SwiGLU over fused gate|up rows (2), column copy (3): kernels/generic_arch.metal:2-17
cudaError_t launch_glue(uint32_t op, const float *x, uint64_t n, uint32_t width, uint32_t offset, uint32_t stride, float value, float *y,
                        const LaunchCtx &ctx);
cudaError_t launch_activation(const float *gate, const float *up, uint64_t n, uint32_t gelu, float *y,
                              const LaunchCtx &ctx);
cudaError_t launch_merge(const float *routed, const float *shared, const float *weights, const float *shared_logit,
                         uint32_t width, uint32_t top, float *y, const LaunchCtx &ctx);
cudaError_t launch_add_rms(const float *a, const float *b, const float *w, float *s, float *y, uint32_t width,
                           uint32_t rows, float eps, uint32_t add, void *y_bf16, void *y_packed, uint32_t pack_bf16,
                           const LaunchCtx &ctx);
cudaError_t launch_expert_layout(const uint32_t *ids, uint32_t n_pairs, uint32_t experts, uint32_t tile_capacity,
                                 uint32_t *layout, uint32_t *tiles, uint32_t *pairs, uint32_t *inverse,
                                 const LaunchCtx &ctx);
cudaError_t launch_combine_packed(const float *routed, const float *w, const uint32_t *inverse, uint32_t width,
                                  uint32_t top, uint32_t tokens, float *y, const LaunchCtx &ctx);
// Y[T][N] = X[T][K] W^T with binary16 operand staging on tcgen05 (Q4_K, Q6_K).  x_half_scratch:
// gemm_scratch_bytes(...) bytes (the binary16 activations, then the partial products of a K split).
size_t gemm_scratch_bytes(uint32_t cols, uint32_t rows, uint32_t tokens, uint32_t sm_count);
cudaError_t launch_gemm_dequant(const uint8_t *w, uint32_t cols, uint32_t rows, uint32_t stride, uint32_t kind, uint32_t expert,
                                const void *x, uint32_t x_bf16, uint32_t tokens, float *y, void *x_half_scratch,
                                const LaunchCtx &ctx);
cudaError_t launch_ep_localize(const uint32_t *ids, const float *w, uint32_t pairs, uint32_t first, uint32_t count,
                               uint32_t *ids_out, float *w_out, const LaunchCtx &ctx);
cudaError_t launch_convert_bf16(const float *x, uint64_t n, void *y_bf16, const LaunchCtx &ctx);
// *counter += 1 by one thread (the step counter of a tensor-parallel group).
cudaError_t launch_increment(uint32_t *counter, const LaunchCtx &ctx);
// Expert-parallel token exchange (dispatch to the experts' owners, receive, return, weighted sum at home).
cudaError_t launch_ep_dispatch(const EpLink &link, const float *x, const uint32_t *ids, uint32_t pairs, uint32_t top, uint32_t hidden,
                               uint32_t cap, uint32_t experts_per_rank, const LaunchCtx &ctx);
cudaError_t launch_ep_receive(const EpLink &link, uint32_t cap, uint32_t *ids_out, const LaunchCtx &ctx);
cudaError_t launch_ep_return(const EpLink &link, const float *rows, const uint32_t *inverse, uint32_t cap, uint32_t hidden,
                             const LaunchCtx &ctx);
cudaError_t launch_ep_combine(const EpLink &link, const float *w, uint32_t hidden, uint32_t top, uint32_t tokens, float *y,
                              const LaunchCtx &ctx);
// One thread waits, with the time limit, until *counter has reached *step x arrivals (counters raised by other GPUs).
cudaError_t launch_collect_tagged(const uint64_t *tagged, float *plain, uint32_t n, const uint32_t *step, uint32_t tag_mul, uint32_t tag_add, const LaunchCtx &ctx);

// The rest of a generic decode step (decode_ops.cu).
struct RopeParams {
    uint32_t head_dim, heads, kv_heads, rotated, position;
    float base;
    uint32_t neox, use_factors, qk_norm;
    float eps;
    uint32_t value_norm;
    float q_scale;
};
cudaError_t launch_embedding(const uint8_t *w, const uint32_t *ids, uint32_t width, uint32_t stride, uint32_t kind, uint32_t count,
                             uint32_t vocab, float *y, const LaunchCtx &ctx);
cudaError_t launch_rope_cache(const float *q, const float *k, const float *v, const float *qn, const float *kn, const float *factors,
                              float *qo, float *kc, float *vc, const RopeParams &p, uint32_t tokens, const LaunchCtx &ctx);
cudaError_t launch_attention_decode(const float *q, const float *k, const float *v, float *out, uint32_t head_dim, uint32_t heads,
                                    uint32_t kv_heads, uint32_t position, uint32_t window, uint32_t tokens, const LaunchCtx &ctx);
// partial: rows * ceil(vocab / 1024) * 3 words of scratch; out: rows * 2 words (token, non-finite flag).
cudaError_t launch_greedy(const float *logits, const uint32_t *mapping, uint32_t rows, uint32_t vocab, uint32_t *partial, uint32_t *out,
                          const LaunchCtx &ctx);

}  // namespace ingot
