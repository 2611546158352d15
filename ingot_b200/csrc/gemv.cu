// GEMV kernels: the bulk-copy streaming kernel for block-quantised weights and
// the plain one-warp-per-row kernel for everything else (float weights,
// unaligned rows).  Dense, fused gate/up and expert-routed forms share both.
#include "dev_common.cuh"
#include "gemv_core.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace ingot {

// ---------------------------------------------------------------------------
// Streaming kernel
// ---------------------------------------------------------------------------

struct GemvArgs {
    GemvPlan plan;
    const uint8_t *w[2];      // weight matrices (expert 0); w[1] only for gate/up
    const void *x;            // activations, f32 or bf16
    float *y;
    const uint32_t *ids;      // routed: expert of each pair (grid.y), else null
    uint32_t expert;          // dense: expert index
    uint32_t n_experts;       // routed: ids must be below this
    uint32_t per_pair, top;   // routed: input row = per_pair ? pair : pair / top
    uint32_t x_bf16;
    uint32_t glu;             // nmat == 2: 1 silu, 2 tanh-gelu
    int *status;              // device status word (0 = ok)
};

template <uint32_t KIND>
__device__ __forceinline__ void stage_x(F4 *xs, const GemvArgs &a, uint32_t x_row0, uint32_t ntok, uint32_t tid,
                                        uint32_t nthreads) {
    const GemvPlan &p = a.plan;
    const uint32_t n4 = p.cols >> 2;
    for (uint32_t t = 0; t < ntok; ++t) {
        const size_t base = (size_t)(x_row0 + t) * p.cols;
        for (uint32_t f = tid; f < n4; f += nthreads) {
            F4 v;
            if (a.x_bf16) {
                const uint2 raw = *reinterpret_cast<const uint2 *>(static_cast<const uint16_t *>(a.x) + base + 4u * f);
                v = permute_x(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                              __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
            } else {
                const float4 raw = *reinterpret_cast<const float4 *>(static_cast<const float *>(a.x) + base + 4u * f);
                v = permute_x(raw.x, raw.y, raw.z, raw.w);
            }
            uint32_t u, i;
            Unit<KIND>::locate(4u * f, u, i);
            xs[x_slot(p, t, u, i)] = v;
        }
    }
}

template <uint32_t KIND, int NTOK, int NMAT>
__global__ void __launch_bounds__(GEMV_THREADS, 2) gemv_stream_kernel(const __grid_constant__ GemvArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const GemvPlan &p = a.plan;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + GEMV_MAX_STAGES;
    F4 *xs = reinterpret_cast<F4 *>(smem + GEMV_BAR_BYTES);
    uint8_t *stages = smem + GEMV_BAR_BYTES + ((p.x_bytes + 127u) & ~127u);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], GEMV_CONSUMER_WARPS);
        }
        ptx::mbar_init_fence();
    }
    __syncthreads();
    ptx::pdl_launch_dependents();

    uint32_t r_begin, r_end;
    cta_rows(p.rows, blockIdx.x, gridDim.x, r_begin, r_end);
    const uint32_t n_tiles = (r_end - r_begin + p.tile_rows - 1) / p.tile_rows;
    const uint32_t pair = blockIdx.y;

    if (warp == GEMV_CONSUMER_WARPS) {
        // ---- producer warp: stream this CTA's rows through the ring ----
        uint32_t expert = a.expert;
        if (a.ids) {                 // ids come from the previous kernel
            ptx::pdl_wait();
            expert = a.ids[pair];
            if (expert >= a.n_experts) return;       // consumers report it
        }
        const size_t mat_off = (size_t)expert * p.rows * p.stride;
        uint32_t it = 0;
        for (uint32_t tile = 0; tile < n_tiles; ++tile) {
            const uint32_t row0 = r_begin + tile * p.tile_rows;
            const uint32_t nrows = (r_end - row0) < p.tile_rows ? (r_end - row0) : p.tile_rows;
            for (uint32_t c = 0; c < p.chunks; ++c, ++it) {
                const uint32_t s = it % p.stages, ph = (it / p.stages) & 1u;
                bool ok = true;
                if (lane == 0) ok = ptx::mbar_wait(&empty[s], ph ^ 1u);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { if (lane == 0) set_status_word(a.status, KERNEL_ERR_PRODUCER_TIMEOUT); return; }
                const uint32_t cb = (c + 1 == p.chunks) ? p.last_chunk_bytes : p.chunk_bytes;
                uint8_t *dst = stages + (size_t)s * p.stage_bytes;
                if (lane == 0) ptx::mbar_expect_tx(&full[s], cb * nrows * NMAT);
                __syncwarp();
                if (p.chunks == 1) {            // whole rows: the tile is one contiguous run
                    if (lane < NMAT)
                        ptx::bulk_g2s(dst + (size_t)lane * p.tile_rows * p.chunk_bytes,
                                      a.w[lane] + mat_off + (size_t)row0 * p.stride, cb * nrows, &full[s]);
                } else {
                    for (uint32_t i = lane; i < nrows * NMAT; i += 32u) {
                        const uint32_t m = i / nrows, r = i - m * nrows;
                        ptx::bulk_g2s(dst + (size_t)(m * p.tile_rows + r) * p.chunk_bytes,
                                      a.w[m] + mat_off + (size_t)(row0 + r) * p.stride + (size_t)c * p.chunk_bytes,
                                      cb, &full[s]);
                    }
                }
            }
        }
        return;
    }

    // ---- consumer warps ----
    ptx::pdl_wait();
    uint32_t x_row0 = 0;
    if (a.ids) {
        const uint32_t e = a.ids[pair];
        if (e >= a.n_experts) {
            if (e == ROUTE_SKIP) {                      // not this device's expert: the row is zero
                float *yz = a.y + (size_t)pair * p.rows;
                for (uint32_t r = r_begin + threadIdx.x; r < r_end; r += GEMV_CONSUMER_WARPS * 32) yz[r] = 0.f;
            } else if (threadIdx.x == 0) set_status_word(a.status, KERNEL_ERR_EXPERT_RANGE);
            return;
        }
        x_row0 = a.per_pair ? pair : pair / a.top;
    }
    stage_x<KIND>(xs, a, x_row0, NTOK, threadIdx.x, GEMV_CONSUMER_WARPS * 32);
    ptx::named_bar_sync(1, GEMV_CONSUMER_WARPS * 32);

    const uint32_t lpr = 1u << p.lpr_log2, sub = lane & (lpr - 1u), rs = lane >> p.lpr_log2;
    const uint32_t slots = 32u >> p.lpr_log2;
    float *y = a.y + (a.ids ? (size_t)pair * p.rows : 0);
    uint32_t it = 0;
    for (uint32_t tile = 0; tile < n_tiles; ++tile) {
        const uint32_t row0 = r_begin + tile * p.tile_rows;
        const uint32_t nrows = (r_end - row0) < p.tile_rows ? (r_end - row0) : p.tile_rows;
        float acc[GEMV_NR][NMAT][NTOK];
#pragma unroll
        for (int nr = 0; nr < GEMV_NR; ++nr)
#pragma unroll
            for (int m = 0; m < NMAT; ++m)
#pragma unroll
                for (int t = 0; t < NTOK; ++t) acc[nr][m][t] = 0.f;
        for (uint32_t c = 0; c < p.chunks; ++c, ++it) {
            const uint32_t s = it % p.stages, ph = (it / p.stages) & 1u;
            if (!ptx::mbar_wait(&full[s], ph)) {
                if (lane == 0) set_status_word(a.status, KERNEL_ERR_CONSUMER_TIMEOUT);
                return;
            }
            consume_chunk<KIND, NTOK, NMAT>(stages + (size_t)s * p.stage_bytes, xs, p, warp, lane, c, nrows, acc);
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty[s]);
        }
#pragma unroll
        for (int nr = 0; nr < GEMV_NR; ++nr) {
            const uint32_t lrow = (warp * GEMV_NR + nr) * slots + rs;
#pragma unroll
            for (int t = 0; t < NTOK; ++t) {
                float v[NMAT];
#pragma unroll
                for (int m = 0; m < NMAT; ++m) {
                    v[m] = acc[nr][m][t];
                    for (uint32_t off = lpr >> 1; off; off >>= 1) v[m] = add_rn(v[m], __shfl_xor_sync(0xffffffffu, v[m], off));
                }
                if (sub == 0 && lrow < nrows) {
                    const size_t o = (size_t)t * p.rows + row0 + lrow;
                    if (NMAT == 2) y[o] = glu_f(v[0], v[NMAT - 1], a.glu == 2);
                    else y[o] = v[0];
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Plain kernel: one warp per (row, token-or-pair); lanes stride over columns
// with the scalar decoder (the shape of the reference's dot_quant_row /
// project_routed_batch: kernels/qwen.metal:93-112).  Any type, any alignment.
// ---------------------------------------------------------------------------

struct PlainArgs {
    const uint8_t *w[2];
    const void *x;
    float *y;
    const uint32_t *ids;
    uint32_t cols, rows, stride, kind, expert, n_experts, per_pair, top, x_bf16, nmat, glu, count;
    int *status;
};

__global__ void __launch_bounds__(128) gemv_plain_kernel(const __grid_constant__ PlainArgs a) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t row = blockIdx.x * 4u + (threadIdx.x >> 5);
    const uint32_t item = blockIdx.y;                 // token (dense) or pair (routed)
    if (row >= a.rows) return;
    uint32_t expert = a.expert, x_row = item;
    if (a.ids) {
        expert = a.ids[item];
        if (expert >= a.n_experts) {
            if (expert == ROUTE_SKIP) { if (lane == 0) a.y[(size_t)item * a.rows + row] = 0.f; }
            else if (lane == 0 && row == 0) set_status_word(a.status, KERNEL_ERR_EXPERT_RANGE);
            return;
        }
        x_row = a.per_pair ? item : item / a.top;
    }
    const size_t woff = ((size_t)expert * a.rows + row) * a.stride;
    const size_t xoff = (size_t)x_row * a.cols;
    float v[2] = {0.f, 0.f};
    for (uint32_t m = 0; m < a.nmat; ++m) {
        const uint8_t *wr = a.w[m] + woff;
        float s = 0.f;
        for (uint32_t j = lane; j < a.cols; j += 32u) s = fma_rn(weight_at(wr, a.kind, j), load_x(a.x, xoff + j, a.x_bf16), s);
        for (uint32_t off = 16; off; off >>= 1) s = add_rn(s, __shfl_xor_sync(0xffffffffu, s, off));
        v[m] = s;
    }
    if (lane == 0) a.y[(size_t)item * a.rows + row] = a.nmat == 2 ? glu_f(v[0], v[1], a.glu == 2) : v[0];
}

// ---------------------------------------------------------------------------
// Launch
// ---------------------------------------------------------------------------

template <uint32_t KIND, int NTOK, int NMAT>
static cudaError_t launch_stream_t(const GemvArgs &a, dim3 grid, cudaStream_t stream, bool pdl) {
    auto kernel = gemv_stream_kernel<KIND, NTOK, NMAT>;
    static DeviceOnce once;
    {
        const cudaError_t e = once.smem(kernel, (int)GEMV_SMEM_MAX);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = a.plan.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, a);
}

template <uint32_t KIND, int NMAT>
static cudaError_t launch_stream_n(const GemvArgs &a, dim3 grid, cudaStream_t stream, bool pdl) {
    switch (a.plan.ntok) {
    case 1: return launch_stream_t<KIND, 1, NMAT>(a, grid, stream, pdl);
    case 2: return launch_stream_t<KIND, 2, NMAT>(a, grid, stream, pdl);
    case 3: return launch_stream_t<KIND, 3, NMAT>(a, grid, stream, pdl);
    case 4: return launch_stream_t<KIND, 4, NMAT>(a, grid, stream, pdl);
    default: return cudaErrorInvalidValue;
    }
}

template <uint32_t KIND>
static cudaError_t launch_stream_k(const GemvArgs &a, dim3 grid, cudaStream_t stream, bool pdl) {
    return a.plan.nmat == 2 ? launch_stream_n<KIND, 2>(a, grid, stream, pdl) : launch_stream_n<KIND, 1>(a, grid, stream, pdl);
}

static cudaError_t launch_stream(const GemvArgs &a, dim3 grid, cudaStream_t stream, bool pdl) {
    switch (a.plan.kind) {
    case KIND_Q4_K: return launch_stream_k<KIND_Q4_K>(a, grid, stream, pdl);
    case KIND_Q6_K: return launch_stream_k<KIND_Q6_K>(a, grid, stream, pdl);
    case KIND_Q4_0: return launch_stream_k<KIND_Q4_0>(a, grid, stream, pdl);
    case KIND_Q8_0: return launch_stream_k<KIND_Q8_0>(a, grid, stream, pdl);
    default: return cudaErrorInvalidValue;
    }
}

static cudaError_t launch_plain(const PlainArgs &a, uint32_t items, cudaStream_t stream, bool pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((a.rows + 3u) / 4u, items);
    cfg.blockDim = dim3(128);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gemv_plain_kernel, a);
}

cudaError_t launch_gemv(const GemvCall &c, const LaunchCtx &ctx) {
    const bool routed = c.ids != nullptr;
    const uint32_t items = routed ? c.pairs : c.count;
    if (items == 0) return cudaSuccess;
    const bool aligned = ((uintptr_t)c.w[0] % 16u) == 0 && (c.nmat < 2 || ((uintptr_t)c.w[1] % 16u) == 0) &&
                         ((uintptr_t)c.x % 16u) == 0 && ((size_t)c.rows * c.stride) % 16u == 0;
    if (!ctx.force_plain && !ctx.no_mma && aligned) {
        cudaError_t e = cudaSuccess;
        if (ctx.use_tc && try_launch_gemv_tc(c, ctx, e)) return e;
        if (try_launch_gemv_mma(c, ctx, e)) return e;
        if (try_launch_gemv_rows(c, ctx, e)) return e;          // 2+ float32 rows: batch-invariant with the one-token kernel
    }
    if (!ctx.force_plain && aligned) {
        // tokens go through in groups the activations' shared-memory area can hold
        uint32_t group = routed ? 1u : (c.count < 4u ? c.count : 4u);
        GemvPlan plan;
        const uint32_t gy = routed ? c.pairs : 1u;
        uint32_t max_ctas = (2u * ctx.sm_count + gy - 1) / gy;
        if (max_ctas < 1) max_ctas = 1;
        bool ok = false;
        uint32_t budget = GEMV_SMEM_BUDGET;
        for (; group >= 1; --group)
            if ((ok = plan_gemv(c.kind, c.cols, c.rows, c.stride, group, c.nmat, max_ctas, plan, budget))) break;
        if (!ok) {                                   // one CTA per SM with the whole shared memory
            budget = GEMV_SMEM_MAX;
            max_ctas = (ctx.sm_count + gy - 1) / gy;
            if (max_ctas < 1) max_ctas = 1;
            for (group = routed ? 1u : (c.count < 4u ? c.count : 4u); group >= 1; --group)
                if ((ok = plan_gemv(c.kind, c.cols, c.rows, c.stride, group, c.nmat, max_ctas, plan, budget))) break;
        }
        if (ok) {
            GemvArgs a = {};
            a.w[0] = c.w[0]; a.w[1] = c.w[1];
            a.ids = c.ids; a.expert = c.expert; a.n_experts = c.n_experts;
            a.per_pair = c.per_pair; a.top = c.top ? c.top : 1u; a.x_bf16 = c.x_bf16; a.glu = c.glu;
            a.status = ctx.status;
            if (routed) {
                a.plan = plan; a.x = c.x; a.y = c.y;
                return launch_stream(a, dim3(plan.ctas, c.pairs), ctx.stream, ctx.pdl);
            }
            const size_t xb = c.x_bf16 ? 2 : 4;
            for (uint32_t t0 = 0; t0 < c.count;) {
                uint32_t n = c.count - t0 < group ? c.count - t0 : group;
                if (n != plan.ntok && !plan_gemv(c.kind, c.cols, c.rows, c.stride, n, c.nmat, max_ctas, plan, budget))
                    return cudaErrorInvalidValue;
                a.plan = plan;
                a.x = static_cast<const uint8_t *>(c.x) + (size_t)t0 * c.cols * xb;
                a.y = c.y + (size_t)t0 * c.rows;
                cudaError_t e = launch_stream(a, dim3(plan.ctas, 1), ctx.stream, ctx.pdl);
                if (e != cudaSuccess) return e;
                t0 += n;
            }
            return cudaSuccess;
        }
    }
    PlainArgs a = {};
    a.w[0] = c.w[0]; a.w[1] = c.w[1]; a.x = c.x; a.y = c.y; a.ids = c.ids;
    a.cols = c.cols; a.rows = c.rows; a.stride = c.stride; a.kind = c.kind; a.expert = c.expert;
    a.n_experts = c.n_experts; a.per_pair = c.per_pair; a.top = c.top ? c.top : 1u; a.x_bf16 = c.x_bf16;
    a.nmat = c.nmat; a.glu = c.glu; a.count = c.count; a.status = ctx.status;
    return launch_plain(a, items, ctx.stream, ctx.pdl);
}

}  // namespace ingot
