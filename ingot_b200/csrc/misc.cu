// The bandwidth-trivial operators around the GEMVs: whole-matrix dequantise,
// top-k routing, weighted expert sum, GLU activation, shared-expert merge,
// residual RMS norm, expert grouping.  All HBM- or latency-bound; each is a
// straight grid of threads with coalesced 16-byte accesses.
#include "dev_common.cuh"
#include "gemv_core.cuh"
#include "kernels.h"
#include "pack.cuh"
#include "ptx.cuh"

namespace ingot {

namespace {

template <class K, class A>
cudaError_t launch(K kernel, dim3 grid, dim3 block, const LaunchCtx &ctx, const A &args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = ctx.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args);
}

__device__ __forceinline__ void pdl_prologue() {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
}

// N 32-bit words starting at a 2-byte aligned global address.
template <int N>
__device__ __forceinline__ void ld_words(const uint8_t *p, uint32_t *out) {
    const uintptr_t addr = reinterpret_cast<uintptr_t>(p);
    const uint32_t *ap = reinterpret_cast<const uint32_t *>(addr & ~uintptr_t(3));
    if (addr & 2u) {
        uint32_t prev = ap[0];
#pragma unroll
        for (int i = 0; i < N; ++i) {
            uint32_t next = ap[i + 1];
            out[i] = __funnelshift_r(prev, next, 16);
            prev = next;
        }
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) out[i] = ap[i];
    }
}

__device__ __forceinline__ float h16(const uint8_t *p) {
    return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(p)));
}

__device__ __forceinline__ void st4(float *out, float a, float b, float c, float d) {
    *reinterpret_cast<float4 *>(out) = make_float4(a, b, c, d);
}

}  // namespace

// ---------------------------------------------------------------------------
// Dequantise (reference read_rows: kernels/qwen.metal:35).  One thread per
// 32-weight unit; every value is formed with the same fp32 operations, in the
// same order, as weight_at, so results are bit-identical to it.
// ---------------------------------------------------------------------------

struct DequantArgs {
    const uint8_t *w;
    float *out;
    uint64_t rows;
    uint32_t cols, stride, kind;
};

__global__ void __launch_bounds__(256) dequant_units_kernel(const __grid_constant__ DequantArgs a) {
    pdl_prologue();
    const uint32_t upr = a.cols >> 5;                       // units per row
    const uint64_t total = a.rows * upr;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t row = idx / upr;
        const uint32_t u = (uint32_t)(idx - row * upr);
        const uint8_t *rp = a.w + row * a.stride;
        float *orow = a.out + row * a.cols;
        if (a.kind == KIND_Q4_K) {
            const uint8_t *b = rp + (size_t)(u >> 3) * 144u;
            const uint32_t p = u & 7u, j = p >> 1, h = p & 1u;
            uint32_t sc0, m0, sc1, m1, q[4];
            q4k_scale_min(b + 4, 2 * j, sc0, m0);
            q4k_scale_min(b + 4, 2 * j + 1, sc1, m1);
            ld_words<4>(b + 16u + 16u * p, q);
            const float d = h16(b), dmin = h16(b + 2);
            const float ds0 = __fmul_rn(d, (float)sc0), ds1 = __fmul_rn(d, (float)sc1);
            const float c0 = __fmul_rn(dmin, (float)m0), c1 = __fmul_rn(dmin, (float)m1);
            float *lo = orow + (u >> 3) * 256u + j * 64u + h * 16u, *hi = lo + 32;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t wl = q[i] & 0x0f0f0f0fu, wh = (q[i] >> 4) & 0x0f0f0f0fu;
                st4(lo + 4 * i, __fsub_rn(__fmul_rn(ds0, byte_f(wl, 0)), c0), __fsub_rn(__fmul_rn(ds0, byte_f(wl, 1)), c0),
                    __fsub_rn(__fmul_rn(ds0, byte_f(wl, 2)), c0), __fsub_rn(__fmul_rn(ds0, byte_f(wl, 3)), c0));
                st4(hi + 4 * i, __fsub_rn(__fmul_rn(ds1, byte_f(wh, 0)), c1), __fsub_rn(__fmul_rn(ds1, byte_f(wh, 1)), c1),
                    __fsub_rn(__fmul_rn(ds1, byte_f(wh, 2)), c1), __fsub_rn(__fmul_rn(ds1, byte_f(wh, 3)), c1));
            }
        } else if (a.kind == KIND_Q6_K) {
            const uint8_t *b = rp + (size_t)(u >> 3) * 210u;
            const uint32_t r = u & 7u, n = r >> 2, k8 = r & 3u;
            uint32_t l0[2], l1[2], hq[2];
            ld_words<2>(b + 64u * n + 8u * k8, l0);
            ld_words<2>(b + 64u * n + 32u + 8u * k8, l1);
            ld_words<2>(b + 128u + 32u * n + 8u * k8, hq);
            const float d = h16(b + 208);
            float *o = orow + (u >> 3) * 256u + n * 128u + k8 * 8u;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int scale = (int)(int8_t)b[192u + 8u * n + (k8 >> 1) + 2u * t];
                const float ds = __fmul_rn(d, (float)scale);
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const uint32_t lo = ((t & 1) ? l1[e] : l0[e]) >> ((t >= 2) ? 4 : 0);
                    const uint32_t qv = (lo & 0x0f0f0f0fu) | (((hq[e] >> (2 * t)) & 0x03030303u) << 4);
                    st4(o + 32 * t + 4 * e, __fmul_rn(ds, (float)((int)((qv >> 0) & 0xff) - 32)),
                        __fmul_rn(ds, (float)((int)((qv >> 8) & 0xff) - 32)),
                        __fmul_rn(ds, (float)((int)((qv >> 16) & 0xff) - 32)),
                        __fmul_rn(ds, (float)((int)((qv >> 24) & 0xff) - 32)));
                }
            }
        } else if (a.kind == KIND_Q4_0) {
            const uint8_t *b = rp + (size_t)u * 18u;
            uint32_t q[4];
            ld_words<4>(b + 2, q);
            const float d = h16(b);
            float *o = orow + u * 32u;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t wl = q[i] & 0x0f0f0f0fu, wh = (q[i] >> 4) & 0x0f0f0f0fu;
                st4(o + 4 * i, __fmul_rn(d, (float)((int)((wl >> 0) & 0xff) - 8)), __fmul_rn(d, (float)((int)((wl >> 8) & 0xff) - 8)),
                    __fmul_rn(d, (float)((int)((wl >> 16) & 0xff) - 8)), __fmul_rn(d, (float)((int)((wl >> 24) & 0xff) - 8)));
                st4(o + 16 + 4 * i, __fmul_rn(d, (float)((int)((wh >> 0) & 0xff) - 8)), __fmul_rn(d, (float)((int)((wh >> 8) & 0xff) - 8)),
                    __fmul_rn(d, (float)((int)((wh >> 16) & 0xff) - 8)), __fmul_rn(d, (float)((int)((wh >> 24) & 0xff) - 8)));
            }
        } else {   // Q8_0
            const uint8_t *b = rp + (size_t)u * 34u;
            uint32_t q[8];
            ld_words<8>(b + 2, q);
            const float d = h16(b);
            float *o = orow + u * 32u;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                st4(o + 4 * i, __fmul_rn(d, (float)(int)(int8_t)(q[i] & 0xff)), __fmul_rn(d, (float)(int)(int8_t)((q[i] >> 8) & 0xff)),
                    __fmul_rn(d, (float)(int)(int8_t)((q[i] >> 16) & 0xff)), __fmul_rn(d, (float)(int)(int8_t)(q[i] >> 24)));
        }
    }
}

// Any type, any alignment: one thread per element.
__global__ void __launch_bounds__(256) dequant_scalar_kernel(const __grid_constant__ DequantArgs a) {
    pdl_prologue();
    const uint64_t total = a.rows * a.cols;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t row = idx / a.cols;
        a.out[idx] = weight_at(a.w + row * a.stride, a.kind, (uint32_t)(idx - row * a.cols));
    }
}

cudaError_t launch_dequant(const uint8_t *w, uint32_t cols, uint64_t rows, uint32_t stride, uint32_t kind, float *out,
                           const LaunchCtx &ctx) {
    DequantArgs a = {w, out, rows, cols, stride, kind};
    const bool quant = kind == KIND_Q4_K || kind == KIND_Q6_K || kind == KIND_Q4_0 || kind == KIND_Q8_0;
    const bool aligned = ((uintptr_t)w % 4u) == 0 && (stride % 2u) == 0 && ((uintptr_t)out % 16u) == 0 && (cols % 32u) == 0;
    const uint64_t work = quant && aligned ? rows * (cols / 32u) : rows * cols;
    uint64_t blocks = (work + 255) / 256;
    const uint64_t cap = (uint64_t)ctx.sm_count * 32u;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) return cudaSuccess;
    if (quant && aligned) return launch(dequant_units_kernel, dim3((uint32_t)blocks), dim3(256), ctx, a);
    return launch(dequant_scalar_kernel, dim3((uint32_t)blocks), dim3(256), ctx, a);
}

// ---------------------------------------------------------------------------
// Routing (reference route_topk: kernels/generic.metal:479-494; CPU route():
// src/lib.rs:43-60).  One warp per token, up to 512 experts in registers.
// k rounds of arg-max, ties to the lowest expert id; weight exp(l - l_top),
// normalised by the sum taken in selection order.
// ---------------------------------------------------------------------------

struct RouteArgs {
    const float *logits;
    uint32_t *ids;
    float *weights;
    uint32_t experts, top, tokens;
    int *status;
};

__global__ void __launch_bounds__(128) route_topk_kernel(const __grid_constant__ RouteArgs a) {
    pdl_prologue();
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t t = blockIdx.x * 4u + (threadIdx.x >> 5);
    if (t >= a.tokens) return;
    const float *l = a.logits + (size_t)t * a.experts;
    float v[16];
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint32_t e = lane + 32u * i;
        v[i] = e < a.experts ? l[e] : -INFINITY;
        if (e < a.experts && !isfinite(v[i])) bad = true;
    }
    if (__any_sync(0xffffffffu, bad)) {
        if (lane == 0) atomicCAS(a.status, 0, KERNEL_ERR_ROUTER_INPUT);
        return;
    }
    float top_score = 0.f, sum = 0.f;
    for (uint32_t k = 0; k < a.top; ++k) {
        float best = -INFINITY;
        uint32_t index = 0xffffffffu;
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (v[i] > best) { best = v[i]; index = lane + 32u * i; }
        float score = best;
        for (uint32_t off = 16; off; off >>= 1) score = fmaxf(score, __shfl_xor_sync(0xffffffffu, score, off));
        uint32_t e = best == score ? index : 0xffffffffu;
        for (uint32_t off = 16; off; off >>= 1) e = min(e, __shfl_xor_sync(0xffffffffu, e, off));
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (lane + 32u * i == e) v[i] = -INFINITY;
        if (k == 0) top_score = score;
        const float w = expf(score - top_score);
        sum = __fadd_rn(sum, w);
        if (lane == 0) { a.ids[(size_t)t * a.top + k] = e; a.weights[(size_t)t * a.top + k] = w; }
    }
    __syncwarp();
    for (uint32_t k = lane; k < a.top; k += 32u) a.weights[(size_t)t * a.top + k] = __fdiv_rn(a.weights[(size_t)t * a.top + k], sum);
}

cudaError_t launch_route_topk(const float *logits, uint32_t experts, uint32_t top, uint32_t tokens, uint32_t *ids,
                              float *weights, const LaunchCtx &ctx) {
    if (tokens == 0) return cudaSuccess;
    RouteArgs a = {logits, ids, weights, experts, top, tokens, ctx.status};
    return launch(route_topk_kernel, dim3((tokens + 3) / 4), dim3(128), ctx, a);
}

// ---------------------------------------------------------------------------
// Weighted sum of each token's expert outputs in route order
// (reference moe_sum: kernels/generic.metal:17).
// ---------------------------------------------------------------------------

struct SumArgs {
    const float *routed, *w;
    const uint32_t *inverse;     // packed position of each pair, or null
    float *y;
    uint32_t width, top, tokens;
};

__global__ void __launch_bounds__(256) moe_sum_kernel(const __grid_constant__ SumArgs a) {
    pdl_prologue();
    const uint32_t w4 = a.width >> 2;
    const uint64_t total = (uint64_t)a.tokens * w4;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(idx / w4), j = (uint32_t)(idx - (uint64_t)t * w4);
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t e = 0; e < a.top; ++e) {
            const uint32_t pair = t * a.top + e;
            const size_t src = a.inverse ? a.inverse[pair] : pair;
            const float4 r = reinterpret_cast<const float4 *>(a.routed + src * a.width)[j];
            const float wt = a.w[pair];
            s.x = __fmaf_rn(r.x, wt, s.x); s.y = __fmaf_rn(r.y, wt, s.y);
            s.z = __fmaf_rn(r.z, wt, s.z); s.w = __fmaf_rn(r.w, wt, s.w);
        }
        reinterpret_cast<float4 *>(a.y + (size_t)t * a.width)[j] = s;
    }
}

static cudaError_t launch_sum(const SumArgs &a, const LaunchCtx &ctx) {
    const uint64_t total = (uint64_t)a.tokens * (a.width >> 2);
    if (total == 0) return cudaSuccess;
    uint64_t blocks = (total + 255) / 256, cap = (uint64_t)ctx.sm_count * 8u;
    if (blocks > cap) blocks = cap;
    return launch(moe_sum_kernel, dim3((uint32_t)blocks), dim3(256), ctx, a);
}

cudaError_t launch_moe_sum(const float *routed, const float *w, uint32_t width, uint32_t top, uint32_t tokens, float *y,
                           const LaunchCtx &ctx) {
    if (width % 4u) return cudaErrorInvalidValue;
    SumArgs a = {routed, w, nullptr, y, width, top, tokens};
    return launch_sum(a, ctx);
}

cudaError_t launch_combine_packed(const float *routed, const float *w, const uint32_t *inverse, uint32_t width,
                                  uint32_t top, uint32_t tokens, float *y, const LaunchCtx &ctx) {
    if (width % 4u) return cudaErrorInvalidValue;
    SumArgs a = {routed, w, inverse, y, width, top, tokens};
    return launch_sum(a, ctx);
}

// ---------------------------------------------------------------------------
// GLU activation (reference swiglu: kernels/moe.metal:405-410; gelu_mul:
// kernels/generic_arch.metal:7-10).
// ---------------------------------------------------------------------------

struct ActArgs {
    const float *gate, *up;
    float *y;
    uint64_t n;
    uint32_t gelu;
};

__global__ void __launch_bounds__(256) activation_kernel(const __grid_constant__ ActArgs a) {
    pdl_prologue();
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += (uint64_t)gridDim.x * blockDim.x)
        a.y[i] = glu_f(a.gate[i], a.up[i], a.gelu != 0);
}

cudaError_t launch_activation(const float *gate, const float *up, uint64_t n, uint32_t gelu, float *y,
                              const LaunchCtx &ctx) {
    if (n == 0) return cudaSuccess;
    ActArgs a = {gate, up, y, n, gelu};
    uint64_t blocks = (n + 255) / 256, cap = (uint64_t)ctx.sm_count * 8u;
    if (blocks > cap) blocks = cap;
    return launch(activation_kernel, dim3((uint32_t)blocks), dim3(256), ctx, a);
}

// ---------------------------------------------------------------------------
// Architecture glue of the generic path (kernels/generic_arch.metal:2-17): one element per thread.
//   scale    y = x * scale
//   softcap  y = c * tanh(x / c)                       (final logit soft-capping)
//   swiglu   y[t][j] = silu(x[t][j]) * x[t][ff + j]    (fused gate|up rows of width 2 ff)
//   columns  y[r][j] = x[r * stride + offset + j]      (columns [offset, offset + width) of rows)
// ---------------------------------------------------------------------------

struct GlueArgs {
    const float *x;
    float *y;
    uint64_t n;
    uint32_t op, width, offset, stride;
    float value;
};

__global__ void __launch_bounds__(256) glue_kernel(const __grid_constant__ GlueArgs a) {
    pdl_prologue();
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += (uint64_t)gridDim.x * blockDim.x) {
        switch (a.op) {
        case 0: a.y[i] = __fmul_rn(a.x[i], a.value); break;
        case 1: a.y[i] = __fmul_rn(a.value, tanhf(__fdiv_rn(a.x[i], a.value))); break;
        case 2: {
            const uint64_t t = i / a.width, j = i - t * a.width;
            const float g = a.x[t * 2u * a.width + j];
            a.y[i] = __fmul_rn(__fdiv_rn(g, 1.0f + expf(-g)), a.x[t * 2u * a.width + a.width + j]);
            break;
        }
        default: {
            const uint64_t r = i / a.width, j = i - r * a.width;
            a.y[i] = a.x[r * a.stride + a.offset + j];
        }
        }
    }
}

struct GatherArgs {
    const float *x;
    const uint32_t *pairs;       // packed position -> pair index
    float *y;
    uint32_t n, top, width;
};

// y[pos] = x[pairs[pos] / top]: the activation rows in the expert grouping's packed order (one warp per row).
__global__ void __launch_bounds__(256) gather_rows_kernel(const __grid_constant__ GatherArgs a) {
    pdl_prologue();
    const uint32_t lane = threadIdx.x & 31u, w4 = a.width >> 2;
    for (uint32_t pos = blockIdx.x * 8u + (threadIdx.x >> 5); pos < a.n; pos += gridDim.x * 8u) {
        const float4 *src = reinterpret_cast<const float4 *>(a.x + (size_t)(a.pairs[pos] / a.top) * a.width);
        float4 *dst = reinterpret_cast<float4 *>(a.y + (size_t)pos * a.width);
        for (uint32_t j = lane; j < w4; j += 32u) dst[j] = src[j];
    }
}

cudaError_t launch_gather_rows(const float *x, const uint32_t *pairs, uint32_t n, uint32_t top, uint32_t width, float *y, const LaunchCtx &ctx) {
    if (n == 0) return cudaSuccess;
    if (width % 4u || top == 0) return cudaErrorInvalidValue;
    GatherArgs a = {x, pairs, y, n, top, width};
    uint32_t blocks = (n + 7u) / 8u;
    if (blocks > ctx.sm_count * 8u) blocks = ctx.sm_count * 8u;
    return launch(gather_rows_kernel, dim3(blocks), dim3(256), ctx, a);
}

cudaError_t launch_glue(uint32_t op, const float *x, uint64_t n, uint32_t width, uint32_t offset, uint32_t stride, float value, float *y,
                        const LaunchCtx &ctx) {
    if (n == 0) return cudaSuccess;
    GlueArgs a = {x, y, n, op, width, offset, stride, value};
    uint64_t blocks = (n + 255) / 256, cap = (uint64_t)ctx.sm_count * 8u;
    if (blocks > cap) blocks = cap;
    return launch(glue_kernel, dim3((uint32_t)blocks), dim3(256), ctx, a);
}

// ---------------------------------------------------------------------------
// Routed sum plus sigmoid-gated shared expert, one token
// (reference combine: kernels/moe.metal:412-422).
// ---------------------------------------------------------------------------

struct MergeArgs {
    const float *routed, *shared, *weights, *shared_logit;
    float *y;
    uint32_t width, top;
};

__global__ void __launch_bounds__(256) merge_kernel(const __grid_constant__ MergeArgs a) {
    pdl_prologue();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.width) return;
    float s = 0.f;
    for (uint32_t e = 0; e < a.top; ++e) s = __fmaf_rn(a.routed[(size_t)e * a.width + i], a.weights[e], s);
    a.y[i] = s + a.shared[i] / (1.0f + expf(-a.shared_logit[0]));
}

cudaError_t launch_merge(const float *routed, const float *shared, const float *weights, const float *shared_logit,
                         uint32_t width, uint32_t top, float *y, const LaunchCtx &ctx) {
    if (width == 0) return cudaSuccess;
    MergeArgs a = {routed, shared, weights, shared_logit, y, width, top};
    return launch(merge_kernel, dim3((width + 255) / 256), dim3(256), ctx, a);
}

// ---------------------------------------------------------------------------
// Residual add + RMS norm per row (reference add_rms:
// kernels/generic.metal:390-404): s = a + b (when add), y = s * inv_rms * w.
// `w` may be null (unit weight); an optional bf16 copy of y feeds GEMVs that
// take bf16 activations.
// ---------------------------------------------------------------------------

struct RmsArgs {
    const float *a, *b, *w;
    float *s, *y;
    uint16_t *y_bf16;
    uint8_t *y_packed;          // rows of packed_x_bytes(width) for the tensor-core GEMV, or null
    uint32_t width, add, pack_bf16;
    float eps;
};

__device__ __forceinline__ uint16_t f2bf(float f) {
    uint32_t x = __float_as_uint(f);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40u);
    x += 0x7fffu + ((x >> 16) & 1u);
    return (uint16_t)(x >> 16);
}

__global__ void __launch_bounds__(256) add_rms_kernel(const __grid_constant__ RmsArgs a) {
    pdl_prologue();
    __shared__ float partial[8];
    const uint32_t row = blockIdx.x, tid = threadIdx.x, n4 = a.width >> 2;
    const size_t base = (size_t)row * n4;
    const float4 *a4 = reinterpret_cast<const float4 *>(a.a) + base;
    const float4 *b4 = a.add ? reinterpret_cast<const float4 *>(a.b) + base : nullptr;
    float sum = 0.f;
    for (uint32_t j = tid; j < n4; j += 256) {
        float4 v = a4[j];
        if (a.add) {
            const float4 o = b4[j];
            v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
            if (a.s) reinterpret_cast<float4 *>(a.s)[base + j] = v;
        }
        sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    for (uint32_t off = 16; off; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if ((tid & 31u) == 0) partial[tid >> 5] = sum;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) total += partial[i];
    const float inv = 1.0f / sqrtf(total / (float)a.width + a.eps);
    float mx = 0.f;
    for (uint32_t j = tid; j < n4; j += 256) {
        float4 v;
        if (a.add && a.s) v = reinterpret_cast<const float4 *>(a.s)[base + j];   // written above by this thread; s may alias a
        else {
            v = a4[j];
            if (a.add) { const float4 o = b4[j]; v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
        }
        float4 wv = a.w ? reinterpret_cast<const float4 *>(a.w)[j] : make_float4(1.f, 1.f, 1.f, 1.f);
        v.x = v.x * inv * wv.x; v.y = v.y * inv * wv.y; v.z = v.z * inv * wv.z; v.w = v.w * inv * wv.w;
        if (a.y) reinterpret_cast<float4 *>(a.y)[base + j] = v;
        if (a.y_bf16) {
            uint2 o;
            o.x = (uint32_t)f2bf(v.x) | ((uint32_t)f2bf(v.y) << 16);
            o.y = (uint32_t)f2bf(v.z) | ((uint32_t)f2bf(v.w) << 16);
            reinterpret_cast<uint2 *>(a.y_bf16)[base + j] = o;
        }
        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    if (!a.y_packed) return;
    // the same activations in the tensor-core GEMV's operand order (what ingot_pack_x
    // would produce from y, or from its bf16 rounding when pack_bf16 is set)
    __syncthreads();
    for (uint32_t off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if ((tid & 31u) == 0) partial[tid >> 5] = mx;
    __syncthreads();
    mx = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) mx = fmaxf(mx, partial[i]);
    const float scale = pack_scale(mx);
    const bool hi = a.pack_bf16 == 3u;
    uint8_t *prow = a.y_packed + (size_t)row * (hi ? packed_hi_bytes(a.width) : packed_x_bytes(a.width));
    for (uint32_t j0 = 0; j0 < n4; j0 += 256) {
        const uint32_t j = j0 + tid;
        const bool live = j < n4;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (live) {
            float4 u;
            if (a.add && a.s) u = reinterpret_cast<const float4 *>(a.s)[base + j];
            else {
                u = a4[j];
                if (a.add) { const float4 o = b4[j]; u.x += o.x; u.y += o.y; u.z += o.z; u.w += o.w; }
            }
            float4 wv = a.w ? reinterpret_cast<const float4 *>(a.w)[j] : make_float4(1.f, 1.f, 1.f, 1.f);
            v[0] = u.x * inv * wv.x; v[1] = u.y * inv * wv.y; v[2] = u.z * inv * wv.z; v[3] = u.w * inv * wv.w;
            if (a.pack_bf16) {
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = __uint_as_float((uint32_t)f2bf(v[i]) << 16);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] *= scale;
        }
        if (hi) pack_hi_store_quad(prow, a.width, j, v, live);
        else pack_store_quad(prow, a.width, j, v, live);
    }
    if (tid == 0) { if (hi) pack_hi_store_unscale(prow, a.width, scale); else pack_store_unscale(prow, a.width, scale); }
}

// The same with every element held in registers between the passes: one read of the inputs,
// two block-wide reductions (sum of squares; largest magnitude for the packing scale).  A
// decode step runs four of these per layer on a single CTA each, so their latency, not their
// bandwidth, is what counts.  Rows of up to RMS_FAST_THREADS * 4 * RMS_FAST_VEC elements.
static constexpr uint32_t RMS_FAST_THREADS = 512, RMS_FAST_VEC = 8;

__device__ __forceinline__ float block_reduce_512(float v, float *partial, bool is_max) {
    for (uint32_t off = 16; off; off >>= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, v, off);
        v = is_max ? fmaxf(v, o) : v + o;
    }
    __syncthreads();                                   // partial[] may still be read from the previous reduction
    if ((threadIdx.x & 31u) == 0) partial[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = partial[0];
#pragma unroll
    for (int i = 1; i < (int)(RMS_FAST_THREADS / 32u); ++i) r = is_max ? fmaxf(r, partial[i]) : r + partial[i];
    return r;
}

__global__ void __launch_bounds__(RMS_FAST_THREADS) add_rms_fast_kernel(const __grid_constant__ RmsArgs a) {
    pdl_prologue();
    __shared__ float partial[RMS_FAST_THREADS / 32u];
    const uint32_t row = blockIdx.x, tid = threadIdx.x, n4 = a.width >> 2;
    const size_t base = (size_t)row * n4;
    const float4 *a4 = reinterpret_cast<const float4 *>(a.a) + base;
    const float4 *b4 = a.add ? reinterpret_cast<const float4 *>(a.b) + base : nullptr;
    float4 v[RMS_FAST_VEC];
    float sum = 0.f;
#pragma unroll
    for (uint32_t i = 0; i < RMS_FAST_VEC; ++i) {
        const uint32_t j = tid + i * RMS_FAST_THREADS;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < n4) {
            v[i] = a4[j];
            if (a.add) {
                const float4 o = b4[j];
                v[i].x += o.x; v[i].y += o.y; v[i].z += o.z; v[i].w += o.w;
                if (a.s) reinterpret_cast<float4 *>(a.s)[base + j] = v[i];
            }
            sum += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    }
    const float total = block_reduce_512(sum, partial, false);
    const float inv = 1.0f / sqrtf(total / (float)a.width + a.eps);
    float mx = 0.f;
#pragma unroll
    for (uint32_t i = 0; i < RMS_FAST_VEC; ++i) {
        const uint32_t j = tid + i * RMS_FAST_THREADS;
        if (j < n4) {
            const float4 wv = a.w ? reinterpret_cast<const float4 *>(a.w)[j] : make_float4(1.f, 1.f, 1.f, 1.f);
            v[i].x = v[i].x * inv * wv.x; v[i].y = v[i].y * inv * wv.y; v[i].z = v[i].z * inv * wv.z; v[i].w = v[i].w * inv * wv.w;
            if (a.y) reinterpret_cast<float4 *>(a.y)[base + j] = v[i];
            if (a.y_bf16) {
                uint2 o;
                o.x = (uint32_t)f2bf(v[i].x) | ((uint32_t)f2bf(v[i].y) << 16);
                o.y = (uint32_t)f2bf(v[i].z) | ((uint32_t)f2bf(v[i].w) << 16);
                reinterpret_cast<uint2 *>(a.y_bf16)[base + j] = o;
            }
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
        }
    }
    if (!a.y_packed) return;
    mx = block_reduce_512(mx, partial, true);
    const float scale = pack_scale(mx);
    const bool hi = a.pack_bf16 == 3u;
    uint8_t *prow = a.y_packed + (size_t)row * (hi ? packed_hi_bytes(a.width) : packed_x_bytes(a.width));
#pragma unroll
    for (uint32_t i = 0; i < RMS_FAST_VEC; ++i) {
        const uint32_t j = tid + i * RMS_FAST_THREADS;
        if (i * RMS_FAST_THREADS >= n4) break;             // uniform over the block: the quad shuffles keep all lanes
        const bool live = j < n4;
        float u[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
        if (a.pack_bf16) {
#pragma unroll
            for (int k = 0; k < 4; ++k) u[k] = __uint_as_float((uint32_t)f2bf(u[k]) << 16);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) u[k] *= scale;
        if (hi) pack_hi_store_quad(prow, a.width, j, u, live);
        else pack_store_quad(prow, a.width, j, u, live);
    }
    if (tid == 0) { if (hi) pack_hi_store_unscale(prow, a.width, scale); else pack_store_unscale(prow, a.width, scale); }
}

cudaError_t launch_add_rms(const float *a, const float *b, const float *w, float *s, float *y, uint32_t width,
                           uint32_t rows, float eps, uint32_t add, void *y_bf16, void *y_packed, uint32_t pack_bf16,
                           const LaunchCtx &ctx) {
    if (width % 4u || (y_packed && width % 64u)) return cudaErrorInvalidValue;
    if (rows == 0) return cudaSuccess;
    RmsArgs args = {a, b, w, s, y, static_cast<uint16_t *>(y_bf16), static_cast<uint8_t *>(y_packed), width, add, pack_bf16, eps};
    if (width <= RMS_FAST_THREADS * 4u * RMS_FAST_VEC) return launch(add_rms_fast_kernel, dim3(rows), dim3(RMS_FAST_THREADS), ctx, args);
    return launch(add_rms_kernel, dim3(rows), dim3(256), ctx, args);
}

struct CvtArgs {
    const float *x;
    uint16_t *y;
    uint64_t n;
};

__global__ void __launch_bounds__(256) convert_bf16_kernel(const __grid_constant__ CvtArgs a) {
    pdl_prologue();
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += (uint64_t)gridDim.x * blockDim.x)
        a.y[i] = f2bf(a.x[i]);
}

cudaError_t launch_convert_bf16(const float *x, uint64_t n, void *y_bf16, const LaunchCtx &ctx) {
    if (n == 0) return cudaSuccess;
    CvtArgs a = {x, static_cast<uint16_t *>(y_bf16), n};
    uint64_t blocks = (n + 255) / 256, cap = (uint64_t)ctx.sm_count * 8u;
    if (blocks > cap) blocks = cap;
    return launch(convert_bf16_kernel, dim3((uint32_t)blocks), dim3(256), ctx, a);
}

__global__ void increment_kernel(uint32_t *counter) {
    pdl_prologue();
    *counter += 1u;
}

struct CollectArgs {
    const uint64_t *tagged;
    float *plain;
    uint32_t n;
    const uint32_t *step;
    uint32_t tag_mul, tag_add;
    int *status;
};

// Copies a vector out of its tagged twin once every word carries this step's tag (bounded wait): after it the plain
// vector holds the rows of every rank.
__global__ void __launch_bounds__(256) collect_tagged_kernel(const __grid_constant__ CollectArgs a) {
    pdl_prologue();
    const uint32_t tag = *reinterpret_cast<const volatile uint32_t *>(a.step) * a.tag_mul + a.tag_add;
    if (a.status && *reinterpret_cast<const volatile int *>(a.status) != 0) return;      // a wait already ran out in this step
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += gridDim.x * blockDim.x) {
        uint64_t t0 = 0;
        for (;;) {
            bool done = false;
            for (int k = 0; k < 256 && !done; ++k) {
                uint64_t w;
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(a.tagged + i) : "memory");
                if ((uint32_t)(w >> 32) == tag) { a.plain[i] = __uint_as_float((uint32_t)w); done = true; }
            }
            if (done) break;
            const uint64_t now = ptx::global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > ptx::WAIT_LIMIT_NS) { set_status_word(a.status, KERNEL_ERR_PEER_TIMEOUT); return; }
        }
    }
}

cudaError_t launch_collect_tagged(const uint64_t *tagged, float *plain, uint32_t n, const uint32_t *step, uint32_t tag_mul, uint32_t tag_add,
                                  const LaunchCtx &ctx) {
    CollectArgs a = {tagged, plain, n, step, tag_mul, tag_add, ctx.status};
    uint32_t blocks = (n + 255u) / 256u;
    if (blocks > ctx.sm_count * 2u) blocks = ctx.sm_count * 2u;
    return launch(collect_tagged_kernel, dim3(blocks ? blocks : 1u), dim3(256), ctx, a);
}

cudaError_t launch_increment(uint32_t *counter, const LaunchCtx &ctx) {
    return launch(increment_kernel, dim3(1), dim3(1), ctx, counter);
}

// ---------------------------------------------------------------------------
// Expert-parallel sharding: keep the pairs whose expert lies in [first, first + count)
// (ids become local), mark the others ROUTE_SKIP with weight 0.  The routed GEMVs
// write zero rows for skipped pairs, so the weighted sum is this device's partial
// result and an all-reduce over the devices gives the full one.
// ---------------------------------------------------------------------------

struct LocalizeArgs {
    const uint32_t *ids;
    const float *w;
    uint32_t *ids_out;
    float *w_out;
    uint32_t pairs, first, count;
};

__global__ void __launch_bounds__(256) ep_localize_kernel(const __grid_constant__ LocalizeArgs a) {
    pdl_prologue();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.pairs) return;
    const uint32_t e = a.ids[i];
    const bool mine = e >= a.first && e - a.first < a.count;
    a.ids_out[i] = mine ? e - a.first : ROUTE_SKIP;
    a.w_out[i] = mine ? a.w[i] : 0.f;
}

cudaError_t launch_ep_localize(const uint32_t *ids, const float *w, uint32_t pairs, uint32_t first, uint32_t count,
                               uint32_t *ids_out, float *w_out, const LaunchCtx &ctx) {
    if (pairs == 0) return cudaSuccess;
    LocalizeArgs a = {ids, w, ids_out, w_out, pairs, first, count};
    return launch(ep_localize_kernel, dim3((pairs + 255) / 256), dim3(256), ctx, a);
}

// ---------------------------------------------------------------------------
// Expert grouping for the packed MoE path.  The tables are the reference's (expert_layout /
// expert_pairs: kernels/prefill.metal:7-35): experts ascending, pair indices ascending inside an
// expert, tiles of at most 32 pairs, mode 1 for tiles of two or more.  They are built by ONE
// CTA in one launch: a shared-memory histogram, a block-wide exclusive scan over the experts
// (warp shuffles, then the warp totals), and a stable placement of the pairs in which the
// sixteen warps take turns in pair order — inside a warp, match_any gives every lane its rank
// among the earlier lanes with the same expert, and the group's first lane advances that
// expert's running position.
// ---------------------------------------------------------------------------

struct LayoutArgs {
    const uint32_t *ids;
    uint32_t *layout, *tiles, *pairs, *inverse;
    uint32_t n_pairs, experts, tile_capacity;
    int *status;
};

static constexpr uint32_t GROUP_THREADS = 512;      // one expert per thread in the scan: at most 512 experts

__global__ void __launch_bounds__(GROUP_THREADS) expert_group_kernel(const __grid_constant__ LayoutArgs a) {
    pdl_prologue();
    __shared__ uint32_t counts[GROUP_THREADS], next_pos[GROUP_THREADS], warp_pairs[GROUP_THREADS / 32], warp_tiles[GROUP_THREADS / 32];
    __shared__ uint32_t total_tiles;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    counts[tid] = 0;
    __syncthreads();
    for (uint32_t i = tid; i < a.n_pairs; i += GROUP_THREADS) {
        const uint32_t e = a.ids[i];
        if (e < a.experts) atomicAdd(&counts[e], 1u);
        else if (e != ROUTE_SKIP) atomicCAS(a.status, 0, KERNEL_ERR_EXPERT_RANGE);       // (a skipped pair takes no place)
    }
    __syncthreads();
    // exclusive scan over the experts of (pairs, tiles): inclusive inside the warp, then the warps' totals
    const uint32_t n = tid < a.experts ? counts[tid] : 0u, nt = (n + 31u) / 32u;
    uint32_t sp = n, st = nt;
    for (uint32_t off = 1; off < 32; off <<= 1) {
        const uint32_t op = __shfl_up_sync(0xffffffffu, sp, off), ot = __shfl_up_sync(0xffffffffu, st, off);
        if (lane >= off) { sp += op; st += ot; }
    }
    if (lane == 31) { warp_pairs[warp] = sp; warp_tiles[warp] = st; }
    __syncthreads();
    uint32_t base_p = 0, base_t = 0;
    for (uint32_t w = 0; w < warp; ++w) { base_p += warp_pairs[w]; base_t += warp_tiles[w]; }
    const uint32_t first = base_p + sp - n, tile0 = base_t + st - nt;
    if (tid == GROUP_THREADS - 1) total_tiles = base_t + st;
    next_pos[tid] = first;
    if (tid < a.experts) {
        a.layout[2 * tid] = n;
        a.layout[2 * tid + 1] = first;
        for (uint32_t k = 0; k < nt; ++k) {
            const uint32_t t = tile0 + k;
            if (t >= a.tile_capacity) { atomicCAS(a.status, 0, KERNEL_ERR_EXPERT_RANGE); break; }
            const uint32_t m = n - 32u * k < 32u ? n - 32u * k : 32u;
            a.tiles[4 * t] = tid; a.tiles[4 * t + 1] = first + 32u * k; a.tiles[4 * t + 2] = m; a.tiles[4 * t + 3] = m >= 2u ? 1u : 0u;
        }
    }
    __syncthreads();
    for (uint32_t t = total_tiles + tid; t < a.tile_capacity; t += GROUP_THREADS)
        a.tiles[4 * t] = a.tiles[4 * t + 1] = a.tiles[4 * t + 2] = a.tiles[4 * t + 3] = 0;
    // stable placement: chunks of 512 pairs in order, the warps of a chunk one after the other
    for (uint32_t i0 = 0; i0 < a.n_pairs; i0 += GROUP_THREADS) {
        const uint32_t i = i0 + tid;
        const uint32_t e = i < a.n_pairs ? a.ids[i] : 0xffffffffu;
        const bool live = e < a.experts;
        if (i < a.n_pairs && !live) a.inverse[i] = ROUTE_SKIP;
        const uint32_t same = __match_any_sync(0xffffffffu, e);
        const uint32_t rank = __popc(same & ((1u << lane) - 1u));
        for (uint32_t w = 0; w < GROUP_THREADS / 32; ++w) {
            if (warp == w && live) {
                const uint32_t at = next_pos[e] + rank;
                a.inverse[i] = at;
                a.pairs[at] = i;
            }
            __syncwarp();
            if (warp == w && live && rank == 0) next_pos[e] += __popc(same);
            __syncthreads();
        }
    }
}

cudaError_t launch_expert_layout(const uint32_t *ids, uint32_t n_pairs, uint32_t experts, uint32_t tile_capacity,
                                 uint32_t *layout, uint32_t *tiles, uint32_t *pairs, uint32_t *inverse,
                                 const LaunchCtx &ctx) {
    if (experts == 0 || experts > GROUP_THREADS) return cudaErrorInvalidValue;
    LayoutArgs a = {ids, layout, tiles, pairs, inverse, n_pairs, experts, tile_capacity, ctx.status};
    return launch(expert_group_kernel, dim3(1), dim3(GROUP_THREADS), ctx, a);
}

}  // namespace ingot
