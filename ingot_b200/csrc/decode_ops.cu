// The rest of a generic decode step around the projections: token embedding rows,
// rotary position embedding with the KV-cache write, causal attention for one to four
// query tokens over a float32 cache, and the greedy token choice.
//
// Reference: embedding_batch (kernels/qwen.metal:139), qk_rope_cache
// (kernels/generic.metal:405-438), attention_decode_<D> (kernels/generic.metal:440-474),
// greedy_select (kernels/qwen.metal:384-410) driven by Gpu::finish_greedy
// (src/metal.rs:1507-1548); the graph that uses them is Generic::hidden
// (src/generic.rs:664-749).  All four are latency- or cache-bandwidth-trivial next to the
// GEMVs; they exist so that a token step is a whole model step.
#include <math.h>

#include "dev_common.cuh"
#include "kernels.h"
#include "ptx.cuh"
#include "quant.cuh"

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

__device__ __forceinline__ float warp_sum(float v) {
    for (uint32_t off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// ---- embedding rows ----------------------------------------------------------------

struct EmbedArgs {
    const uint8_t *w;
    const uint32_t *ids;
    float *y;
    uint32_t width, stride, kind, count, vocab;
    int *status;
};

// y[t][j] = weight_at(row ids[t], j): the scalar decoder, so the rows are bit-exact.
__global__ void __launch_bounds__(256) embedding_kernel(const __grid_constant__ EmbedArgs a) {
    pdl_prologue();
    const uint64_t n = (uint64_t)a.width * a.count;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(i / a.width), j = (uint32_t)(i % a.width);
        const uint32_t id = a.ids[t];
        if (id >= a.vocab) {                          // a token outside the vocabulary is an error code, not a fault
            if (j == 0) set_status_word(a.status, KERNEL_ERR_EXPERT_RANGE);
            a.y[i] = 0.f;
            continue;
        }
        a.y[i] = weight_at(a.w + (size_t)id * a.stride, a.kind, j);
    }
}

// ---- rotary embedding + cache write ---------------------------------------------------

struct RopeArgs {
    const float *q, *k, *v, *qn, *kn, *factors;
    float *qo, *kc, *vc;
    RopeParams p;
};

// One warp per head row of one token: rows of q, then k, then v.
__global__ void __launch_bounds__(32) rope_cache_kernel(const __grid_constant__ RopeArgs a) {
    pdl_prologue();
    __shared__ float row[512];
    const RopeParams &p = a.p;
    const uint32_t D = p.head_dim, H = p.heads, KV = p.kv_heads, r = blockIdx.x, t = blockIdx.y, rot = p.rotated, lane = threadIdx.x;
    if (r >= H + KV) {
        const uint32_t h = r - H - KV;
        const float *src = a.v + ((size_t)t * KV + h) * D;
        float *dst = a.vc + ((size_t)(p.position + t) * KV + h) * D;
        float inv = 1.f;
        if (p.value_norm) {
            float s = 0.f;
            for (uint32_t j = lane; j < D; j += 32) { const float x = src[j]; s += x * x; }
            inv = rsqrtf(warp_sum(s) / (float)D + p.eps);
        }
        for (uint32_t j = lane; j < D; j += 32) dst[j] = p.value_norm ? src[j] * inv : src[j];
        return;
    }
    const bool isq = r < H;
    const uint32_t h = isq ? r : r - H;
    const float *src = isq ? a.q + ((size_t)t * H + h) * D : a.k + ((size_t)t * KV + h) * D;
    float *dst = isq ? a.qo + ((size_t)t * H + h) * D : a.kc + ((size_t)(p.position + t) * KV + h) * D;
    const float *w = isq ? a.qn : a.kn;
    float inv = 1.f;
    if (p.qk_norm) {
        float s = 0.f;
        for (uint32_t j = lane; j < D; j += 32) { const float x = src[j]; s += x * x; }
        inv = rsqrtf(warp_sum(s) / (float)D + p.eps);
    }
    for (uint32_t j = lane; j < D; j += 32) row[j] = p.qk_norm ? src[j] * inv * w[j] : src[j];
    __syncwarp();
    const float qs = isq ? p.q_scale : 1.0f;
    for (uint32_t j = lane; j < D; j += 32) {
        if (j >= rot) { dst[j] = row[j] * qs; continue; }
        const uint32_t f = p.neox ? j % (rot / 2) : j / 2;
        const uint32_t ia = p.neox ? f : (j & ~1u), ib = p.neox ? ia + rot / 2 : ia + 1;
        float theta = (float)(p.position + t) * powf(p.base, -2.0f * (float)f / (float)rot);
        if (p.use_factors) theta /= a.factors[f];
        const float c = cosf(theta), s = sinf(theta);
        const bool first = p.neox ? j < rot / 2 : (j & 1u) == 0;
        const float y = first ? row[ia] * c - row[ib] * s : row[ia] * s + row[ib] * c;
        dst[j] = y * qs;
    }
}

// ---- causal attention for one to four query tokens ---------------------------------------

struct AttnArgs {
    const float *q, *k, *v;
    float *out;
    uint32_t heads, kv_heads, position, window;
};

// One CTA per (head, token); its eight warps take every eighth key with an online softmax, then
// warp 0 merges the eight partial results.
template <uint32_t D>
__global__ void __launch_bounds__(256) attention_decode_kernel(const __grid_constant__ AttnArgs a) {
    pdl_prologue();
    constexpr uint32_t J = D / 32;
    __shared__ float part[8 * D + 16];
    const uint32_t h = blockIdx.x, t = blockIdx.y, lane = threadIdx.x & 31u, sg = threadIdx.x >> 5;
    const uint32_t kh = h / (a.heads / a.kv_heads), stride = a.kv_heads * D, length = a.position + t + 1;
    const uint32_t start = a.window && length > a.window ? length - a.window : 0;
    const float scale = rsqrtf((float)D);
    float qv[J], o[J];
#pragma unroll
    for (uint32_t j = 0; j < J; ++j) { qv[j] = a.q[((size_t)t * a.heads + h) * D + lane + 32 * j]; o[j] = 0.f; }
    float m = -INFINITY, l = 0.f;
    for (uint32_t pos = start + sg; pos < length; pos += 8) {
        const float *kr = a.k + (size_t)pos * stride + kh * D, *vr = a.v + (size_t)pos * stride + kh * D;
        float s = 0.f;
#pragma unroll
        for (uint32_t j = 0; j < J; ++j) s += qv[j] * kr[lane + 32 * j];
        s = warp_sum(s) * scale;
        const float next = fmaxf(m, s), f = expf(m - next), e = expf(s - next);
        l = l * f + e;
        m = next;
#pragma unroll
        for (uint32_t j = 0; j < J; ++j) o[j] = o[j] * f + e * vr[lane + 32 * j];
    }
    float *ms = part + 8 * D, *ls = ms + 8;
    if (!lane) { ms[sg] = m; ls[sg] = l; }
#pragma unroll
    for (uint32_t j = 0; j < J; ++j) part[sg * D + lane + 32 * j] = o[j];
    __syncthreads();
    if (sg) return;
    float M = -INFINITY;
    for (uint32_t i = 0; i < 8; ++i) M = fmaxf(M, ms[i]);
    float L = 0.f, w[8];
    for (uint32_t i = 0; i < 8; ++i) { w[i] = expf(ms[i] - M); L += ls[i] * w[i]; }
#pragma unroll
    for (uint32_t j = 0; j < J; ++j) {
        float acc = 0.f;
        for (uint32_t i = 0; i < 8; ++i) acc += part[i * D + lane + 32 * j] * w[i];
        a.out[((size_t)t * a.heads + h) * D + lane + 32 * j] = acc / L;
    }
}

// ---- greedy choice -------------------------------------------------------------------

struct GreedyArgs {
    const float *logits;
    const uint32_t *mapping;
    uint32_t *partial, *out;
    uint32_t vocab, chunks, stage, mapped;
};

// Stage 0: one warp per 1024 logits of a row -> (max bits, token, non-finite seen).  Stage 1: one warp per
// row over its chunks.  Equal values (signed zeros included) go to the smaller token id.
__global__ void __launch_bounds__(32) greedy_kernel(const __grid_constant__ GreedyArgs a) {
    pdl_prologue();
    const uint32_t lane = threadIdx.x, gx = blockIdx.x, gy = blockIdx.y;
    float best = -INFINITY;
    uint32_t id = 0xffffffffu, bad = 0;
    const uint32_t end = a.stage ? a.chunks : min(a.vocab, (gx + 1) * 1024u), start = a.stage ? 0u : gx * 1024u;
    for (uint32_t i = start + lane; i < end; i += 32) {
        const size_t off = ((size_t)gy * a.chunks + i) * 3;
        const float value = a.stage ? __uint_as_float(a.partial[off]) : a.logits[(size_t)gy * a.vocab + i];
        const uint32_t token = a.stage ? a.partial[off + 1] : (a.mapped ? a.mapping[i] : i);
        bad |= a.stage ? a.partial[off + 2] : (uint32_t)!isfinite(value);
        if (value > best || (value == best && token < id)) { best = value; id = token; }
    }
    float maximum = best;
    for (uint32_t o = 16; o; o >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, o));
    uint32_t winner = best == maximum ? id : 0xffffffffu;
    for (uint32_t o = 16; o; o >>= 1) winner = min(winner, __shfl_xor_sync(0xffffffffu, winner, o));
    for (uint32_t o = 16; o; o >>= 1) bad |= __shfl_xor_sync(0xffffffffu, bad, o);
    if (lane == 0) {
        if (a.stage) { a.out[gy * 2] = winner; a.out[gy * 2 + 1] = bad; }
        else {
            const size_t off = ((size_t)gy * a.chunks + gx) * 3;
            a.partial[off] = __float_as_uint(maximum); a.partial[off + 1] = winner; a.partial[off + 2] = bad;
        }
    }
}

}  // namespace

cudaError_t launch_embedding(const uint8_t *w, const uint32_t *ids, uint32_t width, uint32_t stride, uint32_t kind, uint32_t count,
                             uint32_t vocab, float *y, const LaunchCtx &ctx) {
    if (count == 0) return cudaSuccess;
    EmbedArgs a = {w, ids, y, width, stride, kind, count, vocab, ctx.status};
    uint64_t blocks = ((uint64_t)width * count + 255) / 256, cap = (uint64_t)ctx.sm_count * 8u;
    if (blocks > cap) blocks = cap;
    return launch(embedding_kernel, dim3((uint32_t)blocks), dim3(256), ctx, a);
}

cudaError_t launch_rope_cache(const float *q, const float *k, const float *v, const float *qn, const float *kn, const float *factors,
                              float *qo, float *kc, float *vc, const RopeParams &p, uint32_t tokens, const LaunchCtx &ctx) {
    if (tokens == 0) return cudaSuccess;
    RopeArgs a = {q, k, v, qn, kn, factors, qo, kc, vc, p};
    return launch(rope_cache_kernel, dim3(p.heads + 2u * p.kv_heads, tokens), dim3(32), ctx, a);
}

cudaError_t launch_attention_decode(const float *q, const float *k, const float *v, float *out, uint32_t head_dim, uint32_t heads,
                                    uint32_t kv_heads, uint32_t position, uint32_t window, uint32_t tokens, const LaunchCtx &ctx) {
    if (tokens == 0) return cudaSuccess;
    AttnArgs a = {q, k, v, out, heads, kv_heads, position, window};
    const dim3 grid(heads, tokens), block(256);
    switch (head_dim) {
    case 64: return launch(attention_decode_kernel<64>, grid, block, ctx, a);
    case 96: return launch(attention_decode_kernel<96>, grid, block, ctx, a);
    case 128: return launch(attention_decode_kernel<128>, grid, block, ctx, a);
    case 256: return launch(attention_decode_kernel<256>, grid, block, ctx, a);
    case 512: return launch(attention_decode_kernel<512>, grid, block, ctx, a);
    default: return cudaErrorNotSupported;
    }
}

cudaError_t launch_greedy(const float *logits, const uint32_t *mapping, uint32_t rows, uint32_t vocab, uint32_t *partial, uint32_t *out,
                          const LaunchCtx &ctx) {
    if (rows == 0) return cudaSuccess;
    const uint32_t chunks = (vocab + 1023u) / 1024u;
    GreedyArgs a = {logits, mapping, partial, out, vocab, chunks, 0u, mapping ? 1u : 0u};
    cudaError_t e = launch(greedy_kernel, dim3(chunks, rows), dim3(32), ctx, a);
    if (e != cudaSuccess) return e;
    a.stage = 1u;
    return launch(greedy_kernel, dim3(1, rows), dim3(32), ctx, a);
}

}  // namespace ingot
