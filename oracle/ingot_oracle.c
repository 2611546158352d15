/*
 * CPU oracle for the ingot decode hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic that the reference's Metal
 * shaders define for GGUF block-quantised weights and the operators built on
 * them.  It is the checker the CUDA kernels are compared against and the
 * timed "CPU baseline"; nothing in the product library links or calls it.
 *
 * Parity pins (what this restatement has been checked against):
 *   - the reference's own shader source for weight_at / mix_weight_at /
 *     kquant_scale_min, compiled as C++ through a shim (oracle/build_ref.sh),
 *     bit-exact on random blocks for kinds 0,1,2,8,12,14,30;
 *   - the closed-form fixtures of the reference's tests
 *     (src/metal/tests.rs:13-137, src/main.rs:341-349);
 *   - the gguf-py 0.19 NumPy dequantiser (tests/golden/make_golden.py),
 *     bit-exact for Q4_0, Q8_0, Q4_K, Q6_K.
 *
 * Every function cites the reference file:line it follows.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

/* ---- scalar conversions ------------------------------------------------ */

/* IEEE binary16 -> binary32, exact.  kernels/moe.metal:6-9 (half_at),
 * kernels/iq3_mix.metal:6 (mix_half). */
ORACLE_API float oracle_half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* binary32 -> binary16, round to nearest even (the conversion `half(x)` does
 * when the prefill GEMM stages operands: kernels/generic.metal:343,355-361;
 * src/expert_bench.rs:639-646 to_half). */
ORACLE_API uint16_t oracle_float_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t abs = x & 0x7fffffffu;
    if (abs >= 0x7f800000u) /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((abs > 0x7f800000u) ? 0x200u : 0));
    if (abs >= 0x477ff000u) /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    if (abs < 0x33000001u) /* < 2^-25 (or == 2^-25, ties to even 0) */
        return (uint16_t)sign;
    int32_t e = (int32_t)(abs >> 23) - 127;
    uint32_t m = (abs & 0x7fffffu) | 0x800000u;
    uint32_t shift, half_bits;
    if (e < -14) { /* subnormal half */
        shift = (uint32_t)(13 + (-14 - e));
        half_bits = 0;
    } else {
        shift = 13;
        half_bits = (uint32_t)(e + 15) << 10;
        m &= 0x7fffffu;
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
    return (uint16_t)(sign | (half_bits + q)); /* carry into exponent is correct */
}

/* bf16 bits -> f32: kernels/moe.metal:47-50 (type 30). */
ORACLE_API float oracle_bf16_to_float(uint16_t b) {
    uint32_t bits = (uint32_t)b << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* f32 -> bf16 bits, round to nearest even (how bf16 activations are produced
 * for the bf16-activation configurations). */
ORACLE_API uint16_t oracle_float_to_bf16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40u);
    x += 0x7fffu + ((x >> 16) & 1u);
    return (uint16_t)(x >> 16);
}

/* ---- block geometry ---------------------------------------------------- */

/* (elements per block, bytes per block) by GGML type id: src/gguf.rs:470-491,
 * restricted to the formats this path covers. Returns 0 on success. */
ORACLE_API int oracle_geometry(uint32_t kind, uint32_t *block, uint32_t *bytes) {
    switch (kind) {
    case 0: *block = 1; *bytes = 4; return 0;    /* F32  */
    case 1: case 30: *block = 1; *bytes = 2; return 0; /* F16 / BF16 */
    case 2: *block = 32; *bytes = 18; return 0;  /* Q4_0 */
    case 8: *block = 32; *bytes = 34; return 0;  /* Q8_0 */
    case 12: *block = 256; *bytes = 144; return 0; /* Q4_K */
    case 14: *block = 256; *bytes = 210; return 0; /* Q6_K */
    default: return -1;
    }
}

static inline uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* Six-bit (scale, min) of 32-value sub-block j of a Q4_K block's 12 scale
 * bytes: kernels/iq3_mix.metal:13-15 (kquant_scale_min). */
static inline void q4k_scale_min(const uint8_t *s, uint32_t j, uint32_t *sc, uint32_t *m) {
    if (j < 4) {
        *sc = s[j] & 63u;
        *m = s[j + 4] & 63u;
    } else {
        *sc = (s[j + 4] & 15u) | ((uint32_t)(s[j - 4] >> 6) << 4);
        *m = (uint32_t)(s[j + 4] >> 4) | ((uint32_t)(s[j] >> 6) << 4);
    }
}

/* The dequantised value of element j of a row: kernels/moe.metal:11-28,47-50
 * (weight_at, types 0,1,2,8,14,30) and kernels/iq3_mix.metal:17-24
 * (mix_weight_at, type 12).  Products are formed in fp32 in the order the
 * shader writes them. */
ORACLE_API float oracle_weight_at(const uint8_t *row, uint32_t kind, uint32_t j) {
    switch (kind) {
    case 0: {
        float f;
        memcpy(&f, row + 4u * j, 4);
        return f;
    }
    case 1: return oracle_half_to_float(rd16(row + 2u * j));
    case 30: return oracle_bf16_to_float(rd16(row + 2u * j));
    case 2: {
        const uint8_t *b = row + (j / 32u) * 18u;
        uint32_t k = j % 32u;
        int q = (int)((b[2 + k % 16u] >> (4u * (k / 16u))) & 15u) - 8;
        return oracle_half_to_float(rd16(b)) * (float)q;
    }
    case 8: {
        const uint8_t *b = row + (j / 32u) * 34u;
        return oracle_half_to_float(rd16(b)) * (float)(int8_t)b[2 + j % 32u];
    }
    case 12: {
        const uint8_t *b = row + (j / 256u) * 144u;
        uint32_t k = j % 256u, g = k / 32u, sc, m;
        q4k_scale_min(b + 4, g, &sc, &m);
        uint32_t q = (b[16u + 32u * (k / 64u) + k % 32u] >> (4u * (g % 2u))) & 15u;
        /* both products are exact in fp32; the subtraction rounds once */
        float a = oracle_half_to_float(rd16(b)) * (float)sc * (float)q;
        float c = oracle_half_to_float(rd16(b + 2)) * (float)m;
        return a - c;
    }
    case 14: {
        const uint8_t *b = row + (j / 256u) * 210u;
        uint32_t k = j % 256u, n = k / 128u, l = k % 32u, t = (k % 128u) / 32u;
        uint32_t low = (b[n * 64u + l + (t % 2u) * 32u] >> (t >= 2u ? 4u : 0u)) & 15u;
        uint32_t high = (b[128u + n * 32u + l] >> (2u * t)) & 3u;
        int scale = (int8_t)b[192u + n * 8u + l / 16u + 2u * t];
        float ds = oracle_half_to_float(rd16(b + 208)) * (float)scale;
        return ds * (float)((int)(low | (high << 4)) - 32);
    }
    default: return NAN;
    }
}

/* Whole-matrix dequantisation, out[r*cols + j]: kernels/qwen.metal:35
 * (read_rows) <- Gpu::dequant src/metal.rs:1581-1601.  `rows` counts rows of
 * every stacked expert.  Returns 0, or -1 for a layout validate_matrix
 * (src/metal.rs:1602-1621) rejects. */
ORACLE_API int oracle_dequant_rows(const uint8_t *data, uint64_t cols, uint64_t rows,
                                   uint64_t stride, uint32_t kind, float *out) {
    uint32_t block, bytes;
    if (oracle_geometry(kind, &block, &bytes) || cols == 0 || rows == 0 || cols % block ||
        stride != cols / block * bytes)
        return -1;
    for (uint64_t r = 0; r < rows; ++r)
        for (uint64_t j = 0; j < cols; ++j)
            out[r * cols + j] = oracle_weight_at(data + r * stride, kind, (uint32_t)j);
    return 0;
}

/* ---- matrix-vector ----------------------------------------------------- */

/* y[t][r] = sum_j W[expert][r][j] * x[t][j], accumulated in f64 over the
 * exactly dequantised fp32 weights: the expectation the reference tests
 * build (tests/projections.rs:37-41, src/expert_bench.rs:690-694). */
ORACLE_API int oracle_matvec_f64(const uint8_t *w, uint64_t cols, uint64_t rows, uint64_t stride,
                                 uint32_t kind, uint64_t expert, const float *x, uint64_t count,
                                 double *y) {
    uint32_t block, bytes;
    if (oracle_geometry(kind, &block, &bytes) || cols % block) return -1;
    float *wr = (float *)malloc(cols * sizeof(float));
    if (!wr) return -2;
    for (uint64_t r = 0; r < rows; ++r) {
        const uint8_t *row = w + (expert * rows + r) * stride;
        for (uint64_t j = 0; j < cols; ++j) wr[j] = oracle_weight_at(row, kind, (uint32_t)j);
        for (uint64_t t = 0; t < count; ++t) {
            double s = 0.0;
            const float *xt = x + t * cols;
            for (uint64_t j = 0; j < cols; ++j) s += (double)wr[j] * (double)xt[j];
            y[t * rows + r] = s;
        }
    }
    free(wr);
    return 0;
}

/* The prefill-GEMM expectation: weights AND activations rounded to f16 before
 * the product (kernels/generic.metal:343,355-361), f64 accumulate
 * (src/expert_bench.rs:734-749). */
ORACLE_API int oracle_gemm_f16_f64(const uint8_t *w, uint64_t cols, uint64_t rows, uint64_t stride,
                                   uint32_t kind, uint64_t expert, const float *x, uint64_t count,
                                   double *y) {
    uint32_t block, bytes;
    if (oracle_geometry(kind, &block, &bytes) || cols % block) return -1;
    float *wr = (float *)malloc(cols * sizeof(float));
    float *xh = (float *)malloc(cols * count * sizeof(float));
    if (!wr || !xh) { free(wr); free(xh); return -2; }
    for (uint64_t i = 0; i < cols * count; ++i)
        xh[i] = oracle_half_to_float(oracle_float_to_half(x[i]));
    for (uint64_t r = 0; r < rows; ++r) {
        const uint8_t *row = w + (expert * rows + r) * stride;
        for (uint64_t j = 0; j < cols; ++j)
            wr[j] = oracle_half_to_float(oracle_float_to_half(oracle_weight_at(row, kind, (uint32_t)j)));
        for (uint64_t t = 0; t < count; ++t) {
            double s = 0.0;
            const float *xt = xh + t * cols;
            for (uint64_t j = 0; j < cols; ++j) s += (double)wr[j] * (double)xt[j];
            y[t * rows + r] = s;
        }
    }
    free(wr);
    free(xh);
    return 0;
}

/* fp32 dequantise-then-dot with output rows split over threads: the timed
 * CPU baseline (scalar decode as in weight_at, fp32 accumulate like the
 * shader's lane sums). */
typedef struct {
    const uint8_t *w;
    uint64_t cols, rows, stride, row0, row1, count;
    uint32_t kind;
    const float *x;
    float *y;
} mv_job;

static void *mv_worker(void *arg) {
    mv_job *j = (mv_job *)arg;
    float *wr = (float *)malloc(j->cols * sizeof(float));
    if (!wr) return NULL;
    for (uint64_t r = j->row0; r < j->row1; ++r) {
        const uint8_t *row = j->w + r * j->stride;
        for (uint64_t c = 0; c < j->cols; ++c) wr[c] = oracle_weight_at(row, j->kind, (uint32_t)c);
        for (uint64_t t = 0; t < j->count; ++t) {
            const float *xt = j->x + t * j->cols;
            float s0 = 0, s1 = 0, s2 = 0, s3 = 0;
            uint64_t c = 0;
            for (; c + 4 <= j->cols; c += 4) {
                s0 += wr[c] * xt[c];
                s1 += wr[c + 1] * xt[c + 1];
                s2 += wr[c + 2] * xt[c + 2];
                s3 += wr[c + 3] * xt[c + 3];
            }
            for (; c < j->cols; ++c) s0 += wr[c] * xt[c];
            j->y[t * j->rows + r] = (s0 + s1) + (s2 + s3);
        }
    }
    free(wr);
    return NULL;
}

ORACLE_API int oracle_matvec_f32_mt(const uint8_t *w, uint64_t cols, uint64_t rows, uint64_t stride,
                                    uint32_t kind, uint64_t expert, const float *x, uint64_t count,
                                    float *y, uint32_t threads) {
    uint32_t block, bytes;
    if (oracle_geometry(kind, &block, &bytes) || cols % block) return -1;
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    if (threads > rows) threads = (uint32_t)rows;
    pthread_t tid[256];
    mv_job jobs[256];
    for (uint32_t i = 0; i < threads; ++i) {
        jobs[i] = (mv_job){w + expert * rows * stride, cols, rows, stride,
                           rows * i / threads, rows * (i + 1) / threads, count, kind, x, y};
        if (threads == 1) mv_worker(&jobs[i]);
        else if (pthread_create(&tid[i], NULL, mv_worker, &jobs[i])) return -3;
    }
    if (threads > 1)
        for (uint32_t i = 0; i < threads; ++i) pthread_join(tid[i], NULL);
    return 0;
}

/* ---- activations ------------------------------------------------------- */

/* silu(g)*u or tanh-GeLU(g)*u in fp32: kernels/generic.metal:298 (glu),
 * kernels/moe.metal:405-410 (swiglu), kernels/generic_arch.metal:7-10. */
ORACLE_API float oracle_glu(float g, float u, int gelu) {
    if (gelu) {
        float inner = 0.79788456080286535587989211986876f * g * (1.0f + 0.044715f * g * g);
        return 0.5f * g * (1.0f + tanhf(inner)) * u;
    }
    return (g / (1.0f + expf(-g))) * u;
}

/* ---- routing ----------------------------------------------------------- */

/* Top-k by repeated arg-max, ties to the lowest expert id; weights
 * exp(l - l_top) divided by their sum accumulated in selection order, all in
 * fp32: src/lib.rs:43-60 (route), kernels/generic.metal:479-494 (route_topk).
 * Returns -1 for top == 0, top > n or a non-finite logit. */
ORACLE_API int oracle_route(const float *logits, uint32_t n, uint32_t top, uint32_t *ids,
                            float *weights) {
    if (top == 0 || top > n) return -1;
    for (uint32_t i = 0; i < n; ++i)
        if (!isfinite(logits[i])) return -1;
    uint8_t *taken = (uint8_t *)calloc(n, 1);
    if (!taken) return -2;
    float total = 0.0f, first = 0.0f;
    for (uint32_t k = 0; k < top; ++k) {
        uint32_t best = 0xffffffffu;
        for (uint32_t i = 0; i < n; ++i)
            if (!taken[i] && (best == 0xffffffffu || logits[i] > logits[best])) best = i;
        taken[best] = 1;
        if (k == 0) first = logits[best];
        ids[k] = best;
        weights[k] = expf(logits[best] - first);
        total += weights[k];
    }
    for (uint32_t k = 0; k < top; ++k) weights[k] /= total;
    free(taken);
    return 0;
}

/* ---- MoE glue ---------------------------------------------------------- */

/* y[t][j] = sum_e routed[t*top+e][j] * w[t*top+e], summed in route order in
 * fp32: kernels/generic.metal:17 (moe_sum). */
ORACLE_API void oracle_moe_sum(const float *routed, const float *w, uint64_t width, uint32_t top,
                               uint64_t tokens, float *y) {
    for (uint64_t t = 0; t < tokens; ++t)
        for (uint64_t j = 0; j < width; ++j) {
            float s = 0.0f;
            for (uint32_t e = 0; e < top; ++e)
                s += routed[(t * top + e) * width + j] * w[t * top + e];
            y[t * width + j] = s;
        }
}

/* One token: out = sum_e routed[e]*w[e] + shared / (1 + exp(-shared_logit)):
 * kernels/moe.metal:412-422 (combine). */
ORACLE_API void oracle_combine(const float *routed, const float *shared, const float *w,
                               float shared_logit, uint64_t width, uint32_t top, float *out) {
    for (uint64_t j = 0; j < width; ++j) {
        float s = 0.0f;
        for (uint32_t e = 0; e < top; ++e) s += routed[e * width + j] * w[e];
        out[j] = s + shared[j] / (1.0f + expf(-shared_logit));
    }
}

/* Stable expert-major grouping of (token, expert) pairs for packed prefill:
 * kernels/prefill.metal:7-35 (expert_layout, expert_pairs).
 * layout[2e] = pairs of expert e, layout[2e+1] = first packed position;
 * tiles[4t..] = [expert, first, n<=32, mode(n>=2)], zero-filled up to
 * tile_capacity; pairs[pos] = original pair index (ascending inside an
 * expert); inverse[pair] = packed position.  Returns the tile count or -1. */
ORACLE_API int oracle_expert_layout(const uint32_t *ids, uint32_t n_pairs, uint32_t experts,
                                    uint32_t tile_capacity, uint32_t *layout, uint32_t *tiles,
                                    uint32_t *pairs, uint32_t *inverse) {
    memset(layout, 0, sizeof(uint32_t) * 2u * experts);
    for (uint32_t i = 0; i < n_pairs; ++i) {
        if (ids[i] >= experts) return -1;
        layout[2u * ids[i]]++;
    }
    uint32_t at = 0, tile = 0;
    for (uint32_t e = 0; e < experts; ++e) {
        uint32_t n = layout[2u * e];
        layout[2u * e + 1] = at;
        for (uint32_t k = 0; 32u * k < n; ++k, ++tile) {
            if (tile >= tile_capacity) return -1;
            uint32_t nt = n - 32u * k < 32u ? n - 32u * k : 32u;
            tiles[4u * tile] = e;
            tiles[4u * tile + 1] = at + 32u * k;
            tiles[4u * tile + 2] = nt;
            tiles[4u * tile + 3] = nt >= 2u ? 1u : 0u;
        }
        at += n;
    }
    for (uint32_t t = tile; t < tile_capacity; ++t)
        tiles[4u * t] = tiles[4u * t + 1] = tiles[4u * t + 2] = tiles[4u * t + 3] = 0;
    uint32_t *cursor = (uint32_t *)malloc(sizeof(uint32_t) * (experts ? experts : 1));
    if (!cursor) return -2;
    for (uint32_t e = 0; e < experts; ++e) cursor[e] = layout[2u * e + 1];
    for (uint32_t i = 0; i < n_pairs; ++i) {
        uint32_t pos = cursor[ids[i]]++;
        inverse[i] = pos;
        pairs[pos] = i;
    }
    free(cursor);
    return (int)tile;
}

/* combine over packed expert outputs, route order:
 * kernels/prefill.metal:39 (combine_packed) without the shared-expert term
 * when `shared` is NULL. */
ORACLE_API void oracle_combine_packed(const float *routed, const float *shared, const float *w,
                                      const float *gate, const uint32_t *inverse, uint64_t width,
                                      uint32_t top, uint64_t tokens, float *out) {
    for (uint64_t t = 0; t < tokens; ++t)
        for (uint64_t j = 0; j < width; ++j) {
            float s = 0.0f;
            for (uint32_t e = 0; e < top; ++e)
                s += routed[(uint64_t)inverse[t * top + e] * width + j] * w[t * top + e];
            if (shared) s = s + shared[t * width + j] / (1.0f + expf(-gate[t]));
            out[t * width + j] = s;
        }
}

/* Residual add + RMS norm of one row (a "next" operator of the decode step):
 * s = a + b (when add), y = s * rsqrt(mean(s^2) + eps) * w:
 * kernels/generic.metal:390-404 (add_rms).  `w` may be NULL (unit weight). */
ORACLE_API void oracle_add_rms(const float *a, const float *b, const float *w, uint64_t width,
                               float eps, int add, float *s_out, float *y) {
    double ss = 0.0;
    for (uint64_t j = 0; j < width; ++j) {
        float s = add ? a[j] + b[j] : a[j];
        if (s_out) s_out[j] = s;
        ss += (double)s * (double)s;
    }
    float scale = (float)(1.0 / sqrt(ss / (double)width + (double)eps));
    for (uint64_t j = 0; j < width; ++j) {
        float s = add ? a[j] + b[j] : a[j];
        y[j] = s * scale * (w ? w[j] : 1.0f);
    }
}

/* ------------------------------------------------------------------------
 * The rest of a generic decode step.
 * ------------------------------------------------------------------------ */

/* embedding_batch (kernels/qwen.metal:139): y[t][j] = weight_at(row ids[t], j). */
ORACLE_API int oracle_embedding(const uint8_t *w, const uint32_t *ids, uint64_t width, uint64_t rows, uint64_t stride,
                                uint32_t kind, uint64_t count, float *y) {
    for (uint64_t t = 0; t < count; ++t) {
        if (ids[t] >= rows) return -1;
        if (oracle_dequant_rows(w + (uint64_t)ids[t] * stride, width, 1, stride, kind, y + t * width)) return -2;
    }
    return 0;
}

/* qk_rope_cache (kernels/generic.metal:405-438), one head row at a time, float arithmetic as written there. */
ORACLE_API void oracle_qk_rope_cache(const float *q, const float *k, const float *v, const float *qn, const float *kn,
                                     const float *factors, float *qo, float *kc, float *vc, uint32_t D, uint32_t H,
                                     uint32_t KV, uint32_t rot, uint32_t position, float base, int neox, int use_factors,
                                     int qk_norm, float eps, int value_norm, float q_scale, uint32_t tokens) {
    float row[512];
    for (uint32_t t = 0; t < tokens; ++t)
        for (uint32_t r = 0; r < H + 2 * KV; ++r) {
            if (r >= H + KV) {
                uint32_t h = r - H - KV;
                const float *src = v + ((uint64_t)t * KV + h) * D;
                float *dst = vc + ((uint64_t)(position + t) * KV + h) * D;
                float inv = 1.0f;
                if (value_norm) {
                    double s = 0.0;
                    for (uint32_t j = 0; j < D; ++j) s += (double)src[j] * src[j];
                    inv = (float)(1.0 / sqrt(s / D + eps));
                }
                for (uint32_t j = 0; j < D; ++j) dst[j] = value_norm ? src[j] * inv : src[j];
                continue;
            }
            int isq = r < H;
            uint32_t h = isq ? r : r - H;
            const float *src = isq ? q + ((uint64_t)t * H + h) * D : k + ((uint64_t)t * KV + h) * D;
            float *dst = isq ? qo + ((uint64_t)t * H + h) * D : kc + ((uint64_t)(position + t) * KV + h) * D;
            const float *w = isq ? qn : kn;
            float inv = 1.0f;
            if (qk_norm) {
                double s = 0.0;
                for (uint32_t j = 0; j < D; ++j) s += (double)src[j] * src[j];
                inv = (float)(1.0 / sqrt(s / D + eps));
            }
            for (uint32_t j = 0; j < D; ++j) row[j] = qk_norm ? src[j] * inv * w[j] : src[j];
            float qs = isq ? q_scale : 1.0f;
            for (uint32_t j = 0; j < D; ++j) {
                if (j >= rot) { dst[j] = row[j] * qs; continue; }
                uint32_t f = neox ? j % (rot / 2) : j / 2, a = neox ? f : (j & ~1u), b = neox ? a + rot / 2 : a + 1;
                double theta = (double)(position + t) * pow((double)base, -2.0 * (double)f / (double)rot);
                if (use_factors) theta /= factors[f];
                double c = cos(theta), s = sin(theta);
                int first = neox ? j < rot / 2 : (j & 1u) == 0;
                double y = first ? row[a] * c - row[b] * s : row[a] * s + row[b] * c;
                dst[j] = (float)(y * qs);
            }
        }
}

/* attention_decode (kernels/generic.metal:440-474) as plain softmax attention in double. */
ORACLE_API void oracle_attention_decode(const float *q, const float *k, const float *v, float *out, uint32_t D, uint32_t H,
                                        uint32_t KV, uint32_t position, uint32_t window, uint32_t tokens) {
    double *score = (double *)malloc(sizeof(double) * (position + tokens + 1));
    for (uint32_t t = 0; t < tokens; ++t)
        for (uint32_t h = 0; h < H; ++h) {
            uint32_t kh = h / (H / KV), stride = KV * D, length = position + t + 1;
            uint32_t start = window && length > window ? length - window : 0;
            const float *qr = q + ((uint64_t)t * H + h) * D;
            double m = -INFINITY;
            for (uint32_t pos = start; pos < length; ++pos) {
                const float *kr = k + (uint64_t)pos * stride + kh * D;
                double s = 0.0;
                for (uint32_t j = 0; j < D; ++j) s += (double)qr[j] * kr[j];
                score[pos] = s / sqrt((double)D);
                if (score[pos] > m) m = score[pos];
            }
            double l = 0.0;
            for (uint32_t pos = start; pos < length; ++pos) { score[pos] = exp(score[pos] - m); l += score[pos]; }
            for (uint32_t j = 0; j < D; ++j) {
                double acc = 0.0;
                for (uint32_t pos = start; pos < length; ++pos) acc += score[pos] * v[(uint64_t)pos * stride + kh * D + j];
                out[((uint64_t)t * H + h) * D + j] = (float)(acc / l);
            }
        }
    free(score);
}

/* greedy_select (kernels/qwen.metal:384-410): largest value, ties (signed zeros included) to the smaller
 * token id; bad = a non-finite value was seen. */
ORACLE_API void oracle_greedy(const float *logits, const uint32_t *mapping, uint64_t rows, uint64_t vocab, uint32_t *out) {
    for (uint64_t r = 0; r < rows; ++r) {
        float best = -INFINITY;
        uint32_t id = 0xffffffffu, bad = 0;
        for (uint64_t i = 0; i < vocab; ++i) {
            float value = logits[r * vocab + i];
            uint32_t token = mapping ? mapping[i] : (uint32_t)i;
            bad |= !isfinite(value);
            if (value > best || (value == best && token < id)) { best = value; id = token; }
        }
        out[2 * r] = id;
        out[2 * r + 1] = bad;
    }
}
