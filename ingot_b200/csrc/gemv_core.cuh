// The streaming GEMV: launch plan and the per-warp arithmetic.
//
// One CTA owns a contiguous range of output rows.  A producer warp streams the
// rows' packed bytes into a ring of shared-memory stages with 1-D bulk async
// copies (16-byte aligned, any block size); eight consumer warps decode units
// out of shared memory and accumulate in fp32.  The activations sit in shared
// memory too, permuted so that every lane reads its eight float4 without bank
// conflicts.  The plan (lanes per row, steps, chunking, stages) is a pure
// function of the shape, so the same plan and the same arithmetic run on the
// host in tests/host_emulation.cpp.
//
// Replaces the reference's mv_q4k/mv_q6k/mv_q4_0 (kernels/generic.metal:182-313),
// kquant_vector (kernels/iq3_mix.metal:85-128), q6k_vector
// (kernels/decode.metal:57-86), q4_0_vector (kernels/generic.metal:150-174) and
// q8_dense (kernels/qwen.metal:1103-1117).
#pragma once
#include "quant.cuh"

namespace ingot {

static constexpr int GEMV_CONSUMER_WARPS = 8;
static constexpr int GEMV_THREADS = (GEMV_CONSUMER_WARPS + 1) * 32;   // + producer warp
static constexpr int GEMV_NR = 2;                  // rows per lane group sharing one x load
static constexpr int GEMV_MAX_STAGES = 8;
static constexpr uint32_t GEMV_SMEM_BUDGET = 112u * 1024u;   // two CTAs per SM
static constexpr uint32_t GEMV_SMEM_MAX = 224u * 1024u;      // one CTA per SM, for shapes that need the room
static constexpr uint32_t GEMV_STAGE_TARGET = 20u * 1024u;
static constexpr uint32_t GEMV_BAR_BYTES = 128;

struct GemvPlan {
    uint32_t kind, cols, rows, stride;
    uint32_t units;          // 32-weight units per row
    uint32_t lpr_log2;       // lanes per row = 1 << lpr_log2 (8, 16 or 32)
    uint32_t steps;          // ceil(units / lpr)
    uint32_t spc;            // steps per chunk
    uint32_t chunks;         // ceil(steps / spc)
    uint32_t chunk_bytes;    // bytes of one row in a full chunk (multiple of 16)
    uint32_t last_chunk_bytes;
    uint32_t tile_rows;      // rows per stage = warps * NR * (32 / lpr)
    uint32_t nmat;           // 1, or 2 for fused gate/up
    uint32_t ntok;
    uint32_t stages, stage_bytes;
    uint32_t x_bytes;        // permuted activations
    uint32_t smem_bytes;
    uint32_t ctas;           // CTAs along the row dimension
};

inline uint32_t units_per_block(uint32_t kind) { return (kind == KIND_Q4_K || kind == KIND_Q6_K) ? 8u : 1u; }

// Builds the plan; false when the shape needs the plain kernel instead
// (unaligned rows, a float weight type, or activations that do not fit).
inline bool plan_gemv(uint32_t kind, uint32_t cols, uint32_t rows, uint32_t stride, uint32_t ntok,
                      uint32_t nmat, uint32_t max_ctas, GemvPlan &p, uint32_t budget = GEMV_SMEM_BUDGET) {
    uint32_t block, bytes;
    if (!geometry(kind, block, bytes) || block == 1) return false;
    if (cols == 0 || rows == 0 || cols % block || stride != cols / block * bytes) return false;
    if (stride % 16u) return false;
    p.kind = kind; p.cols = cols; p.rows = rows; p.stride = stride; p.nmat = nmat; p.ntok = ntok;
    p.units = cols / 32u;
    // lanes per row: least padding, then the widest
    uint32_t best = 5, best_waste = ~0u;
    for (uint32_t lg = 5; lg >= 3; --lg) {
        uint32_t lpr = 1u << lg, waste = (p.units + lpr - 1) / lpr * lpr - p.units;
        if (waste < best_waste) { best_waste = waste; best = lg; }
    }
    p.lpr_log2 = best;
    const uint32_t lpr = 1u << best, upb = units_per_block(kind);
    p.steps = (p.units + lpr - 1) / lpr;
    p.tile_rows = GEMV_CONSUMER_WARPS * GEMV_NR * (32u / lpr);
    p.x_bytes = ntok * p.steps * lpr * 8u * 16u;
    if (p.x_bytes + GEMV_BAR_BYTES >= budget) return false;
    // chunk: the largest aligned number of steps whose stage stays near the target
    uint32_t pick = 0;
    for (uint32_t spc = 1; spc <= p.steps; ++spc) {
        uint32_t cb;
        if (spc == p.steps) cb = stride;
        else {
            if ((spc * lpr) % upb) continue;
            cb = spc * lpr / upb * bytes;
            if (cb % 16u) continue;
        }
        uint32_t sb = cb * p.tile_rows * nmat;
        if (pick == 0) pick = spc;                    // smallest legal chunk
        else if (sb <= GEMV_STAGE_TARGET) pick = spc;
    }
    if (pick == 0) return false;
    p.spc = pick;
    p.chunks = (p.steps + pick - 1) / pick;
    p.chunk_bytes = (pick == p.steps) ? stride : pick * lpr / upb * bytes;
    p.last_chunk_bytes = stride - (p.chunks - 1) * p.chunk_bytes;
    p.stage_bytes = (p.chunk_bytes * p.tile_rows * nmat + 16u + 127u) & ~127u;
    uint32_t x_al = (p.x_bytes + 127u) & ~127u;
    uint32_t room = budget - GEMV_BAR_BYTES - x_al;
    p.stages = room / p.stage_bytes;
    if (p.stages > GEMV_MAX_STAGES) p.stages = GEMV_MAX_STAGES;
    if (p.stages < 2) return false;
    p.smem_bytes = GEMV_BAR_BYTES + x_al + p.stages * p.stage_bytes;
    uint32_t want = (rows + 3u) / 4u;                 // at least four rows per CTA
    p.ctas = want < max_ctas ? want : max_ctas;
    if (p.ctas == 0) p.ctas = 1;
    return true;
}

// Rows [begin, end) of CTA `cta` out of `ctas`.
IG_HD void cta_rows(uint32_t rows, uint32_t cta, uint32_t ctas, uint32_t &begin, uint32_t &end) {
    begin = (uint32_t)((uint64_t)rows * cta / ctas);
    end = (uint32_t)((uint64_t)rows * (cta + 1) / ctas);
}

// Position (in float4) of activation float4 `i` of unit `u`, token `t`.
IG_HD uint32_t x_slot(const GemvPlan &p, uint32_t t, uint32_t u, uint32_t i) {
    uint32_t lpr = 1u << p.lpr_log2, step = u >> p.lpr_log2, sub = u & (lpr - 1u);
    return (((t * p.steps + step) * 8u + i) << p.lpr_log2) + sub;
}

// One consumer warp's lane on one chunk of one tile.  `stage` holds, for each
// matrix m and tile row r, the chunk's bytes at (m * tile_rows + r) * chunk_bytes.
template <uint32_t KIND, int NTOK, int NMAT>
IG_HD void consume_chunk(const uint8_t *stage, const F4 *xs, const GemvPlan &p, uint32_t warp,
                         uint32_t lane, uint32_t chunk, uint32_t rows_valid,
                         float (&acc)[GEMV_NR][NMAT][NTOK]) {
    using Un = Unit<KIND>;
    const uint32_t lpr = 1u << p.lpr_log2, sub = lane & (lpr - 1u), rs = lane >> p.lpr_log2;
    const uint32_t slots = 32u >> p.lpr_log2;
    const uint32_t step0 = chunk * p.spc;
    const uint32_t nsteps = (p.steps - step0) < p.spc ? (p.steps - step0) : p.spc;
    uint32_t lrow[GEMV_NR];
    bool ok[GEMV_NR];
#pragma unroll
    for (int nr = 0; nr < GEMV_NR; ++nr) {
        lrow[nr] = (warp * GEMV_NR + nr) * slots + rs;
        ok[nr] = lrow[nr] < rows_valid;
    }
    for (uint32_t cs = 0; cs < nsteps; ++cs) {
        const uint32_t step = step0 + cs, u = (step << p.lpr_log2) + sub;
        if (u >= p.units) continue;
        const uint32_t uc = (cs << p.lpr_log2) + sub;
        typename Un::W w[GEMV_NR][NMAT];
#pragma unroll
        for (int nr = 0; nr < GEMV_NR; ++nr)
#pragma unroll
            for (int m = 0; m < NMAT; ++m)
                if (ok[nr]) w[nr][m] = Un::load(stage + (size_t)(m * p.tile_rows + lrow[nr]) * p.chunk_bytes, uc);
#pragma unroll
        for (int t = 0; t < NTOK; ++t) {
            F4 x[8];
            const F4 *xp = xs + ((((uint32_t)t * p.steps + step) * 8u) << p.lpr_log2) + sub;
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = xp[(uint32_t)i << p.lpr_log2];
            const typename Un::Aux ax = Un::aux(x);
#pragma unroll
            for (int nr = 0; nr < GEMV_NR; ++nr)
#pragma unroll
                for (int m = 0; m < NMAT; ++m)
                    if (ok[nr]) acc[nr][m][t] = add_rn(acc[nr][m][t], Un::dot(w[nr][m], x, ax));
        }
    }
}

// Bytes of one activation row packed for the tensor-core GEMV: binary16 (xh, xl)
// pairs in B-operand order, fp32 sums of each 16 columns, and 16 bytes holding
// 1/scale.  cols must be a multiple of 64.
IG_HD uint32_t packed_x_bytes(uint32_t cols) { return cols * 4u + cols / 4u + 16u; }
// The same holding only the high binary16 part (bfloat16 activations).
IG_HD uint32_t packed_hi_bytes(uint32_t cols) { return cols * 2u + cols / 4u + 16u; }

// Bytes of one activation row in fixed point for the int8 mma.sync GEMV: `nd` digit planes per
// sub-block of 32 and two float2 of scale and run sum per sub-block (pack.cuh: fx_store).
IG_HD uint32_t fx_row_bytes(uint32_t cols, uint32_t nd) { return cols * nd + cols / 2u; }

// Bytes of one activation row as base-256 digits for the int8 tensor-core GEMV: the
// N = 8 operand image (8 bytes per column), fp32 sums of each 16 columns, 16 bytes
// holding 1/scale.  cols must be a multiple of 256.
IG_HD uint32_t packed_digits_bytes(uint32_t cols) { return cols * 8u + cols / 4u + 16u; }

// silu(g)*u or tanh-GeLU(g)*u (reference glu: kernels/generic.metal:298).
IG_HD float glu_f(float g, float u, bool gelu) {
    if (gelu) {
        float inner = 0.79788456080286535587989211986876f * g * (1.0f + 0.044715f * g * g);
        return 0.5f * g * (1.0f + tanhf(inner)) * u;
    }
    return (g / (1.0f + expf(-g))) * u;
}

}  // namespace ingot
