// CPU emulation of the streaming GEMV kernel: the same launch plan, the same
// activation permutation and the same per-lane arithmetic (quant.cuh and
// gemv_core.cuh compile as plain C++), with the bulk copies replaced by memcpy
// and the warp shuffles by loops over 32 lane values.  Built by
// tests/test_host_emulation.py; lets index arithmetic and rounding behaviour be
// checked against the oracle without a GPU.
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "../ingot_b200/csrc/gemv_core.cuh"

using namespace ingot;

namespace {

template <uint32_t KIND, int NTOK, int NMAT>
int run(const GemvPlan &p, const uint8_t *w0, const uint8_t *w1, uint32_t expert, const float *x, float *y, int gelu) {
    const uint8_t *w[2] = {w0, w1};
    const uint32_t lpr = 1u << p.lpr_log2, slots = 32u >> p.lpr_log2;
    // permuted activations, exactly as stage_x lays them out
    std::vector<F4> xs(p.x_bytes / 16u);
    for (uint32_t t = 0; t < (uint32_t)NTOK; ++t)
        for (uint32_t f = 0; f < p.cols / 4u; ++f) {
            uint32_t u, i;
            Unit<KIND>::locate(4u * f, u, i);
            if (Unit<KIND>::col(u, i) != 4u * f) return -10;         // locate must invert col
            const float *s = x + (size_t)t * p.cols + 4u * f;
            F4 v = permute_x(s[0], s[1], s[2], s[3]);
            xs[x_slot(p, t, u, i)] = v;
        }
    void *raw = nullptr;
    if (posix_memalign(&raw, 128, (size_t)p.stages * p.stage_bytes)) return -11;
    uint8_t *stages = static_cast<uint8_t *>(raw);
    const size_t mat_off = (size_t)expert * p.rows * p.stride;
    for (uint32_t cta = 0; cta < p.ctas; ++cta) {
        uint32_t r_begin, r_end;
        cta_rows(p.rows, cta, p.ctas, r_begin, r_end);
        const uint32_t n_tiles = (r_end - r_begin + p.tile_rows - 1) / p.tile_rows;
        uint32_t it = 0;
        for (uint32_t tile = 0; tile < n_tiles; ++tile) {
            const uint32_t row0 = r_begin + tile * p.tile_rows;
            const uint32_t nrows = (r_end - row0) < p.tile_rows ? (r_end - row0) : p.tile_rows;
            std::vector<float> acc((size_t)GEMV_CONSUMER_WARPS * 32 * GEMV_NR * NMAT * NTOK, 0.f);
            for (uint32_t c = 0; c < p.chunks; ++c, ++it) {
                uint8_t *dst = stages + (size_t)(it % p.stages) * p.stage_bytes;
                memset(dst, 0xA5, p.stage_bytes);                       // stale bytes must never matter
                const uint32_t cb = (c + 1 == p.chunks) ? p.last_chunk_bytes : p.chunk_bytes;
                for (uint32_t m = 0; m < (uint32_t)NMAT; ++m)
                    for (uint32_t r = 0; r < nrows; ++r)
                        memcpy(dst + (size_t)(m * p.tile_rows + r) * p.chunk_bytes,
                               w[m] + mat_off + (size_t)(row0 + r) * p.stride + (size_t)c * p.chunk_bytes, cb);
                for (uint32_t warp = 0; warp < (uint32_t)GEMV_CONSUMER_WARPS; ++warp)
                    for (uint32_t lane = 0; lane < 32; ++lane) {
                        float a[GEMV_NR][NMAT][NTOK];
                        float *slot = &acc[((size_t)warp * 32 + lane) * GEMV_NR * NMAT * NTOK];
                        memcpy(a, slot, sizeof(a));
                        consume_chunk<KIND, NTOK, NMAT>(dst, xs.data(), p, warp, lane, c, nrows, a);
                        memcpy(slot, a, sizeof(a));
                    }
            }
            for (uint32_t warp = 0; warp < (uint32_t)GEMV_CONSUMER_WARPS; ++warp)
                for (int nr = 0; nr < GEMV_NR; ++nr)
                    for (int t = 0; t < NTOK; ++t) {
                        float red[NMAT][32];
                        for (int m = 0; m < NMAT; ++m) {
                            for (uint32_t lane = 0; lane < 32; ++lane)
                                red[m][lane] = acc[(((size_t)warp * 32 + lane) * GEMV_NR + nr) * NMAT * NTOK + (size_t)m * NTOK + t];
                            for (uint32_t off = lpr >> 1; off; off >>= 1) {
                                float next[32];
                                for (uint32_t lane = 0; lane < 32; ++lane) next[lane] = red[m][lane] + red[m][lane ^ off];
                                memcpy(red[m], next, sizeof(next));
                            }
                        }
                        for (uint32_t rs = 0; rs < slots; ++rs) {
                            const uint32_t lrow = (warp * GEMV_NR + nr) * slots + rs;
                            if (lrow >= nrows) continue;
                            const uint32_t lane = rs << p.lpr_log2;
                            const size_t o = (size_t)t * p.rows + row0 + lrow;
                            y[o] = NMAT == 2 ? glu_f(red[0][lane], red[NMAT - 1][lane], gelu != 0) : red[0][lane];
                        }
                    }
        }
    }
    free(raw);
    return 0;
}

template <uint32_t KIND, int NMAT>
int run_n(const GemvPlan &p, const uint8_t *w0, const uint8_t *w1, uint32_t e, const float *x, float *y, int gelu) {
    switch (p.ntok) {
    case 1: return run<KIND, 1, NMAT>(p, w0, w1, e, x, y, gelu);
    case 2: return run<KIND, 2, NMAT>(p, w0, w1, e, x, y, gelu);
    case 3: return run<KIND, 3, NMAT>(p, w0, w1, e, x, y, gelu);
    case 4: return run<KIND, 4, NMAT>(p, w0, w1, e, x, y, gelu);
    }
    return -12;
}

template <uint32_t KIND>
int run_k(const GemvPlan &p, const uint8_t *w0, const uint8_t *w1, uint32_t e, const float *x, float *y, int gelu) {
    return p.nmat == 2 ? run_n<KIND, 2>(p, w0, w1, e, x, y, gelu) : run_n<KIND, 1>(p, w0, w1, e, x, y, gelu);
}

}  // namespace

extern "C" {

// Returns 0, 1 when the plan says "use the plain kernel", negative on error.
// plan_out (may be null) receives the GemvPlan as uint32 words.
int emulate_gemv(uint32_t kind, const uint8_t *w0, const uint8_t *w1, uint32_t cols, uint32_t rows, uint32_t stride,
                 uint32_t expert, const float *x, uint32_t ntok, uint32_t nmat, int gelu, uint32_t max_ctas, float *y,
                 uint32_t *plan_out) {
    GemvPlan p;
    if (!plan_gemv(kind, cols, rows, stride, ntok, nmat, max_ctas, p)) return 1;
    if (plan_out) memcpy(plan_out, &p, sizeof(p));
    switch (kind) {
    case KIND_Q4_K: return run_k<KIND_Q4_K>(p, w0, w1, expert, x, y, gelu);
    case KIND_Q6_K: return run_k<KIND_Q6_K>(p, w0, w1, expert, x, y, gelu);
    case KIND_Q4_0: return run_k<KIND_Q4_0>(p, w0, w1, expert, x, y, gelu);
    case KIND_Q8_0: return run_k<KIND_Q8_0>(p, w0, w1, expert, x, y, gelu);
    }
    return -13;
}

float emulate_weight_at(const uint8_t *row, uint32_t kind, uint32_t j) { return weight_at(row, kind, j); }

uint32_t emulate_plan_words(void) { return (uint32_t)(sizeof(GemvPlan) / 4u); }
}
