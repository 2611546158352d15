// Batched prefill: Y[T][N] = X[T][K] . W^T for block-quantised W, on the 5th-generation
// tensor cores (tcgen05) with dequantise-on-load.
//
// Replaces the reference's generic_gemm / gemm_q4k / gemm_q6k (kernels/generic.metal:315-388):
// like it, weights AND activations are rounded to binary16 before the product and the
// accumulation is fp32 (its simdgroup_half8x8 staging, :343,355-361), so results are held
// to the same expectation (f64 dot of F16-rounded operands, src/expert_bench.rs:734-749).
//
// One CTA computes a 128 (weight rows) x 256 (tokens) tile of Y^T — or, for more than 256 tokens,
// two such tiles side by side (512 tokens, two accumulators) so that every decoded weight tile is
// used twice: the decode, not the tensor pipe, bounds this kernel.  Per 64-column K step:
//   * eight warps (two groups of eight take alternate steps) decode half a weight row each (32
//     columns) — the fp32 value d*sc*q - dmin*m
//     (Q4_K) or d*scale*(q-32) (Q6_K) exactly as weight_at forms it, rounded to binary16 — and
//     store the 128 x 64 tile K-major with the 128-byte swizzle the tensor core expects;
//   * one thread brings each 256 x 64 activation tile (already binary16) with one 2-D TMA
//     copy whose tensor map applies the same 128-byte swizzle;
//   * one thread per accumulator issues four tcgen05.mma (M 128, N 256, K 16), accumulating in
//     tensor memory (256 columns x 128 lanes of fp32 each), and a tcgen05.commit frees the stage.
// After the last step the sixteen decode warps read the accumulator with tcgen05.ld (each warp
// its 32 lanes and a quarter of the token columns) and write Y (token-major) with coalesced stores.
// Every wait is bounded.
#include <cuda_fp16.h>

#include "dev_common.cuh"
#include "gemv_core.cuh"
#include "kernels.h"
#include "ptx.cuh"
#include "tensor_map.h"

namespace ingot {

static constexpr uint32_t GEMM_M = 128;          // weight rows per CTA (MMA M)
static constexpr uint32_t GEMM_N = 256;          // tokens per CTA (MMA N)
static constexpr uint32_t GEMM_K = 64;           // columns per stage (4 MMAs of K 16)
static constexpr uint32_t GEMM_MAX_STAGES = 4;
static constexpr uint32_t GEMM_A_BYTES = GEMM_M * GEMM_K * 2;       // 16 KB
static constexpr uint32_t GEMM_B_BYTES = GEMM_N * GEMM_K * 2;       // 32 KB per block of 256 tokens
// NB = blocks of 256 tokens per CTA, each with its own 256-column accumulator: with two, a decoded
// weight tile is multiplied with 512 tokens.  The weight tiles and the activation tiles have rings
// of their own.  Two stages each with two accumulators (162 KB): a third activation stage (231 KB)
// left the decode loads 25 KB of L1 and ran Q6_K 25 % slower, Q4_K no faster.
template <uint32_t NB> struct GemmShape {
    static constexpr uint32_t A_STAGES = NB == 1 ? 4u : 2u;
    static constexpr uint32_t B_STAGES = NB == 1 ? 4u : 2u;
    static constexpr uint32_t B_STAGE_BYTES = NB * GEMM_B_BYTES;
    static constexpr uint32_t SMEM = 1024 + A_STAGES * GEMM_A_BYTES + B_STAGES * B_STAGE_BYTES + 1024;   // + alignment slack
};
static constexpr uint32_t GEMM_DECODE_THREADS = 256;    // 8 warps decode one K step (half a weight row per thread) ...
static constexpr uint32_t GEMM_DECODE_GROUPS = 2;       // ... and two such groups take alternate steps: the decode is a long
                                                        // dependent chain per thread, and more warps hide its latency
static constexpr uint32_t GEMM_DECODE_WARPS = GEMM_DECODE_GROUPS * GEMM_DECODE_THREADS / 32u;
// + 1 copy warp and one MMA warp per accumulator: issuing a tcgen05.mma costs its thread about 100 cycles,
// so one thread issuing the eight MMAs of a step (two accumulators) would take most of the step's tensor time
static constexpr uint32_t GEMM_THREADS = (GEMM_DECODE_WARPS + 3u) * 32u;

struct GemmArgs {
    const uint8_t *w;          // [rows][stride] of expert `expert`
    const __half *x;           // [tokens][cols] binary16
    float *y;                  // [tokens][rows]
    uint32_t cols, rows, stride, kind, tokens;
    int *status;
    // K split over gridDim.z CTAs when the tiles alone do not fill the GPU: split z writes its partial
    // products to partial[z][tokens][rows] and a second kernel adds them in order
    float *partial;
};

// ---- tcgen05 wrappers -------------------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_addr(dst_smem)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ptx::smem_addr(bar))
                 : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, binary16 operands, fp32 accumulate
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 32 consecutive fp32 columns of tensor memory -> 32 registers per thread
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor: K-major tile of 128-byte rows, 128-byte swizzle, eight-row
// groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_k128(uint32_t smem_byte_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_byte_addr & 0x3ffffu) >> 4);       // start address
    d |= (uint64_t)1 << 16;                                    // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024u >> 4) << 32;                         // stride byte offset: 8 rows x 128 B
    d |= (uint64_t)1 << 46;                                    // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                                    // SWIZZLE_128B
    return d;
}
// kind::f16 instruction descriptor: F16 x F16 -> F32, both operands K-major, M x N
__device__ __forceinline__ uint32_t idesc_f16(uint32_t m, uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// byte offset of element (row, k) in a K-major tile of 64 binary16 per row with the 128-byte swizzle
__device__ __forceinline__ uint32_t swz_off(uint32_t row, uint32_t chunk16) { return row * 128u + ((chunk16 ^ (row & 7u)) << 4); }

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// Byte i of `v` as a float, through the bits of 2^23 + byte (exact; no integer-to-float conversion,
// which runs on a slower pipe than the fp32 arithmetic that follows).
__device__ __forceinline__ float magic_byte(uint32_t v, uint32_t i) {
    return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7650u | i));      // 8388608 + byte
}
static constexpr float MAGIC = 8388608.0f;

// ---- decoding 32 consecutive weights of one row into half a swizzled tile row ----------------
// Split in two: `load` brings the raw bytes of a step into registers (issued one step ahead, so the
// global-memory latency overlaps the previous step's arithmetic), `emit` decodes and stores.

struct GemmRaw {
    uint32_t w[18];
};

// Q4_K: K step ks covers group j = ks % 4 of block ks / 4: 32 bytes whose low nibbles are sub-block
// 2j (columns 0..31 of the step, half 0) and whose high nibbles are sub-block 2j+1 (columns 32..63,
// half 1).  Raw: header (4 words), quants (8 words).
__device__ __forceinline__ void load32_q4k(const uint8_t *row, uint32_t ks, GemmRaw &raw) {
    const uint8_t *b = row + (size_t)(ks >> 2) * 144u;
    const uint32_t j = ks & 3u;
    const uint4 hdr = *reinterpret_cast<const uint4 *>(b);
    const uint4 q0 = *reinterpret_cast<const uint4 *>(b + 16u + 32u * j);
    const uint4 q1 = *reinterpret_cast<const uint4 *>(b + 32u + 32u * j);
    raw.w[0] = hdr.x; raw.w[1] = hdr.y; raw.w[2] = hdr.z; raw.w[3] = hdr.w;
    raw.w[4] = q0.x; raw.w[5] = q0.y; raw.w[6] = q0.z; raw.w[7] = q0.w;
    raw.w[8] = q1.x; raw.w[9] = q1.y; raw.w[10] = q1.z; raw.w[11] = q1.w;
}
__device__ __forceinline__ void emit32_q4k(const GemmRaw &raw, uint32_t ks, uint32_t half, uint8_t *dst_row_base, uint32_t r) {
    const uint32_t sb = 2u * (ks & 3u) + half;
    // six-bit (scale, min) of sub-block sb (get_scale_min_k4): words 1, 2, 3 = scale bytes 0..3, 4..7, 8..11
    uint32_t sc, mn;
    if (sb < 4u) {
        sc = (raw.w[1] >> (8u * sb)) & 63u;
        mn = (raw.w[2] >> (8u * sb)) & 63u;
    } else {
        const uint32_t hi = (raw.w[3] >> (8u * (sb - 4u))) & 0xffu;
        sc = (hi & 15u) | ((((raw.w[1] >> (8u * (sb - 4u))) >> 6) & 3u) << 4);
        mn = (hi >> 4) | ((((raw.w[2] >> (8u * (sb - 4u))) >> 6) & 3u) << 4);
    }
    const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&raw.w[0]));
    const float ds = __fmul_rn(dd.x, (float)sc), c = __fmul_rn(dd.y, (float)mn);
    // ds * q with one rounding, as fmul would give: fma(ds, 2^23 + q, -(ds * 2^23)); the product with
    // 2^23 is exact
    const float nds = -__fmul_rn(ds, MAGIC);
    const uint32_t sh = 4u * half;
#pragma unroll
    for (uint32_t ch = 0; ch < 4; ++ch) {           // 16-byte chunk: 8 columns = bytes 8 ch .. 8 ch + 7 of the group
        uint32_t out[4];
#pragma unroll
        for (uint32_t i = 0; i < 2; ++i) {
            const uint32_t wq = (raw.w[4 + 2 * ch + i] >> sh) & 0x0f0f0f0fu;
            const float p0 = __fmaf_rn(ds, magic_byte(wq, 0), nds), p1 = __fmaf_rn(ds, magic_byte(wq, 1), nds);
            const float p2 = __fmaf_rn(ds, magic_byte(wq, 2), nds), p3 = __fmaf_rn(ds, magic_byte(wq, 3), nds);
            out[2 * i] = pack_h2(__fsub_rn(p0, c), __fsub_rn(p1, c));
            out[2 * i + 1] = pack_h2(__fsub_rn(p2, c), __fsub_rn(p3, c));
        }
        *reinterpret_cast<uint4 *>(dst_row_base + swz_off(r, 4u * half + ch)) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// 32-bit word at a 2-byte aligned global address
__device__ __forceinline__ uint32_t ldg32_u2(const uint8_t *p) {
    const unsigned short *h = reinterpret_cast<const unsigned short *>(p);
    return (uint32_t)h[0] | ((uint32_t)h[1] << 16);
}

// Q4_0 (the reference's gemm_q4_0: generic_gemm instantiated at kernels/generic.metal:387): a thread's 32 columns
// are one 18-byte block (binary16 d, then 16 bytes whose low nibbles are elements 0..15 and whose high nibbles are
// elements 16..31; w = d (q - 8)).  Blocks are only 2-byte aligned.  Raw: d, then the four words of quants.
__device__ __forceinline__ void load32_q40(const uint8_t *row, uint32_t ks, uint32_t half, GemmRaw &raw) {
    const uint8_t *b = row + (size_t)(2u * ks + half) * 18u;
    raw.w[0] = *reinterpret_cast<const unsigned short *>(b);
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) raw.w[1 + i] = ldg32_u2(b + 2u + 4u * i);
}
__device__ __forceinline__ void emit32_q40(const GemmRaw &raw, uint32_t half, uint8_t *dst_row_base, uint32_t r) {
    const float d = __half2float(__ushort_as_half((unsigned short)raw.w[0]));
#pragma unroll
    for (uint32_t ch = 0; ch < 4; ++ch) {           // 8 columns: bytes 8 (ch % 2) .. + 7, low nibbles for ch < 2, high for the rest
        uint32_t out[4];
#pragma unroll
        for (uint32_t i = 0; i < 2; ++i) {
            const uint32_t wq = (raw.w[1 + 2 * (ch & 1u) + i] >> (4u * (ch >> 1))) & 0x0f0f0f0fu;
            const float p0 = __fmul_rn(d, (float)(int)(wq & 0xffu) - 8.0f), p1 = __fmul_rn(d, (float)(int)((wq >> 8) & 0xffu) - 8.0f);
            const float p2 = __fmul_rn(d, (float)(int)((wq >> 16) & 0xffu) - 8.0f), p3 = __fmul_rn(d, (float)(int)(wq >> 24) - 8.0f);
            out[2 * i] = pack_h2(p0, p1);
            out[2 * i + 1] = pack_h2(p2, p3);
        }
        *reinterpret_cast<uint4 *>(dst_row_base + swz_off(r, 4u * half + ch)) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// 32 bytes at p, where p is CLS bytes (0, 2, 4 or 6) past an 8-byte boundary: four or five 64-bit loads and,
// for the odd classes, funnel shifts.  The decode of Q6_K is bound by the number of its global loads.
template <uint32_t CLS>
__device__ __forceinline__ void ldg_span32(const uint8_t *p, uint32_t *out) {
    const uint2 *q = reinterpret_cast<const uint2 *>(p - CLS);
    if (CLS == 0) {
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) { const uint2 v = q[i]; out[2 * i] = v.x; out[2 * i + 1] = v.y; }
        return;
    }
    uint32_t t[10];
#pragma unroll
    for (uint32_t i = 0; i < 5; ++i) { const uint2 v = q[i]; t[2 * i] = v.x; t[2 * i + 1] = v.y; }
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
        if (CLS == 4) out[i] = t[i + 1];
        else if (CLS == 2) out[i] = __funnelshift_r(t[i], t[i + 1], 16u);
        else out[i] = __funnelshift_r(t[i + 1], t[i + 2], 16u);
    }
}

// Q6_K: K step ks covers half n = (ks % 4) / 2 of block ks / 4 and quarters 2 (ks % 2) and 2 (ks % 2) + 1;
// this thread takes quarter q = 2 (ks % 2) + half: 32 columns, two runs of 16 with their own scale.
// Raw: 8 words of ql, 8 words of qh, the two scale bytes, d.
// rows4: every row starts on a 4-byte boundary (the stride is a multiple of 4).  A block is 210 bytes,
// so the words of even blocks are then aligned and those of odd blocks lie 2 bytes past a boundary —
// the same for every thread of the CTA: whole-word loads (and a funnel shift) instead of 16-bit ones.
// rows8: every row starts on an 8-byte boundary: block b then starts 2 b mod 8 bytes past one.
__device__ __forceinline__ void load32_q6k(const uint8_t *row, uint32_t ks, uint32_t half, bool rows4, bool rows8, GemmRaw &raw) {
    const uint8_t *b = row + (size_t)(ks >> 2) * 210u;
    const uint32_t n = (ks >> 1) & 1u, q = 2u * (ks & 1u) + half;
    const uint8_t *ql = b + 64u * n + 32u * (q & 1u), *qh = b + 128u + 32u * n;
    if (rows8) {
        switch ((ks >> 2) & 3u) {
        case 0: ldg_span32<0>(ql, raw.w); ldg_span32<0>(qh, raw.w + 8); break;
        case 1: ldg_span32<2>(ql, raw.w); ldg_span32<2>(qh, raw.w + 8); break;
        case 2: ldg_span32<4>(ql, raw.w); ldg_span32<4>(qh, raw.w + 8); break;
        default: ldg_span32<6>(ql, raw.w); ldg_span32<6>(qh, raw.w + 8); break;
        }
    } else if (!rows4) {
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) {
            raw.w[i] = ldg32_u2(ql + 4u * i);
            raw.w[8 + i] = ldg32_u2(qh + 4u * i);
        }
    } else if (((ks >> 2) & 1u) == 0u) {
        const uint32_t *l = reinterpret_cast<const uint32_t *>(ql), *h = reinterpret_cast<const uint32_t *>(qh);
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) { raw.w[i] = l[i]; raw.w[8 + i] = h[i]; }
    } else {
        const uint32_t *l = reinterpret_cast<const uint32_t *>(ql - 2), *h = reinterpret_cast<const uint32_t *>(qh - 2);
        uint32_t tl[9], th[9];
#pragma unroll
        for (uint32_t i = 0; i < 9; ++i) { tl[i] = l[i]; th[i] = h[i]; }
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) {
            raw.w[i] = __funnelshift_r(tl[i], tl[i + 1], 16u);
            raw.w[8 + i] = __funnelshift_r(th[i], th[i + 1], 16u);
        }
    }
    raw.w[16] = *reinterpret_cast<const unsigned short *>(b + 192u + 8u * n + 2u * q);
    raw.w[17] = *reinterpret_cast<const unsigned short *>(b + 208u);
}
__device__ __forceinline__ void emit32_q6k(const GemmRaw &raw, uint32_t ks, uint32_t half, uint8_t *dst_row_base, uint32_t r) {
    const uint32_t q = 2u * (ks & 1u) + half;
    const float d = __half2float(__ushort_as_half((unsigned short)raw.w[17]));
    const uint32_t lsh = q >= 2u ? 4u : 0u, hsh = 2u * q;
    const float ds0 = __fmul_rn(d, (float)(int)(int8_t)(raw.w[16] & 0xffu)), ds1 = __fmul_rn(d, (float)(int)(int8_t)(raw.w[16] >> 8));
#pragma unroll
    for (uint32_t ch = 0; ch < 4; ++ch) {           // columns 8 ch .. 8 ch + 7 of the quarter
        const float ds = ch < 2 ? ds0 : ds1;
        uint32_t out[4];
#pragma unroll
        for (uint32_t i = 0; i < 2; ++i) {
            const uint32_t lw = raw.w[2 * ch + i], hw = raw.w[8 + 2 * ch + i];
            const uint32_t v = ((lw >> lsh) & 0x0f0f0f0fu) | (((hw >> hsh) & 0x03030303u) << 4);     // four 6-bit values
            const float a0 = __fsub_rn(magic_byte(v, 0), MAGIC + 32.0f), a1 = __fsub_rn(magic_byte(v, 1), MAGIC + 32.0f);     // q - 32, exact
            const float a2 = __fsub_rn(magic_byte(v, 2), MAGIC + 32.0f), a3 = __fsub_rn(magic_byte(v, 3), MAGIC + 32.0f);
            out[2 * i] = pack_h2(__fmul_rn(ds, a0), __fmul_rn(ds, a1));
            out[2 * i + 1] = pack_h2(__fmul_rn(ds, a2), __fmul_rn(ds, a3));
        }
        *reinterpret_cast<uint4 *>(dst_row_base + swz_off(r, 4u * half + ch)) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

template <uint32_t NB>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_dequant_tcgen05_kernel(const __grid_constant__ CUtensorMap xmap,
                                                                               const __grid_constant__ GemmArgs a) {
    constexpr uint32_t A_STAGES = GemmShape<NB>::A_STAGES, B_STAGES = GemmShape<NB>::B_STAGES, B_STAGE_BYTES = GemmShape<NB>::B_STAGE_BYTES;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte aligned tiles (the swizzle pattern repeats every 1024 bytes)
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    uint64_t *full_a = reinterpret_cast<uint64_t *>(smem);          // [A_STAGES] decode warps -> MMA
    uint64_t *full_b = full_a + GEMM_MAX_STAGES;                      // [B_STAGES] copy thread -> MMA
    uint64_t *empty_a = full_b + GEMM_MAX_STAGES;                     // [A_STAGES] MMA -> decode warps
    uint64_t *empty_b = empty_a + GEMM_MAX_STAGES;                    // [B_STAGES] MMA -> copy thread
    uint64_t *acc_full = empty_b + GEMM_MAX_STAGES;                   // accumulator complete
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
    uint8_t *tiles_a = smem + 1024, *tiles_b = tiles_a + A_STAGES * GEMM_A_BYTES;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t n0 = blockIdx.x * GEMM_M, t0 = blockIdx.y * GEMM_N * NB;
    const uint32_t all_steps = a.cols / GEMM_K;
    const uint32_t ks0 = (uint32_t)((uint64_t)all_steps * blockIdx.z / gridDim.z);
    const uint32_t ksteps = (uint32_t)((uint64_t)all_steps * (blockIdx.z + 1) / gridDim.z) - ks0;      // this CTA's K steps
    float *const out = a.partial ? a.partial + (size_t)blockIdx.z * a.tokens * a.rows : a.y;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < GEMM_MAX_STAGES; ++s) {
            ptx::mbar_init(&full_a[s], GEMM_DECODE_THREADS);
            ptx::mbar_init(&full_b[s], 1);
            ptx::mbar_init(&empty_a[s], NB);          // one commit per MMA thread
            ptx::mbar_init(&empty_b[s], NB);
        }
        ptx::mbar_init(acc_full, NB);
        ptx::mbar_init_fence();
    }
    if (warp == GEMM_DECODE_WARPS + 1u) tmem_alloc(tmem_slot, GEMM_N * NB);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();

    bool failed = false;
    if (warp < GEMM_DECODE_WARPS) {
        // ---- decode warps: half a weight row (32 columns of the step) per thread; group `grp` takes
        // steps grp, grp + 2, ... ----
        const uint32_t r = threadIdx.x & 127u, half = (threadIdx.x >> 7) & 1u;   // row inside the tile = TMEM lane
        const uint32_t grp = threadIdx.x >> 8;
        const bool live = n0 + r < a.rows;
        const uint8_t *row = a.w + (size_t)(live ? n0 + r : 0) * a.stride;
        const bool q4k = a.kind == KIND_Q4_K, q40 = a.kind == KIND_Q4_0;
        const bool rows4 = (a.stride % 4u) == 0u, rows8 = (a.stride % 8u) == 0u;           // the weight base is 16-byte aligned
        GemmRaw cur = {}, nxt = {};
        auto load = [&](uint32_t ks, GemmRaw &raw) {
            if (q4k) load32_q4k(row, ks, raw);
            else if (q40) load32_q40(row, ks, half, raw);
            else load32_q6k(row, ks, half, rows4, rows8, raw);
        };
        if (live && grp < ksteps) load(ks0 + grp, cur);
        for (uint32_t ks = grp; ks < ksteps && !failed; ks += GEMM_DECODE_GROUPS) {
            const uint32_t s = ks % A_STAGES, ph = (ks / A_STAGES) & 1u;
            if (live && ks + GEMM_DECODE_GROUPS < ksteps) load(ks0 + ks + GEMM_DECODE_GROUPS, nxt);
            if (!ptx::mbar_wait_sleep<20>(&empty_a[s], ph ^ 1u)) { failed = true; break; }
            uint8_t *dst = tiles_a + (size_t)s * GEMM_A_BYTES;
            if (live) {
                if (q4k) emit32_q4k(cur, ks0 + ks, half, dst, r);
                else if (q40) emit32_q40(cur, half, dst, r);
                else emit32_q6k(cur, ks0 + ks, half, dst, r);
            } else {
#pragma unroll
                for (uint32_t c = 0; c < 4; ++c) *reinterpret_cast<uint4 *>(dst + swz_off(r, 4u * half + c)) = make_uint4(0, 0, 0, 0);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy stores -> tensor core reads
            ptx::mbar_arrive(&full_a[s]);
            cur = nxt;
        }
        // ---- epilogue: this warp reads TMEM lanes 32 * (warp % 4) .. + 31 and a quarter of the token columns ----
        if (!failed && !ptx::mbar_wait_sleep<64>(acc_full, 0)) failed = true;
        if (!failed) {
            tc_fence_after();
            const uint32_t rowg = n0 + r;
#pragma unroll 1
            constexpr uint32_t SLICE = GEMM_N * NB / (GEMM_DECODE_WARPS / 4u);
            for (uint32_t c0 = (warp >> 2) * SLICE; c0 < ((warp >> 2) + 1u) * SLICE; c0 += 32) {
                if (t0 + c0 >= a.tokens) break;
                float v[32];
                tmem_ld32(tmem_base + (((warp & 3u) * 32u) << 16) + c0, v);
                if (rowg < a.rows) {
#pragma unroll
                    for (uint32_t i = 0; i < 32; ++i) {
                        const uint32_t t = t0 + c0 + i;
                        if (t < a.tokens) out[(size_t)t * a.rows + rowg] = v[i];
                    }
                }
            }
        }
    } else if (warp == GEMM_DECODE_WARPS) {
        // ---- copy thread: 256 tokens x 64 columns of binary16 per stage, one TMA copy (rows past the last
        // token read as zero) ----
        if (lane == 0) {
            uint32_t issued = 0;
            for (uint32_t ks = 0; ks < ksteps && !failed; ++ks, ++issued) {
                const uint32_t s = ks % B_STAGES, ph = (ks / B_STAGES) & 1u;
                if (!ptx::mbar_wait_sleep<20>(&empty_b[s], ph ^ 1u)) { failed = true; break; }
                uint8_t *dst = tiles_b + (size_t)s * B_STAGE_BYTES;
                ptx::mbar_expect_tx(&full_b[s], NB * GEMM_B_BYTES);
#pragma unroll
                for (uint32_t nb = 0; nb < NB; ++nb)
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                        ::"r"(ptx::smem_addr(dst + nb * GEMM_B_BYTES)), "l"(&xmap), "r"((ks0 + ks) * GEMM_K), "r"(t0 + nb * GEMM_N),
                          "r"(ptx::smem_addr(&full_b[s]))
                        : "memory");
            }
            // no copy of this CTA may still be in flight when it leaves (the MMA thread has waited for
            // all of them unless a wait ran out): wait for the last copies of every stage, bounded
            for (uint32_t j = issued > B_STAGES ? issued - B_STAGES : 0u; j < issued; ++j)
                if (!ptx::mbar_wait_sleep<20>(&full_b[j % B_STAGES], (j / B_STAGES) & 1u)) failed = true;
        }
    } else if (lane == 0 && warp - (GEMM_DECODE_WARPS + 1u) < NB) {
        // ---- MMA thread of accumulator nb ----
        const uint32_t nb = warp - (GEMM_DECODE_WARPS + 1u);
        const uint32_t idesc = idesc_f16(GEMM_M, GEMM_N);
        for (uint32_t ks = 0; ks < ksteps && !failed; ++ks) {
            const uint32_t sa = ks % A_STAGES, sb = ks % B_STAGES;
            if (!ptx::mbar_wait_sleep<0>(&full_a[sa], (ks / A_STAGES) & 1u) || !ptx::mbar_wait_sleep<0>(&full_b[sb], (ks / B_STAGES) & 1u)) {
                failed = true;
                break;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // tiles were written through the generic proxy
            tc_fence_after();
            const uint32_t a_addr = ptx::smem_addr(tiles_a + (size_t)sa * GEMM_A_BYTES), b_addr = ptx::smem_addr(tiles_b + (size_t)sb * B_STAGE_BYTES);
#pragma unroll
            for (uint32_t k = 0; k < GEMM_K / 16u; ++k)
                tc_mma_f16(tmem_base + nb * GEMM_N, smem_desc_k128(a_addr + k * 32u), smem_desc_k128(b_addr + nb * GEMM_B_BYTES + k * 32u),
                           idesc, (ks | k) != 0u);
            tc_commit(&empty_a[sa]);                                  // frees the stages when these MMAs are done
            tc_commit(&empty_b[sb]);
        }
        tc_commit(acc_full);
        // after a wait that ran out nobody reads the accumulator: let the issued MMAs finish (bounded)
        // before tensor memory is freed
        if (failed) ptx::mbar_wait_sleep<64>(acc_full, 0);
    }
    if (failed && lane == 0) set_status_word(a.status, KERNEL_ERR_GEMM_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == GEMM_DECODE_WARPS + 1u) tmem_dealloc(tmem_base, GEMM_N * NB);
}

// ---- activations -> binary16 ------------------------------------------------------------

struct ToHalfArgs {
    const void *x;
    __half *y;
    uint64_t n;
    uint32_t bf16;
};

__global__ void __launch_bounds__(256) to_half_kernel(const __grid_constant__ ToHalfArgs a) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += (uint64_t)gridDim.x * blockDim.x)
        a.y[i] = __float2half_rn(load_x(a.x, i, a.bf16));
}

// ---- sum of the K splits ------------------------------------------------------------------

struct SplitSumArgs {
    const float *partial;      // [splits][n]
    float *y;
    uint64_t n;                // tokens * rows (a multiple of 4 is not required)
    uint32_t splits;
};

__global__ void __launch_bounds__(256) split_sum_kernel(const __grid_constant__ SplitSumArgs a) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += (uint64_t)gridDim.x * blockDim.x) {
        float s = a.partial[i];
        for (uint32_t z = 1; z < a.splits; ++z) s = __fadd_rn(s, a.partial[(uint64_t)z * a.n + i]);
        a.y[i] = s;
    }
}

// K splits for a grid of `ctas` tiles: whole extra waves only, at least 1024 columns per split.
static uint32_t gemm_splits(uint32_t cols, uint32_t rows, uint32_t tokens, uint32_t sm_count) {
    const uint32_t tok_tile = tokens > GEMM_N ? 2u * GEMM_N : GEMM_N;
    const uint32_t ctas = ((rows + GEMM_M - 1) / GEMM_M) * ((tokens + tok_tile - 1) / tok_tile);
    uint32_t splits = sm_count / (ctas ? ctas : 1u);
    const uint32_t by_k = cols / GEMM_K / 16u;
    if (splits > by_k) splits = by_k;
    if (splits > 8u) splits = 8u;
    return splits < 2u ? 1u : splits;
}

size_t gemm_scratch_bytes(uint32_t cols, uint32_t rows, uint32_t tokens, uint32_t sm_count) {
    const size_t xh = ((size_t)tokens * cols * 2u + 255u) & ~(size_t)255u;
    const uint32_t splits = gemm_splits(cols, rows, tokens, sm_count);
    return xh + (splits > 1 ? (size_t)splits * tokens * rows * 4u : 0u);
}

cudaError_t launch_gemm_dequant(const uint8_t *w, uint32_t cols, uint32_t rows, uint32_t stride, uint32_t kind, uint32_t expert,
                                const void *x, uint32_t x_bf16, uint32_t tokens, float *y, void *x_half_scratch,
                                const LaunchCtx &ctx) {
    if (kind != KIND_Q4_K && kind != KIND_Q6_K && kind != KIND_Q4_0) return cudaErrorNotSupported;
    if (cols % 256u || tokens == 0 || rows == 0) return cudaErrorInvalidValue;
    if (((uintptr_t)w % 16u) || (stride % 2u) || (kind == KIND_Q4_K && stride % 16u)) return cudaErrorNotSupported;
    ToHalfArgs h = {x, static_cast<__half *>(x_half_scratch), (uint64_t)tokens * cols, x_bf16};
    uint64_t blocks = (h.n + 255) / 256, cap = (uint64_t)ctx.sm_count * 16u;
    if (blocks > cap) blocks = cap;
    to_half_kernel<<<(uint32_t)blocks, 256, 0, ctx.stream>>>(h);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    static DeviceOnce once1, once2;
    e = once1.smem(gemm_dequant_tcgen05_kernel<1>, (int)GemmShape<1>::SMEM);
    if (e == cudaSuccess) e = once2.smem(gemm_dequant_tcgen05_kernel<2>, (int)GemmShape<2>::SMEM);
    if (e != cudaSuccess) return e;
    const uint32_t splits = gemm_splits(cols, rows, tokens, ctx.sm_count);
    float *partial = splits > 1 ? reinterpret_cast<float *>(static_cast<uint8_t *>(x_half_scratch) + (((size_t)tokens * cols * 2u + 255u) & ~(size_t)255u))
                                : nullptr;
    GemmArgs a = {w + (size_t)expert * rows * stride, static_cast<const __half *>(x_half_scratch), y, cols, rows, stride, kind, tokens,
                  ctx.status, partial};
    CUtensorMap xmap;
    if (((uintptr_t)x_half_scratch % 16u) ||
        !make_tensor_map_2d(xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x_half_scratch, cols, tokens, (uint64_t)cols * 2u, GEMM_K, GEMM_N,
                            CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorNotSupported;
    if (tokens > GEMM_N) {          // 512 tokens per decoded weight tile
        dim3 grid((rows + GEMM_M - 1) / GEMM_M, (tokens + 2u * GEMM_N - 1) / (2u * GEMM_N), splits);
        gemm_dequant_tcgen05_kernel<2><<<grid, GEMM_THREADS, GemmShape<2>::SMEM, ctx.stream>>>(xmap, a);
    } else {
        dim3 grid((rows + GEMM_M - 1) / GEMM_M, 1, splits);
        gemm_dequant_tcgen05_kernel<1><<<grid, GEMM_THREADS, GemmShape<1>::SMEM, ctx.stream>>>(xmap, a);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess || splits == 1) return e;
    SplitSumArgs sa = {partial, y, (uint64_t)tokens * rows, splits};
    uint64_t sblocks = (sa.n + 255) / 256;
    if (sblocks > cap) sblocks = cap;
    split_sum_kernel<<<(uint32_t)sblocks, 256, 0, ctx.stream>>>(sa);
    return cudaGetLastError();
}

}  // namespace ingot
