// Streaming GEMV whose inner products run on the tensor cores from registers.
//
// Why: on sm_100 an fp32 multiply-add per weight needs an integer extract, an
// int->float step and an FMA — at least 3.7 issued instructions per weight, with
// the half-rate integer pipe the first to saturate — which caps 4-bit formats
// near half of HBM bandwidth (measured; see the profile summaries).  Here a lane
// turns packed quants into binary16 operand registers with ONE logic op per TWO
// weights — masked in place, the bits of a quant are a subnormal binary16 whose
// value is the quant times 2^-24 (undone in the scale) — and a warp-level mma.sync
// m16n8k16 (f16 x f16 -> f32) multiplies 16 rows by 16 columns at once.  (The e4m3
// mma.sync, which would take four weights per register, is emulated on sm_100 by
// unpacking to binary16 — measured slower — so it is not used.)  Nothing is staged
// through shared memory in decoded form and the kernel stays a bandwidth-bound
// GEMV: one CTA streams a contiguous range of rows through a ring of bulk-copy
// stages, eight warps split the columns of each 16-row tile.
//
// Numerics: quants are small integers, exact in binary16.  An activation x is
// split into xh = f16(x) and xl = f16(x - xh) (two columns of the B operand), so
// q * x keeps 22 bits of x; products are exact and accumulate in fp32.  Scales
// are applied in fp32 outside the MMA, group by group, in the factored forms the
// reference's kernels use (kernels/iq3_mix.metal:104-123,
// kernels/decode.metal:66-83, kernels/generic.metal:242-269).
//
// One m16n8k16 covers 16 consecutive columns [16 mi, 16 mi + 16) of 16 rows.  For
// lane (g = lane / 4, t = lane % 4):
//   A (rows x k): a0 = row g,   k {2t, 2t+1};   a1 = row g+8, same k;
//                 a2 = row g,   k {2t+8, 2t+9}; a3 = row g+8, same k
//   B (k x n):    b0 = k {2t, 2t+1}, n = g;     b1 = k {2t+8, 2t+9}, n = g
//   C (rows x n): c0,c1 = row g, n {2t, 2t+1};  c2,c3 = row g+8, same n
// Lane t supplies columns 16 mi + 4t .. +3 from ONE 32-bit word of quants: bytes
// (0,2) form one operand register and bytes (1,3) the other, i.e. k slots
// {2t, 2t+1, 2t+8, 2t+9} = bytes {0, 2, 1, 3}.  Activations are pre-packed to
// match (pack_x_kernel): [mi][part: xh, xl][t][4 halves].  Even columns n carry xh
// and odd ones xl, replicated over the quads, so every lane ends with (sum q xh,
// sum q xl) in (c0, c1) and the four lanes of a quad share the scale work.
#include <cuda_fp16.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <type_traits>
#include <vector>

#include "dev_common.cuh"
#include "gemv_core.cuh"
#include "kernels.h"
#include "pack.cuh"
#include "ptx.cuh"
#include "tensor_map.h"

namespace ingot {

static constexpr int MMA_WARPS = 8;                       // consumer warps
static constexpr int MMA_THREADS = (MMA_WARPS + 1) * 32;  // + producer warp
static constexpr uint32_t MMA_SMEM_BUDGET = 112u * 1024u; // two CTAs per SM
static constexpr uint32_t MMA_SMEM_SMALL = 74u * 1024u;   // three CTAs per SM
static constexpr uint32_t MMA_SMEM_MAX = 224u * 1024u;
static constexpr uint32_t MMA_STAGE_TARGET = 24u * 1024u;
static constexpr int MMA_MAX_STAGES = 6;                  // barriers: full[6], empty[6], x, tile[8] (<= 128 bytes... 21 x 8)
static constexpr uint32_t MMA_RED_SLOTS = 8;              // > MMA_MAX_STAGES: a warp is never that many tiles ahead
static constexpr uint32_t MMA_ZERO_BYTES = 1024;          // B operands of one step, all zero
static constexpr uint32_t MMA_BAR_BYTES = 256;

struct MmaPlan {
    uint32_t kind, cols, rows, stride, nmat;
    uint32_t step_cols;      // columns one warp handles per step (format dependent)
    uint32_t step_bytes;     // bytes of a row in one step
    uint32_t nsteps;         // cols / step_cols
    uint32_t kw_log2;        // warps splitting K: 1 << kw_log2
    uint32_t row_tiles;      // 16-row tiles per stage = 8 >> kw_log2
    uint32_t spw;            // steps per warp per chunk
    uint32_t chunks, chunk_bytes;
    uint32_t row_pitch;      // bytes between rows inside a stage (16 mod 128: conflict-free word loads)
    uint32_t stages, stage_bytes;
    uint32_t x_bytes;        // packed activations of one token
    uint32_t red_bytes, smem_bytes;
    uint32_t ctas;
    uint32_t red_slots;      // ring of partial-sum buffers, > stages
    uint32_t xm;             // form of the activation row in shared memory (XM_*)
    uint32_t x_row_stride;   // bytes between activation rows when several are held (tiles of one expert)
};

// Activation row forms.  The binary16 forms are what ingot_pack_x / ingot_pack_x_hi write; the
// fixed-point forms are built by the CTA itself (fused norm, or plain float32 rows) and feed the int8 MMA.
enum : uint32_t {
    XM_F16 = 0,      // binary16 (high, low) parts
    XM_F16_HI = 1,   // binary16 high part only (bfloat16 activations are exact in it)
    XM_FX2 = 2,      // fixed point, two base-256 digits per activation (bfloat16-rounded activations)
    XM_FX4 = 3       // fixed point, four digits (float32 activations)
};
static uint32_t x_row_bytes(uint32_t xm, uint32_t cols) {
    return xm == XM_F16 ? packed_x_bytes(cols) : xm == XM_F16_HI ? packed_hi_bytes(cols) : fx_row_bytes(cols, xm == XM_FX2 ? 2u : 4u);
}

struct MmaArgs {
    MmaPlan plan;
    const uint8_t *w[2];
    const uint8_t *xp;        // packed activations [row][packed_x_bytes(cols)]
    float *y;
    const uint32_t *ids;
    uint32_t expert, n_experts, per_pair, top, glu;
    int *status;
    // optional fused normalisation of the activations (dense, one token): x = rms_norm(na + nb) * nw
    // computed by every CTA into its own packed row instead of fetching one; CTA 0 stores the sum
    const float *na, *nb, *nw;
    float *ns;
    float neps;
    uint32_t nround_bf16;
    // npack: na holds plain float32 activation rows (row `pair / top` or `pair` of a routed call) that
    // the CTA only packs — no sum, no norm, no rounding: the packing launch folded into the GEMV
    uint32_t npack;
    // optional tensor maps (device memory) of the matrices as rows of 8-byte elements, in boxes of
    // (row_pitch / 8) x (16 row_tiles): a stage then arrives by one tiled copy instead of one copy per row
    const void *tmap[2];
    // row shards over several GPUs (tensor parallel): the results are also stored into the same place of
    // every peer's window, then every CTA raises a counter on every rank; a projection whose inputs are
    // assembled that way waits, with a time limit, until its own counters have reached step x arrivals
    TpLink tp;
};

static bool mma_kind(uint32_t kind) { return kind == KIND_Q4_K || kind == KIND_Q6_K || kind == KIND_Q4_0 || kind == KIND_Q8_0; }

static void step_geometry(uint32_t kind, uint32_t &cols, uint32_t &bytes) {
    switch (kind) {
    case KIND_Q4_K: cols = 256; bytes = 144; break;
    case KIND_Q6_K: cols = 256; bytes = 210; break;
    case KIND_Q4_0: cols = 128; bytes = 72; break;
    default: cols = 128; bytes = 136; break;     // Q8_0
    }
}

// Row pitch inside a stage: `lead` mod 128, so that the loads of one instruction hit different banks
// (16: eight rows x 4 lanes x 4 bytes; 32: four rows x 4 lanes x 8 bytes per half-warp of a 64-bit load).
static uint32_t pitch_of(uint32_t chunk_bytes, uint32_t lead = 16u) { return chunk_bytes + ((lead + 128u - (chunk_bytes % 128u)) % 128u); }

// Shared-memory geometry that several projections of one kernel have in common: the region of the
// activation row, and a ring of `slots` stages of `slot_bytes` each.
struct MmaFixed {
    uint32_t x_bytes, slot_bytes, slots;
    uint32_t warps;          // consumer warps of the kernel (8 or 16)
};
static constexpr uint32_t MMA_TILE_TOKENS = 4;      // pairs of one expert multiplied per pass over its rows

static bool plan_mma(uint32_t kind, uint32_t cols, uint32_t rows, uint32_t stride, uint32_t nmat, uint32_t max_ctas,
                     uint32_t budget, uint32_t xm, MmaPlan &p, const MmaFixed *common = nullptr, uint32_t tokens = 1,
                     uint32_t x_rows = 0) {
    if (!mma_kind(kind)) return false;
    uint32_t block, bytes;
    geometry(kind, block, bytes);
    if (cols == 0 || rows == 0 || cols % block || stride != cols / block * bytes) return false;
    step_geometry(kind, p.step_cols, p.step_bytes);
    if (cols % p.step_cols || stride % 16u) return false;
    p.kind = kind; p.cols = cols; p.rows = rows; p.stride = stride; p.nmat = nmat;
    p.nsteps = cols / p.step_cols;
    uint32_t kw = 3;
    while (kw > 0 && (p.nsteps % (1u << kw))) --kw;
    p.kw_log2 = kw;
    p.row_tiles = (uint32_t)MMA_WARPS >> kw;
    const uint32_t per_warp = p.nsteps >> kw;                 // steps each warp owns per row
    p.xm = xm;
    p.x_row_stride = (x_row_bytes(xm, cols) + 15u) & ~15u;
    // (a multi-token kernel keeps `tokens` partial sums per row; x_rows of them, all by default, have their
    // activation rows resident at a time)
    p.x_bytes = common ? common->x_bytes : tokens > 1 ? (x_rows ? x_rows : tokens) * p.x_row_stride : x_row_bytes(xm, cols);
    if (common && x_row_bytes(xm, cols) > common->x_bytes) return false;
    // the int8 steps of the K-quants read 8 bytes per lane
    const uint32_t lead = (xm >= XM_FX2 && (kind == KIND_Q4_K || kind == KIND_Q6_K)) ? 32u : 16u;
    p.red_slots = (budget <= MMA_SMEM_SMALL || tokens > 1) ? 4u : MMA_RED_SLOTS;
    p.red_bytes = p.red_slots * MMA_WARPS * tokens * 2u * 16u * 4u + MMA_ZERO_BYTES;   // [slot][warp][token][mat][row] + zeros
    const uint32_t fixed = MMA_BAR_BYTES + ((p.x_bytes + 127u) & ~127u) + p.red_bytes;
    if (fixed >= budget) return false;
    // chunk = the most steps per warp whose stage stays near the target, leaves at least
    // two stages, and keeps every copy 16-byte aligned
    const uint32_t room = budget - fixed;
    uint32_t pick = 0;
    for (uint32_t spw = 1; spw <= per_warp; ++spw) {
        if (per_warp % spw) continue;
        const uint32_t cb = spw * (1u << kw) * p.step_bytes;
        if (cb % 16u) continue;
        const uint32_t sb = (pitch_of(cb, lead) * 16u * p.row_tiles + 64u + 127u) & ~127u;      // one matrix per stage
        if (common) {                                 // the most steps whose stage fits a slot
            if (sb <= common->slot_bytes) pick = spw;
            continue;
        }
        if (room / sb < 2) break;
        if (pick == 0 || sb <= MMA_STAGE_TARGET) pick = spw;
    }
    if (pick == 0) return false;
    p.spw = pick;
    p.chunks = per_warp / pick;
    p.chunk_bytes = pick * (1u << kw) * p.step_bytes;
    p.row_pitch = pitch_of(p.chunk_bytes, lead);
    p.stage_bytes = (p.row_pitch * 16u * p.row_tiles + 64u + 127u) & ~127u;
    p.stages = room / p.stage_bytes;
    if (common) {
        p.stage_bytes = common->slot_bytes;
        p.stages = common->slots;
        if ((uint64_t)p.stages * p.stage_bytes > room) return false;
    }
    if (p.stages > (uint32_t)MMA_MAX_STAGES) p.stages = MMA_MAX_STAGES;
    if (p.stages > p.red_slots - 2u) p.stages = p.red_slots - 2u;
    if (p.stages < 2) return false;
    p.smem_bytes = fixed + p.stages * p.stage_bytes;
    const uint32_t want = (rows + 7u) / 8u;
    p.ctas = want < max_ctas ? want : max_ctas;
    if (p.ctas == 0) p.ctas = 1;
    return true;
}

// ---------------------------------------------------------------------------
// Packing activations into the B-operand order.  One CTA per activation row.
// Packed row: [cols/16 MMAs][2 parts][4 lanes][4 halves] | cols/16 fp32 sums of
// each 16 (scaled) activations | 16 bytes: 1/scale.  x is pre-multiplied by a
// power of two when its magnitude would overflow binary16.
// ---------------------------------------------------------------------------

struct PackArgs {
    const void *x;
    uint8_t *out;
    uint32_t cols, bf16;
    uint32_t hi;             // high-part rows (x holds bfloat16 values)
};

__global__ void __launch_bounds__(256) pack_x_kernel(const __grid_constant__ PackArgs a) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    __shared__ float part_max[8];
    const uint32_t tid = threadIdx.x;
    const size_t base = (size_t)blockIdx.x * a.cols;
    uint8_t *row = a.out + (size_t)blockIdx.x * (a.hi ? packed_hi_bytes(a.cols) : packed_x_bytes(a.cols));
    float mx = 0.f;
    for (uint32_t c = tid; c < a.cols; c += 256) mx = fmaxf(mx, fabsf(load_x(a.x, base + c, a.bf16)));
    for (uint32_t off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if ((tid & 31u) == 0) part_max[tid >> 5] = mx;
    __syncthreads();
    mx = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) mx = fmaxf(mx, part_max[i]);
    const float scale = pack_scale(mx);
    // one thread per 4 consecutive columns = one lane's word of one MMA; every thread
    // runs the same number of rounds so the quad shuffles always have all lanes
    const uint32_t n4 = a.cols / 4u;
    for (uint32_t q0 = 0; q0 < n4; q0 += 256) {
        const uint32_t q = q0 + tid;
        const bool live = q < n4;
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = live ? load_x(a.x, base + 4u * q + i, a.bf16) * scale : 0.f;
        if (a.hi) pack_hi_store_quad(row, a.cols, q, v, live);
        else pack_store_quad(row, a.cols, q, v, live);
    }
    if (tid == 0) { if (a.hi) pack_hi_store_unscale(row, a.cols, scale); else pack_store_unscale(row, a.cols, scale); }
}

static cudaError_t launch_pack_args(const PackArgs &a, uint32_t rows, const LaunchCtx &ctx);

cudaError_t launch_pack_x(const void *x, uint32_t bf16, uint32_t rows, uint32_t cols, void *packed, const LaunchCtx &ctx) {
    if (rows == 0) return cudaSuccess;
    if (cols % 64u) return cudaErrorInvalidValue;
    PackArgs a = {x, static_cast<uint8_t *>(packed), cols, bf16, 0};
    return launch_pack_args(a, rows, ctx);
}

cudaError_t launch_pack_x_hi(const void *x_bf16, uint32_t rows, uint32_t cols, void *packed, const LaunchCtx &ctx) {
    if (rows == 0) return cudaSuccess;
    if (cols % 64u) return cudaErrorInvalidValue;
    PackArgs a = {x_bf16, static_cast<uint8_t *>(packed), cols, 1, 1};
    return launch_pack_args(a, rows, ctx);
}

static cudaError_t launch_pack_args(const PackArgs &a, uint32_t rows, const LaunchCtx &ctx) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, pack_x_kernel, a);
}

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// d = A B (accumulator starts at zero without zeroing registers first)
__device__ __forceinline__ void mma16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// two binary16 magic numbers (bias + v) -> the two integers v, exactly
template <unsigned short BIAS_BITS>
__device__ __forceinline__ uint32_t unmagic(uint32_t h2) {
    const __half2 r = __hsub2(*reinterpret_cast<const __half2 *>(&h2), __half2half2(__ushort_as_half(BIAS_BITS)));
    return *reinterpret_cast<const uint32_t *>(&r);
}

// 32-bit word at a shared address that is known to be 4-byte aligned (`mis` false) or 2 bytes past
// such an address (`mis` true).  With `mis` a compile-time constant after inlining this is one
// load, or two loads and a funnel shift, with no address arithmetic.
__device__ __forceinline__ uint32_t lds32_known(const uint8_t *p, bool mis) {
    if (!mis) return *reinterpret_cast<const uint32_t *>(p);
    const uint32_t *q = reinterpret_cast<const uint32_t *>(p - 2);
    return __funnelshift_r(q[0], q[1], 16u);
}
__device__ __forceinline__ uint32_t lds32(const uint8_t *p) { return *reinterpret_cast<const uint32_t *>(p); }
__device__ __forceinline__ float lds_half(const uint8_t *p) { return __half2float(*reinterpret_cast<const __half *>(p)); }
__device__ __forceinline__ uint32_t lds16(const uint8_t *p) { return *reinterpret_cast<const unsigned short *>(p); }

// ---------------------------------------------------------------------------
// per-format warp steps.  r0 / r1: the step's bytes of rows g and g+8 in shared
// memory; xf: B operands of the step's first MMA; sx: its 16-column sums.
// (acc0, acc1): this lane's share of rows g and g+8 (summed over the quad later).
// ---------------------------------------------------------------------------

// xb[grp]: this lane's B-operand pointer for scale group `grp` of the step — the real
// packed activations when the lane's quad position owns that group, else a block of
// zeros.  A group's MMAs therefore add to the accumulator only in the lane that owns
// it, so all groups of a step chain into the same accumulator registers and each lane
// applies its own group's scale once, without selects.
#define IG_BFRAG(grp, mi) (*reinterpret_cast<const uint2 *>(xb[grp] + (mi) * XS))
// A binary16 whose exponent field is zero is subnormal: its value is mantissa * 2^-24,
// exactly, with no implicit one.  So the masked quant bits ARE the operand (times
// 2^-24, undone in the scale); no bias to subtract.  The tensor cores take binary16
// subnormals at full rate.
#define IG_LO(w) ((w) & 0x000f000fu)
#define IG_HI(w) ((w) & 0x00f000f0u)     /* 16 * nibble */
static constexpr float SUBNORMAL_SCALE = 16777216.0f;       // 2^24

template <uint32_t KIND> struct MmaStep;

// Q4_K: 256 columns = 4 groups j of 64: 32 bytes whose low nibbles are sub-block 2j
// and high nibbles sub-block 2j+1.  Lane t owns group j = t: its low-nibble MMAs
// (4j, 4j+1) and high-nibble MMAs (4j+2, 4j+3).
template <> struct MmaStep<KIND_Q4_K> {
    // (d * sc_2t, d * sc_2t+1 / 16, dmin * m_2t, dmin * m_2t+1) of group j = t of one row's block
    static __device__ __forceinline__ void scales(const uint8_t *r, uint32_t t, float &dsc0, float &dsc1, float &dm0, float &dm1) {
        const U4 hdr = *reinterpret_cast<const U4 *>(r);
        const uint32_t sh = (t & 1u) * 16u;
        const uint32_t a = hdr.y >> sh, bb = hdr.z >> sh, c = hdr.w >> sh;
        uint32_t sc, m;
        if (t < 2) { sc = a & 0x3f3fu; m = bb & 0x3f3fu; }
        else { sc = (c & 0x0f0fu) | ((a >> 2) & 0x3030u); m = ((c >> 4) & 0x0f0fu) | ((bb >> 2) & 0x3030u); }
        const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));      // (d, dmin)
        dsc0 = mul_rn(mul_rn(dd.x, (float)(sc & 0xffu)), SUBNORMAL_SCALE);
        dsc1 = mul_rn(mul_rn(dd.x, (float)(sc >> 8)), SUBNORMAL_SCALE * 0.0625f);
        dm0 = mul_rn(dd.y, (float)(m & 0xffu));
        dm1 = mul_rn(dd.y, (float)(m >> 8));
    }
    template <uint32_t XS>      // bytes of packed activations per MMA: 64 (high and low parts) or 32 (high part only)
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, const uint8_t *const (&xb)[4], const float *sx,
                                               uint32_t t, float &acc0, float &acc1, bool) {
        float s00, s01, m00, m01, s10, s11, m10, m11;
        scales(r0, t, s00, s01, m00, m01);
        scales(r1, t, s10, s11, m10, m11);
        const uint8_t *q0 = r0 + 16u + 4u * t, *q1 = r1 + 16u + 4u * t;
        float lo[4], hi[4];
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j)
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h) {
                const uint32_t a = lds32(q0 + 32u * j + 16u * h), b = lds32(q1 + 32u * j + 16u * h);
                const uint32_t as = a >> 8, bs = b >> 8;
                const uint2 bl = IG_BFRAG(j, 4u * j + h), bh = IG_BFRAG(j, 4u * j + 2u + h);
                if (j == 0 && h == 0) {
                    mma16816_first(lo, IG_LO(a), IG_LO(b), IG_LO(as), IG_LO(bs), bl.x, bl.y);
                    mma16816_first(hi, IG_HI(a), IG_HI(b), IG_HI(as), IG_HI(bs), bh.x, bh.y);
                } else {
                    mma16816(lo, IG_LO(a), IG_LO(b), IG_LO(as), IG_LO(bs), bl.x, bl.y);
                    mma16816(hi, IG_HI(a), IG_HI(b), IG_HI(as), IG_HI(bs), bh.x, bh.y);
                }
            }
        // - dmin * (m_2t * sum x over sub-block 2t + m_2t+1 * sum x over sub-block 2t+1)
        const float4 sq = *reinterpret_cast<const float4 *>(sx + 4u * t);
        const float sa = add_rn(sq.x, sq.y), sb = add_rn(sq.z, sq.w);
        acc0 = add_rn(acc0, sub_rn(fma_rn(s01, add_rn(hi[0], hi[1]), mul_rn(s00, add_rn(lo[0], lo[1]))),
                                   fma_rn(m01, sb, mul_rn(m00, sa))));
        acc1 = add_rn(acc1, sub_rn(fma_rn(s11, add_rn(hi[2], hi[3]), mul_rn(s10, add_rn(lo[2], lo[3]))),
                                   fma_rn(m11, sb, mul_rn(m10, sa))));
    }
};

// Q6_K: 256 columns = 2 halves n of 128 = 4 quarters q of 32 = 2 runs h of 16, each
// run with its own int8 scale (index 8n + 2q + h).  A run's 6-bit values come from
// a word of ql (low nibble for q < 2, high nibble — kept in place, times 16 — for
// q >= 2; ql + 32 for odd q) and two bits of a word of qh.  Lane t owns quarter
// q = t.  Blocks are only 2-byte aligned.
template <> struct MmaStep<KIND_Q6_K> {
    template <int Q>
    static __device__ __forceinline__ uint32_t six(uint32_t L, uint32_t H) {       // bytes (0,2) of the words
        constexpr uint32_t nib = (Q >= 2) ? 0x00f000f0u : 0x000f000fu;
        constexpr uint32_t hmask = 0x00030003u << (2 * Q);
        constexpr uint32_t mult = (Q == 0 || Q == 2) ? 16u : 4u;                 // two high bits to bit 4 (q < 2) or 8
        return (L & nib) | ((H & hmask) * mult);            // subnormal binary16 pair: value * 2^-24
    }
    template <int Q, bool FIRST>
    static __device__ __forceinline__ void quarter(uint32_t la, uint32_t lb, uint32_t ha, uint32_t hb, uint2 bf, float (&c)[4]) {
        if (FIRST) mma16816_first(c, six<Q>(la, ha), six<Q>(lb, hb), six<Q>(la >> 8, ha >> 8), six<Q>(lb >> 8, hb >> 8), bf.x, bf.y);
        else mma16816(c, six<Q>(la, ha), six<Q>(lb, hb), six<Q>(la >> 8, ha >> 8), six<Q>(lb >> 8, hb >> 8), bf.x, bf.y);
    }
    // mis: the block starts 2 bytes past a 4-byte boundary (odd blocks of a 16-byte aligned row)
    template <uint32_t XS>      // bytes of packed activations per MMA: 64 (high and low parts) or 32 (high part only)
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, const uint8_t *const (&xb)[4], const float *sx,
                                               uint32_t t, float &acc0, float &acc1, bool mis) {
        const float d0 = lds_half(r0 + 208u), d1 = lds_half(r1 + 208u);
        const float up = t < 2 ? SUBNORMAL_SCALE : SUBNORMAL_SCALE * 0.0625f;       // x16 of the in-place high nibble undone
        float t0 = 0.f, t1 = 0.f;
#pragma unroll
        for (uint32_t n = 0; n < 2; ++n) {
            // scales of quarter q = t: runs h = 0, 1 are consecutive bytes 8n + 2t, 8n + 2t + 1
            const uint32_t s0 = lds16(r0 + 192u + 8u * n + 2u * t), s1 = lds16(r1 + 192u + 8u * n + 2u * t);
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h) {
                const uint32_t o = 64u * n + 16u * h + 4u * t;
                const uint32_t oh = 128u + 32u * n + 16u * h + 4u * t;
                const uint32_t a_lo = lds32_known(r0 + o, mis), a_hi = lds32_known(r0 + o + 32u, mis), a_h = lds32_known(r0 + oh, mis);
                const uint32_t b_lo = lds32_known(r1 + o, mis), b_hi = lds32_known(r1 + o + 32u, mis), b_h = lds32_known(r1 + oh, mis);
                float c[4];
                quarter<0, true>(a_lo, b_lo, a_h, b_h, IG_BFRAG(0, 8u * n + 0u + h), c);
                quarter<1, false>(a_hi, b_hi, a_h, b_h, IG_BFRAG(1, 8u * n + 2u + h), c);
                quarter<2, false>(a_lo, b_lo, a_h, b_h, IG_BFRAG(2, 8u * n + 4u + h), c);
                quarter<3, false>(a_hi, b_hi, a_h, b_h, IG_BFRAG(3, 8u * n + 6u + h), c);
                // value - 32 through the run's activation sum
                const float sc0 = (float)(int)(int8_t)((s0 >> (8u * h)) & 0xffu), sc1 = (float)(int)(int8_t)((s1 >> (8u * h)) & 0xffu);
                const float sxv = mul_rn(sx[8u * n + 2u * t + h], -32.0f);
                t0 = fma_rn(sc0, fma_rn(add_rn(c[0], c[1]), up, sxv), t0);
                t1 = fma_rn(sc1, fma_rn(add_rn(c[2], c[3]), up, sxv), t1);
            }
        }
        acc0 = fma_rn(d0, t0, acc0);
        acc1 = fma_rn(d1, t1, acc1);
    }
};

// Q4_0: step = 4 blocks of 32 (18 bytes each, 2-byte aligned): MMA 2b is the block's
// low nibbles (elements 0..15), MMA 2b+1 its high nibbles (16..31).  Lane t owns
// block b = t.
template <> struct MmaStep<KIND_Q4_0> {
    template <uint32_t XS>      // bytes of packed activations per MMA: 64 (high and low parts) or 32 (high part only)
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, const uint8_t *const (&xb)[4], const float *sx,
                                               uint32_t t, float &acc0, float &acc1, bool) {
        const float d0 = lds_half(r0 + 18u * t), d1 = lds_half(r1 + 18u * t);
        const float sxv = mul_rn(add_rn(sx[2u * t], sx[2u * t + 1u]), -8.0f);
        float lo[4], hi[4];
#pragma unroll
        for (uint32_t b = 0; b < 4; ++b) {
            // a step (72 bytes) starts on a 4-byte boundary: the quants of even blocks lie 2 bytes past one
            const uint32_t wa = lds32_known(r0 + 18u * b + 2u + 4u * t, (b & 1u) == 0u), wb = lds32_known(r1 + 18u * b + 2u + 4u * t, (b & 1u) == 0u);
            const uint32_t as = wa >> 8, bs = wb >> 8;
            const uint2 bl = IG_BFRAG(b, 2u * b), bh = IG_BFRAG(b, 2u * b + 1u);
            if (b == 0) {
                mma16816_first(lo, IG_LO(wa), IG_LO(wb), IG_LO(as), IG_LO(bs), bl.x, bl.y);
                mma16816_first(hi, IG_HI(wa), IG_HI(wb), IG_HI(as), IG_HI(bs), bh.x, bh.y);
            } else {
                mma16816(lo, IG_LO(wa), IG_LO(wb), IG_LO(as), IG_LO(bs), bl.x, bl.y);
                mma16816(hi, IG_HI(wa), IG_HI(wb), IG_HI(as), IG_HI(bs), bh.x, bh.y);
            }
        }
        const float q0 = mul_rn(fma_rn(add_rn(hi[0], hi[1]), 0.0625f, add_rn(lo[0], lo[1])), SUBNORMAL_SCALE);
        const float q1 = mul_rn(fma_rn(add_rn(hi[2], hi[3]), 0.0625f, add_rn(lo[2], lo[3])), SUBNORMAL_SCALE);
        acc0 = fma_rn(d0, add_rn(q0, sxv), acc0);
        acc1 = fma_rn(d1, add_rn(q1, sxv), acc1);
    }
};

// Q8_0: step = 4 blocks of 32 int8 (34 bytes each, 2-byte aligned): MMAs 2b and 2b+1.
// Lane t owns block b = t.  A byte b becomes (b + 128) * 2^-24; the 128 comes off
// through the block's activation sum.
template <> struct MmaStep<KIND_Q8_0> {
    static __device__ __forceinline__ uint32_t s8(uint32_t w) { return (w & 0x00ff00ffu) ^ 0x00800080u; }
    template <uint32_t XS>      // bytes of packed activations per MMA: 64 (high and low parts) or 32 (high part only)
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, const uint8_t *const (&xb)[4], const float *sx,
                                               uint32_t t, float &acc0, float &acc1, bool) {
        const float d0 = lds_half(r0 + 34u * t), d1 = lds_half(r1 + 34u * t);
        const float sxv = mul_rn(add_rn(sx[2u * t], sx[2u * t + 1u]), -128.0f);
        float c[4];
#pragma unroll
        for (uint32_t b = 0; b < 4; ++b)
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h) {
                // a step (136 bytes) starts on a 4-byte boundary: the quants of even blocks lie 2 bytes past one
                const uint32_t wa = lds32_known(r0 + 34u * b + 2u + 16u * h + 4u * t, (b & 1u) == 0u);
                const uint32_t wb = lds32_known(r1 + 34u * b + 2u + 16u * h + 4u * t, (b & 1u) == 0u);
                const uint2 bf = IG_BFRAG(b, 2u * b + h);
                if (b == 0 && h == 0) mma16816_first(c, s8(wa), s8(wb), s8(wa >> 8), s8(wb >> 8), bf.x, bf.y);
                else mma16816(c, s8(wa), s8(wb), s8(wa >> 8), s8(wb >> 8), bf.x, bf.y);
            }
        acc0 = fma_rn(d0, fma_rn(add_rn(c[0], c[1]), SUBNORMAL_SCALE, sxv), acc0);
        acc1 = fma_rn(d1, fma_rn(add_rn(c[2], c[3]), SUBNORMAL_SCALE, sxv), acc1);
    }
};

#undef IG_BFRAG
#undef IG_LO
#undef IG_HI

// ---------------------------------------------------------------------------
// int8 steps: mma.sync m16n8k32 (u8 or s8 weights x s8 activation digits -> s32) on fixed-point
// activation rows (pack.cuh: fx_store).  One MMA covers one sub-block of 32 columns of 16 rows:
//   A (rows x k): a0 = row g, k 4t..4t+3;  a1 = row g+8, same k;  a2 = row g, k 16+4t..;  a3 = row g+8
//   B (k x n):    b0 = k 4t..4t+3, n = g;  b1 = k 16+4t.., n = g
//   C (rows x n): c0, c1 = row g, n 2t, 2t+1;  c2, c3 = row g+8, same n
// A nibble mask turns four packed quants into four operand bytes with one logic op, twice as many
// weights per operand register as binary16 takes and half as many MMAs.  The eight B columns are
// (position in the chain, digit) pairs: a lane supplies digits only at the chain position it owns
// and zeros elsewhere, so the MMAs of a chain add into the same accumulator registers and lane t
// ends with the exact integer sums of the sub-block it owns, one per digit.  Digits recombine in
// integers (256 c0 + c1), the sub-block's power-of-two scale and the format's scales apply in fp32.
// Two digits make one pass; float32 activations take a second pass over the same A registers with
// digits 2 and 3.
// ---------------------------------------------------------------------------

template <bool SIGNED_A, bool FIRST>
__device__ __forceinline__ void imma16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    if (FIRST) {
        if (SIGNED_A)
            asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
        else
            asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    } else {
        if (SIGNED_A)
            asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
        else
            asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

// The exact digit sums of one row as a float: element i (row g) or i + 2 (row g+8) of the accumulators.
template <int NP>
__device__ __forceinline__ float fx_sum(const int (&c)[NP][4], int i) {
    const float hi = (float)(c[0][i] * 256 + c[0][i + 1]);
    if (NP == 1) return hi;
    return fma_rn(hi, 65536.0f, (float)(c[NP - 1][i] * 256 + c[NP - 1][i + 1]));
}

#define IG_B8(ptr) (*reinterpret_cast<const uint2 *>(ptr))
static constexpr uint32_t NIB = 0x0f0f0f0fu;

template <uint32_t KIND> struct ImmaStep;

// Q4_K.  Chain X = sub-blocks 0..3 of the block, chain Y = sub-blocks 4..7; the 32 quant bytes of
// chunk c hold sub-block 2c in their low nibbles and 2c+1 in their high nibbles (kept in place as
// 16 q; the factor comes off in the scale of the lanes that own odd sub-blocks).  Lane t owns
// sub-blocks t and t+4: their six-bit scales and mins are bytes t, t+4 and t+8 of the 12 scale bytes.
template <> struct ImmaStep<KIND_Q4_K> {
    static constexpr uint32_t POS_STRIDE = 1;        // chain position p reads sub-block p (+ 4 in chain Y)
    static __device__ __forceinline__ void scales(const uint8_t *r, uint32_t sel, float &d, float &dmin, float &sa, float &sb, float &ma,
                                                  float &mb) {
        const U4 hdr = *reinterpret_cast<const U4 *>(r);
        const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
        d = dd.x; dmin = dd.y;
        const uint32_t a = __byte_perm(hdr.y, 0u, sel), b = __byte_perm(hdr.z, 0u, sel), c = __byte_perm(hdr.w, 0u, sel);
        sa = (float)(a & 63u);
        ma = (float)(b & 63u);
        sb = (float)((c & 15u) | ((a >> 2) & 0x30u));
        mb = (float)((c >> 4) | ((b >> 2) & 0x30u));
    }
    template <int ND>
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, const uint8_t *const (&bx)[4], const uint8_t *meta,
                                               uint32_t t, float nibf, float &acc0, float &acc1, uint32_t) {
        constexpr uint32_t SBS = ND * 32u;
        constexpr int NP = ND / 2;
        int cx[NP][4], cy[NP][4];
        const uint8_t *q0 = r0 + 16u + 8u * t, *q1 = r1 + 16u + 8u * t;
#pragma unroll
        for (uint32_t c = 0; c < 4; ++c) {
            const uint2 wa = IG_B8(q0 + 32u * c), wb = IG_B8(q1 + 32u * c);
            const uint32_t p = 2u * (c & 1u), off = (c >> 1) * 4u * SBS;
#pragma unroll
            for (int ps = 0; ps < NP; ++ps) {
                const uint2 bl = IG_B8(bx[p] + off + ps * 64), bh = IG_B8(bx[p + 1u] + off + ps * 64);
                if (c == 0) imma16832<false, true>(cx[ps], wa.x & NIB, wb.x & NIB, wa.y & NIB, wb.y & NIB, bl.x, bl.y);
                else if (c == 1) imma16832<false, false>(cx[ps], wa.x & NIB, wb.x & NIB, wa.y & NIB, wb.y & NIB, bl.x, bl.y);
                else if (c == 2) imma16832<false, true>(cy[ps], wa.x & NIB, wb.x & NIB, wa.y & NIB, wb.y & NIB, bl.x, bl.y);
                else imma16832<false, false>(cy[ps], wa.x & NIB, wb.x & NIB, wa.y & NIB, wb.y & NIB, bl.x, bl.y);
                if (c < 2) imma16832<false, false>(cx[ps], wa.x & ~NIB, wb.x & ~NIB, wa.y & ~NIB, wb.y & ~NIB, bh.x, bh.y);
                else imma16832<false, false>(cy[ps], wa.x & ~NIB, wb.x & ~NIB, wa.y & ~NIB, wb.y & ~NIB, bh.x, bh.y);
            }
        }
        const uint32_t sel = 0x4440u + t;
        float d0, n0, sa0, sb0, ma0, mb0, d1, n1, sa1, sb1, ma1, mb1;
        scales(r0, sel, d0, n0, sa0, sb0, ma0, mb0);
        scales(r1, sel, d1, n1, sa1, sb1, ma1, mb1);
        // {1/S, sum of run 0, 1/S, sum of run 1} of sub-blocks t and t+4
        const float4 mx = *reinterpret_cast<const float4 *>(meta + 16u * t), my = *reinterpret_cast<const float4 *>(meta + 16u * t + 64u);
        const float ex = mul_rn(mx.x, nibf), ey = mul_rn(my.x, nibf);
        const float sxx = add_rn(mx.y, mx.w), sxy = add_rn(my.y, my.w);
        const float zx0 = mul_rn(fx_sum<NP>(cx, 0), ex), zy0 = mul_rn(fx_sum<NP>(cy, 0), ey);
        const float zx1 = mul_rn(fx_sum<NP>(cx, 2), ex), zy1 = mul_rn(fx_sum<NP>(cy, 2), ey);
        acc0 = add_rn(acc0, sub_rn(mul_rn(d0, fma_rn(sb0, zy0, mul_rn(sa0, zx0))), mul_rn(n0, fma_rn(mb0, sxy, mul_rn(ma0, sxx)))));
        acc1 = add_rn(acc1, sub_rn(mul_rn(d1, fma_rn(sb1, zy1, mul_rn(sa1, zx1))), mul_rn(n1, fma_rn(mb1, sxy, mul_rn(ma1, sxx)))));
    }
};

// Q6_K.  A quarter (n, q) is 32 columns: two runs of 16, each with its own int8 scale.  The eight B
// columns are (position, run, digit): the lanes with t < 2 hold the k slots of run 0 and supply the
// run-0 columns, the lanes with t >= 2 the run-1 columns, so lane t ends with the sums of quarter
// position t / 2, run t % 2.  Chains: (n, 0) + (n, 2), which share their ql bytes (low and high
// nibbles), and (n, 1) + (n, 3).  Blocks are only 2-byte aligned: CLS = (block start mod 8) / 2.
template <> struct ImmaStep<KIND_Q6_K> {
    static constexpr uint32_t POS_STRIDE = 2;        // chain position p reads quarter q0 + 2 p
    template <int CLS>
    static __device__ __forceinline__ uint2 ld8(const uint8_t *p) {      // 8 bytes at an address that is 2 CLS mod 8
        if (CLS == 0) return *reinterpret_cast<const uint2 *>(p);
        if (CLS == 2) return make_uint2(*reinterpret_cast<const uint32_t *>(p), *reinterpret_cast<const uint32_t *>(p + 4));
        if (CLS == 1) {
            const uint2 a = *reinterpret_cast<const uint2 *>(p - 2);
            const uint32_t b = *reinterpret_cast<const uint32_t *>(p + 6);
            return make_uint2(__funnelshift_r(a.x, a.y, 16u), __funnelshift_r(a.y, b, 16u));
        }
        const uint32_t a = *reinterpret_cast<const uint32_t *>(p - 2);
        const uint2 b = *reinterpret_cast<const uint2 *>(p + 2);
        return make_uint2(__funnelshift_r(a, b.x, 16u), __funnelshift_r(b.x, b.y, 16u));
    }
    // The six-bit values of the four quarters of a half block, four columns at a time: la / lb = a word of
    // ql (low nibbles: quarter 0 / 1, high nibbles: quarter 2 / 3), h = the word of qh (two bits per
    // quarter).  The qh fields are masked in pairs (0x33: quarters 0 and 2, or 1 and 3 after a shift by
    // two), so that one select per quarter puts a nibble of ql under a two-bit field of qh.
    struct Six4 { uint32_t q[4]; };
    static __device__ __forceinline__ uint32_t under(uint32_t nib, uint32_t top) { return (nib & NIB) | (top & ~NIB); }
    static __device__ __forceinline__ Six4 six4(uint32_t la, uint32_t lb, uint32_t h) {
        const uint32_t ha = h & 0x33333333u, hb = (h >> 2) & 0x33333333u;
        Six4 r;
        r.q[0] = under(la, ha << 4);
        r.q[1] = under(lb, hb << 4);
        r.q[2] = under(la >> 4, ha);
        r.q[3] = under(lb >> 4, hb);
        return r;
    }
    template <int ND, int CLS>
    static __device__ __forceinline__ void run_cls(const uint8_t *r0, const uint8_t *r1, const uint8_t *const (&bx)[4], const uint8_t *meta,
                                                   uint32_t t, float &acc0, float &acc1) {
        constexpr uint32_t SBS = ND * 32u;
        constexpr int NP = ND / 2;
        const float d0 = lds_half(r0 + 208u), d1 = lds_half(r1 + 208u);
        const uint32_t run = t & 1u, pos = t >> 1;
        float t0 = 0.f, t1 = 0.f;
#pragma unroll
        for (uint32_t n = 0; n < 2; ++n) {
            const uint2 la0 = ld8<CLS>(r0 + 64u * n + 8u * t), lb0 = ld8<CLS>(r0 + 64u * n + 32u + 8u * t), h0 = ld8<CLS>(r0 + 128u + 32u * n + 8u * t);
            const uint2 la1 = ld8<CLS>(r1 + 64u * n + 8u * t), lb1 = ld8<CLS>(r1 + 64u * n + 32u + 8u * t), h1 = ld8<CLS>(r1 + 128u + 32u * n + 8u * t);
            const Six4 x0 = six4(la0.x, lb0.x, h0.x), y0 = six4(la0.y, lb0.y, h0.y);      // row g: k slots 4t.., 16+4t..
            const Six4 x1 = six4(la1.x, lb1.x, h1.x), y1 = six4(la1.y, lb1.y, h1.y);      // row g+8
#pragma unroll
            for (uint32_t ch = 0; ch < 2; ++ch) {
                int c[NP][4];
#pragma unroll
                for (int ps = 0; ps < NP; ++ps) {
                    const uint2 b_lo = IG_B8(bx[0] + (4u * n + ch) * SBS + ps * 64), b_hi = IG_B8(bx[1] + (4u * n + ch) * SBS + ps * 64);
                    imma16832<false, true>(c[ps], x0.q[ch], x1.q[ch], y0.q[ch], y1.q[ch], b_lo.x, b_lo.y);
                    imma16832<false, false>(c[ps], x0.q[ch + 2u], x1.q[ch + 2u], y0.q[ch + 2u], y1.q[ch + 2u], b_hi.x, b_hi.y);
                }
                // this lane: quarter q = ch + 2 pos, run `run`; value - 32 through the run's activation sum
                const uint32_t q = ch + 2u * pos, idx = 8u * n + 2u * q + run;
                const float s0 = (float)(int)*reinterpret_cast<const int8_t *>(r0 + 192u + idx);
                const float s1 = (float)(int)*reinterpret_cast<const int8_t *>(r1 + 192u + idx);
                const float2 mt = *reinterpret_cast<const float2 *>(meta + (4u * n + q) * 16u + run * 8u);      // {1/S, run sum}
                const float off = mul_rn(mt.y, -32.0f);
                t0 = fma_rn(s0, fma_rn(fx_sum<NP>(c, 0), mt.x, off), t0);
                t1 = fma_rn(s1, fma_rn(fx_sum<NP>(c, 2), mt.x, off), t1);
            }
        }
        acc0 = fma_rn(d0, t0, acc0);
        acc1 = fma_rn(d1, t1, acc1);
    }
    template <int ND>
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, const uint8_t *const (&bx)[4], const uint8_t *meta,
                                               uint32_t t, float, float &acc0, float &acc1, uint32_t cls) {
        switch (cls) {          // warp-uniform
        case 0: run_cls<ND, 0>(r0, r1, bx, meta, t, acc0, acc1); break;
        case 1: run_cls<ND, 1>(r0, r1, bx, meta, t, acc0, acc1); break;
        case 2: run_cls<ND, 2>(r0, r1, bx, meta, t, acc0, acc1); break;
        default: run_cls<ND, 3>(r0, r1, bx, meta, t, acc0, acc1); break;
        }
    }
};

// Q4_0: step = 4 blocks of 32 (18 bytes each, 2-byte aligned), one MMA per block: the low nibbles of
// a word are columns 4t..4t+3, its high nibbles columns 16+4t...  Lane t owns block t.
template <> struct ImmaStep<KIND_Q4_0> {
    static constexpr uint32_t POS_STRIDE = 1;
    template <int ND>
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, const uint8_t *const (&bx)[4], const uint8_t *meta,
                                               uint32_t t, float, float &acc0, float &acc1, uint32_t) {
        constexpr int NP = ND / 2;
        int c[NP][4];
#pragma unroll
        for (uint32_t b = 0; b < 4; ++b) {
            // a step (72 bytes) starts on a 4-byte boundary: the quants of even blocks lie 2 bytes past one
            const uint32_t wa = lds32_known(r0 + 18u * b + 2u + 4u * t, (b & 1u) == 0u), wb = lds32_known(r1 + 18u * b + 2u + 4u * t, (b & 1u) == 0u);
#pragma unroll
            for (int ps = 0; ps < NP; ++ps) {
                const uint8_t *xb = bx[b] + ps * 64;
                const uint32_t b0 = lds32(xb), b1 = lds32(xb + 16);
                if (b == 0) imma16832<false, true>(c[ps], wa & NIB, wb & NIB, (wa >> 4) & NIB, (wb >> 4) & NIB, b0, b1);
                else imma16832<false, false>(c[ps], wa & NIB, wb & NIB, (wa >> 4) & NIB, (wb >> 4) & NIB, b0, b1);
            }
        }
        const float d0 = lds_half(r0 + 18u * t), d1 = lds_half(r1 + 18u * t);
        const float4 mt = *reinterpret_cast<const float4 *>(meta + 16u * t);
        const float off = mul_rn(add_rn(mt.y, mt.w), -8.0f);
        acc0 = fma_rn(d0, fma_rn(fx_sum<NP>(c, 0), mt.x, off), acc0);
        acc1 = fma_rn(d1, fma_rn(fx_sum<NP>(c, 2), mt.x, off), acc1);
    }
};

// Q8_0: step = 4 blocks of 32 int8 (34 bytes each, 2-byte aligned), one MMA per block with signed
// weights.  Lane t owns block t.
template <> struct ImmaStep<KIND_Q8_0> {
    static constexpr uint32_t POS_STRIDE = 1;
    template <int ND>
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, const uint8_t *const (&bx)[4], const uint8_t *meta,
                                               uint32_t t, float, float &acc0, float &acc1, uint32_t) {
        constexpr int NP = ND / 2;
        int c[NP][4];
#pragma unroll
        for (uint32_t b = 0; b < 4; ++b) {
            // a step (136 bytes) starts on a 4-byte boundary: the quants of even blocks lie 2 bytes past one
            const bool mis = (b & 1u) == 0u;
            const uint32_t wa0 = lds32_known(r0 + 34u * b + 2u + 4u * t, mis), wa1 = lds32_known(r0 + 34u * b + 18u + 4u * t, mis);
            const uint32_t wb0 = lds32_known(r1 + 34u * b + 2u + 4u * t, mis), wb1 = lds32_known(r1 + 34u * b + 18u + 4u * t, mis);
#pragma unroll
            for (int ps = 0; ps < NP; ++ps) {
                const uint8_t *xb = bx[b] + ps * 64;
                const uint32_t b0 = lds32(xb), b1 = lds32(xb + 16);
                if (b == 0) imma16832<true, true>(c[ps], wa0, wb0, wa1, wb1, b0, b1);
                else imma16832<true, false>(c[ps], wa0, wb0, wa1, wb1, b0, b1);
            }
        }
        const float d0 = lds_half(r0 + 34u * t), d1 = lds_half(r1 + 34u * t);
        const float inv = *reinterpret_cast<const float *>(meta + 16u * t);
        acc0 = fma_rn(d0, mul_rn(fx_sum<NP>(c, 0), inv), acc0);
        acc1 = fma_rn(d1, mul_rn(fx_sum<NP>(c, 2), inv), acc1);
    }
};
#undef IG_B8

// ---------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------

// Four elements of a tagged vector: two 16-byte loads of two {value, tag} words each (every 8-byte word is read
// whole).  False unless all four carry the tag.
__device__ __forceinline__ bool tagged_load4(const uint64_t *tagged, uint32_t j, uint32_t tag, float4 &v) {
    uint64_t w0, w1, w2, w3;
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(w0), "=l"(w1) : "l"(tagged + 4u * (size_t)j) : "memory");
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(w2), "=l"(w3) : "l"(tagged + 4u * (size_t)j + 2u) : "memory");
    v = make_float4(__uint_as_float((uint32_t)w0), __uint_as_float((uint32_t)w1), __uint_as_float((uint32_t)w2), __uint_as_float((uint32_t)w3));
    return (uint32_t)(w0 >> 32) == tag && (uint32_t)(w1 >> 32) == tag && (uint32_t)(w2 >> 32) == tag && (uint32_t)(w3 >> 32) == tag;
}

// What a thread carries from one projection to the next when a kernel runs several of them
// back to back over the same ring (the one-projection kernels use a fresh one).
struct MmaRun {
    uint32_t itg[2] = {0u, 0u};   // stage fills so far in the ring of each consumer group (a consumer counts its own group's)
    uint32_t tiles = 0;      // tiles so far: slot and phase of the partial-sum ring
    bool setup = true;       // initialise the barriers and the zero block (first projection only)
    bool build_x = true;     // consumers build the activation row; false: the row of the previous projection is still there
    unsigned long long *trace = nullptr;    // debugging: where thread 0 stores the time at which the activation row was ready
};

// A group of up to TK routed pairs that share one expert (one pass over a tile of the expert grouping):
// the expert's rows are streamed once and multiplied with each pair's activation row.
struct MmaTile {
    uint32_t expert;         // the tile's expert
    uint32_t first;          // packed position of the pass's first pair
    uint32_t nt;             // pairs in this pass (1..TK)
    uint32_t gather;         // the activation row of packed position q is row pairs[q] / top of x (else row q)
    const uint32_t *pairs;   // packed position -> pair index
};

// The whole CTA's work on one projection: CTA `cta` of `nctas` (its share of the rows), pair `pair`.
// False when a bounded wait ran out (the status word says which).
// CW consumer warps in groups of eight: a group splits the columns of a tile among its warps and takes
// every (CW / 8)-th tile, so with sixteen warps two stages of the ring are in work at once.
// TK > 1: `tile` names up to TK pairs of one expert; their rows sit TK deep in shared memory (p.x_row_stride apart).
// (LINK: the kernel exchanges row shards with other GPUs — tagged words out, tagged inputs in.  It is a template
// parameter because the polling loads would otherwise sit in every launch's prologue, whose time is
// instruction fetch: with them the single-GPU step ran 2.79 ms instead of 2.28 ms.  For the same reason which
// of the two normalised inputs is tagged is known at compile time in the common cases, so a prologue holds
// one form of each input's loads: LINK_OUT = plain inputs, LINK_A / LINK_B = that input tagged, LINK_ANY =
// decided at run time.)
enum { LINK_NONE = 0, LINK_OUT = 1, LINK_A = 2, LINK_B = 3, LINK_ANY = 4 };
template <uint32_t KIND, int NMAT, int XM, int CW = MMA_WARPS, int TK = 1, int LINK = LINK_NONE>
__device__ __forceinline__ bool gemv_mma_body(const MmaArgs &a, uint8_t *smem, const uint32_t cta, const uint32_t nctas, const uint32_t pair,
                                              const bool whole_tiles, MmaRun &run, const MmaTile *tile = nullptr) {
    const MmaPlan &p = a.plan;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + MMA_MAX_STAGES;
    uint64_t *xbar = empty + MMA_MAX_STAGES;
    uint64_t *tbar = xbar + 1;                                   // [MMA_RED_SLOTS]
    uint8_t *xrow = smem + MMA_BAR_BYTES;
    constexpr bool HI = XM == XM_F16_HI;
    constexpr bool FX = XM >= XM_FX2;                     // fixed-point rows, int8 MMA
    constexpr int ND = XM == XM_FX4 ? 4 : 2;              // digits per activation (fixed point)
    constexpr uint32_t XB = FX ? (uint32_t)ND : HI ? 2u : 4u;       // packed bytes per activation
    const float *sx = reinterpret_cast<const float *>(xrow + (size_t)p.cols * XB);     // binary16 rows: 16-column sums; fixed point: {1/S, run sum} pairs
    float *red = reinterpret_cast<float *>(xrow + ((p.x_bytes + 127u) & ~127u));
    uint8_t *zeros = reinterpret_cast<uint8_t *>(red) + p.red_bytes - MMA_ZERO_BYTES;
    uint8_t *stages = reinterpret_cast<uint8_t *>(red) + p.red_bytes;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    if (run.setup) {
        if (threadIdx.x == 0) {
            for (uint32_t s = 0; s < p.stages; ++s) {
                ptx::mbar_init(&full[s], 1);
                ptx::mbar_init(&empty[s], MMA_WARPS);
            }
            ptx::mbar_init(xbar, 1);
            for (uint32_t i = 0; i < p.red_slots; ++i) ptx::mbar_init(&tbar[i], MMA_WARPS);
            ptx::mbar_init_fence();
        }
        for (uint32_t i = threadIdx.x; i < MMA_ZERO_BYTES / 4u; i += (CW + 1) * 32) reinterpret_cast<uint32_t *>(zeros)[i] = 0u;
        __syncthreads();
        ptx::pdl_launch_dependents();
        run.setup = false;
    }

    uint32_t r_begin, r_end;
    const uint32_t stage_rows = 16u * p.row_tiles;
    {
        // An even split of the rows keeps every CTA's bytes equal (long launches are bound by the
        // CTA that streams the most).  The grouped launch asks for whole tiles per CTA instead:
        // its parts are short and a tile costs its arithmetic whether or not all its rows are live.
        const uint32_t tiles = (p.rows + stage_rows - 1) / stage_rows;
        if (whole_tiles && nctas < tiles) {
            r_begin = (uint32_t)((uint64_t)tiles * cta / nctas) * stage_rows;
            r_end = (uint32_t)((uint64_t)tiles * (cta + 1) / nctas) * stage_rows;
            if (r_end > p.rows) r_end = p.rows;
        } else {
            cta_rows(p.rows, cta, nctas, r_begin, r_end);
        }
    }
    const uint32_t n_tiles = (r_end - r_begin + stage_rows - 1) / stage_rows;

    if (warp == (uint32_t)CW) {
        // ---- producer warp: weights first (they do not depend on the previous kernel),
        // then, once the ring is primed, wait for the previous kernel and fetch the
        // packed activations ----
        uint32_t expert = tile ? tile->expert : a.expert, x_row = 0;
        if (a.ids && !tile) {                          // routing comes from the previous kernel
            ptx::pdl_wait();
            expert = a.ids[pair];
            if (expert >= a.n_experts) return true;    // skipped pair, or out of range: consumers handle it
            x_row = a.per_pair ? pair : pair / a.top;
        }
        const size_t mat_off = (size_t)expert * p.rows * p.stride;
        // Each consumer group has its own ring (stages / GROUPS slots) and takes every GROUPS-th tile; the
        // producer fills the groups' rings in turn, one stage each, so that all groups are fed at once.
        bool x_sent = false;
        constexpr uint32_t GROUPS_P = CW / MMA_WARPS;
        const uint32_t fpt = p.chunks * NMAT, sg = p.stages / GROUPS_P;
        uint32_t fills_g[GROUPS_P], tile_g[GROUPS_P], cm_g[GROUPS_P], done_g[GROUPS_P], max_fills = 0, issued = 0;
#pragma unroll
        for (uint32_t gq = 0; gq < GROUPS_P; ++gq) {
            fills_g[gq] = n_tiles > gq ? ((n_tiles - 1u - gq) / GROUPS_P + 1u) * fpt : 0u;
            tile_g[gq] = gq; cm_g[gq] = 0u; done_g[gq] = 0u;
            if (fills_g[gq] > max_fills) max_fills = fills_g[gq];
        }
        for (uint32_t j = 0; j < max_fills; ++j) {
#pragma unroll
            for (uint32_t gq = 0; gq < GROUPS_P; ++gq) {
                if (done_g[gq] >= fills_g[gq]) continue;
                const uint32_t tile = tile_g[gq], cm = cm_g[gq];
                const uint32_t row0 = r_begin + tile * stage_rows;
                const uint32_t nrows = (r_end - row0) < stage_rows ? (r_end - row0) : stage_rows;
                const uint32_t c = cm / NMAT, m = cm - c * NMAT;
                if (!x_sent && issued == p.stages && !a.na) {   // ring primed: the next wait needs the consumers
                    if (!a.ids) ptx::pdl_wait();
                    if (lane == 0) {
                        ptx::mbar_expect_tx(xbar, p.x_bytes);
                        ptx::bulk_g2s(xrow, a.xp + (size_t)x_row * p.x_bytes, p.x_bytes, xbar);
                    }
                    x_sent = true;
                }
                const uint32_t itl = run.itg[gq] + done_g[gq];
                const uint32_t s = gq * sg + itl % sg, ph = (itl / sg) & 1u;
                bool ok = true;
                if (lane == 0) ok = ptx::mbar_wait_sleep<128>(&empty[s], ph ^ 1u);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { if (lane == 0) set_status_word(a.status, KERNEL_ERR_PRODUCER_TIMEOUT); return false; }
                uint8_t *dst = stages + (size_t)s * p.stage_bytes;
                if (a.tmap[m]) {
                    // one tiled copy brings the whole stage: stage_rows rows of row_pitch bytes each (the chunk and the
                    // first bytes of the next one, which make the pitch; rows past the matrix read as zeros).  A 1-D
                    // bulk copy per row costs the issuing warp about 150 cycles each, more than the rows take to stream.
                    if (lane == 0) {
                        ptx::mbar_expect_tx(&full[s], p.row_pitch * stage_rows);
                        ptx::tma_load_2d(dst, a.tmap[m], (c * p.chunk_bytes) >> 3, row0, &full[s]);
                    }
                } else {
                    if (lane == 0) ptx::mbar_expect_tx(&full[s], p.chunk_bytes * nrows);
                    __syncwarp();
                    for (uint32_t r = lane; r < nrows; r += 32u)
                        ptx::bulk_g2s(dst + (size_t)r * p.row_pitch,
                                      a.w[m] + mat_off + (size_t)(row0 + r) * p.stride + (size_t)c * p.chunk_bytes,
                                      p.chunk_bytes, &full[s]);
                }
                ++issued; ++done_g[gq];
                if (++cm_g[gq] == fpt) { cm_g[gq] = 0u; tile_g[gq] += GROUPS_P; }
            }
        }
        if (!x_sent && !a.na) {                          // fewer stage fills than ring slots
            if (!a.ids) ptx::pdl_wait();
            if (lane == 0) {
                ptx::mbar_expect_tx(xbar, p.x_bytes);
                ptx::bulk_g2s(xrow, a.xp + (size_t)x_row * p.x_bytes, p.x_bytes, xbar);
            }
        }
#pragma unroll
        for (uint32_t gq = 0; gq < GROUPS_P; ++gq) run.itg[gq] += fills_g[gq];
        return true;
    }

    // ---- consumer warps ----
    const uint32_t ntok = tile ? tile->nt : 1u;        // activation rows in work
    const uint32_t xrs = TK > 1 ? p.x_row_stride : 0u;
    if (a.ids && !tile) {
        ptx::pdl_wait();
        const uint32_t e = a.ids[pair];
        if (e >= a.n_experts) {
            if (e == ROUTE_SKIP) {                      // not this device's expert: the row is zero
                float *yz = a.y + (size_t)pair * p.rows;
                for (uint32_t r = r_begin + threadIdx.x; r < r_end; r += CW * 32) yz[r] = 0.f;
            } else if (threadIdx.x == 0) set_status_word(a.status, KERNEL_ERR_EXPERT_RANGE);
            return true;
        }
    }
    if constexpr (FX) {
      if (run.build_x && warp < (uint32_t)MMA_WARPS) {
        // ---- fused add + RMS normalisation + packing (what add_rms with a packed output computes,
        // kernels/generic.metal:390-404): the 256 consumer threads of every CTA build the packed row ----
        ptx::pdl_wait();
        const uint32_t tid = threadIdx.x, n4 = p.cols >> 2;
        // inputs assembled from every rank's rows are read from their tagged twins, polling until each word carries
        // this step's tag (bounded; on a time-out the step goes on with what is there and the status word tells)
        const uint64_t *const ta = (LINK == LINK_A || LINK == LINK_ANY) ? a.tp.in[0] : nullptr;
        const uint64_t *const tb = (LINK == LINK_B || LINK == LINK_ANY) ? a.tp.in[1] : nullptr;
        const bool use_ta = LINK == LINK_A || (LINK == LINK_ANY && ta), use_tb = LINK == LINK_B || (LINK == LINK_ANY && tb);
        uint32_t tag_a = 0, tag_b = 0;
        if (use_ta || use_tb) {
            const uint32_t step = *reinterpret_cast<const volatile uint32_t *>(a.tp.step);
            tag_a = step * a.tp.tag_mul + a.tp.in_tag[0];
            tag_b = step * a.tp.tag_mul + a.tp.in_tag[1];
        }
        // (a wait that ran out earlier in the step has set the status word: do not wait again)
        bool gave_up = (use_ta || use_tb) && a.status && *reinterpret_cast<const volatile int *>(a.status) != 0;
        auto poll = [&](auto pass) {                   // pass() issues a batch of loads and says whether all were this step's
            uint64_t t0 = 0;
            for (uint32_t spins = 1; !pass() && !gave_up; ++spins) {
                if ((spins & 63u) != 0u) continue;
                const uint64_t now = ptx::global_timer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > ptx::WAIT_LIMIT_NS) { set_status_word(a.status, KERNEL_ERR_PEER_TIMEOUT); gave_up = true; }
            }
        };
       for (uint32_t ti = 0; ti < ntok; ++ti) {
        const uint32_t in_row = tile ? (tile->gather ? tile->pairs[tile->first + ti] / a.top : tile->first + ti)
                                     : a.ids ? (a.per_pair ? pair : pair / a.top) : 0u;
        uint8_t *const xrow_t = xrow + (size_t)ti * xrs;
        const float4 *a4 = reinterpret_cast<const float4 *>(a.na) + (size_t)in_row * n4, *b4 = reinterpret_cast<const float4 *>(a.nb);
        float *scratch = red;                          // the partial-sum area is idle until the first tile ends
        auto load = [&](uint32_t j) {
            // (read through L2: in a kernel that runs several projections the vectors come from other CTAs)
            float4 v, o;
            if (use_ta) poll([&] { return tagged_load4(ta, j, tag_a, v); });
            else v = __ldcg(a4 + j);
            if (b4) {
                if (use_tb) poll([&] { return tagged_load4(tb, j, tag_b, o); });
                else o = __ldcg(b4 + j);
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
            }
            return v;
        };
        auto reduce = [&](float v, bool is_max) {
            for (uint32_t off = 16; off; off >>= 1) {
                const float o = __shfl_xor_sync(0xffffffffu, v, off);
                v = is_max ? fmaxf(v, o) : v + o;
            }
            ptx::named_bar_sync(1, MMA_WARPS * 32);
            if (lane == 0) scratch[warp] = v;
            ptx::named_bar_sync(1, MMA_WARPS * 32);
            float r = scratch[0];
#pragma unroll
            for (int i = 1; i < MMA_WARPS; ++i) r = is_max ? fmaxf(r, scratch[i]) : r + scratch[i];
            return r;
        };
        constexpr uint32_t NT = MMA_WARPS * 32;
        // the row stays in registers, NV float4 per thread (the unrolled loops issue their instructions
        // for dead slots too, so narrow rows take the short form)
        auto in_registers = [&](auto nv_const) {
            constexpr uint32_t NV = decltype(nv_const)::value;
            float4 v[NV];
            float sum = 0.f;
            // all loads of the row first, nothing that depends on one of them in between: one trip to L2 for the
            // whole row (a store of the residual sum after each load would make every load wait for the one before)
            if (use_ta) {
                poll([&] {
                    bool all = true;
#pragma unroll
                    for (uint32_t i = 0; i < NV; ++i) {
                        const uint32_t j = tid + i * NT;
                        if (j < n4) all &= tagged_load4(ta, j, tag_a, v[i]);
                        else v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    return all;
                });
            } else {
#pragma unroll
                for (uint32_t i = 0; i < NV; ++i) {
                    const uint32_t j = tid + i * NT;
                    v[i] = j < n4 ? __ldcg(a4 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            if (b4) {                                  // (four at a time: the second vector's loads are in flight together with the first's)
#pragma unroll
                for (uint32_t i0 = 0; i0 < NV; i0 += 4u) {
                    float4 o[4];
                    if (use_tb) {
                        poll([&] {
                            bool all = true;
#pragma unroll
                            for (uint32_t k = 0; k < 4u; ++k) {
                                const uint32_t j = tid + (i0 + k) * NT;
                                if (i0 + k < NV && j < n4) all &= tagged_load4(tb, j, tag_b, o[k]);
                                else o[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                            return all;
                        });
                    } else {
#pragma unroll
                        for (uint32_t k = 0; k < 4u; ++k) {
                            const uint32_t j = tid + (i0 + k) * NT;
                            o[k] = (i0 + k < NV && j < n4) ? __ldcg(b4 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
#pragma unroll
                    for (uint32_t k = 0; k < 4u; ++k)
                        if (i0 + k < NV) { v[i0 + k].x += o[k].x; v[i0 + k].y += o[k].y; v[i0 + k].z += o[k].z; v[i0 + k].w += o[k].w; }
                }
            }
#pragma unroll
            for (uint32_t i = 0; i < NV; ++i) {
                const uint32_t j = tid + i * NT;
                if (j < n4) {
                    if (a.ns && cta == 0) reinterpret_cast<float4 *>(a.ns)[j] = v[i];
                    sum += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
                }
            }
            if (run.trace && threadIdx.x == 0) run.trace[2] = ptx::global_timer_ns() + (unsigned long long)(sum == 12345.678f);
            const float inv = a.npack ? 1.0f : 1.0f / sqrtf(reduce(sum, false) / (float)p.cols + a.neps);
            if (run.trace && threadIdx.x == 0) run.trace[3] = ptx::global_timer_ns();
#pragma unroll
            for (uint32_t i = 0; i < NV; ++i) {
                if (i * NT >= n4) break;                               // uniform: the shuffles of a sub-block keep all its lanes
                const uint32_t j = tid + i * NT;
                fx_norm_store<ND>(xrow_t, p.cols, j, v[i], inv, a.nw, a.nround_bf16, j < n4);
            }
        };
        if (n4 <= 4u * NT) in_registers(std::integral_constant<uint32_t, 4>{});            // up to 4096 columns
        else if (n4 <= 12u * NT) in_registers(std::integral_constant<uint32_t, 12>{});     // up to 12288
        else {
            float sum = 0.f;
            for (uint32_t j = tid; j < n4; j += NT) {
                const float4 v = load(j);
                if (a.ns && cta == 0) reinterpret_cast<float4 *>(a.ns)[j] = v;
                sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
            const float inv = a.npack ? 1.0f : 1.0f / sqrtf(reduce(sum, false) / (float)p.cols + a.neps);
            for (uint32_t j0 = 0; j0 < n4; j0 += NT) {                 // uniform trip count: the shuffles of a sub-block keep all its lanes
                const uint32_t j = j0 + tid;
                const bool live = j < n4;
                fx_norm_store<ND>(xrow_t, p.cols, j, live ? load(j) : make_float4(0.f, 0.f, 0.f, 0.f), inv, a.nw, a.nround_bf16, live);
            }
        }
       }
        ptx::named_bar_sync(1, MMA_WARPS * 32);
      }
      // (the first eight warps build the row, so its arithmetic does not depend on CW; the others wait here)
      if (CW > MMA_WARPS && run.build_x) ptx::named_bar_sync(2, CW * 32);
      if (run.trace && threadIdx.x == 0) *run.trace = ptx::global_timer_ns();
    } else {
        if (!ptx::mbar_wait(xbar, 0)) {
            if (lane == 0) set_status_word(a.status, KERNEL_ERR_CONSUMER_TIMEOUT);
            return false;
        }
    }
    ptx::pdl_wait();          // outputs may be read by the previous kernel until it ends
    // binary16 rows carry one power-of-two scale for the whole row; fixed-point rows one per sub-block, applied in the steps
    const float unscale = FX ? 1.0f : *reinterpret_cast<const float *>(xrow + (size_t)p.cols * XB + p.cols / 4u);

    const uint32_t g = lane >> 2, t = lane & 3u;
    constexpr uint32_t GROUPS = CW / MMA_WARPS;
    const uint32_t grp = warp / MMA_WARPS, wg = warp % MMA_WARPS;         // consumer group and the warp's place in it
    const uint32_t kw = wg & ((1u << p.kw_log2) - 1u), rt = wg >> p.kw_log2;
    constexpr uint32_t STEP_BYTES = KIND == KIND_Q4_K ? 144u : KIND == KIND_Q6_K ? 210u : KIND == KIND_Q4_0 ? 72u : 136u;
    constexpr uint32_t MMAS = (KIND == KIND_Q4_K || KIND == KIND_Q6_K) ? 16u : 8u;     // binary16 MMAs (16 columns each) per step
    constexpr uint32_t XS = FX ? (uint32_t)ND * 16u : HI ? 32u : 64u;                   // packed bytes per 16 columns
    const uint32_t step_stride = STEP_BYTES << p.kw_log2;                               // this warp's next step
    const uint32_t x_stride = (MMAS * XS) << p.kw_log2, s_stride = MMAS << p.kw_log2;     // bytes, floats (fixed point: 8 bytes of scale and sum per 16 columns = 2 floats)
    // B operands: column n = g of the MMA belongs to lane g; columns 2j, 2j+1 carry (xh, xl)
    // for group j only, so this lane reads the real activations for group own = g / 2 and
    // zeros for the others
    // (with only the high part packed, the low-part columns — odd g — always read zeros)
    // (fixed point: column g is digit g % 2 of chain position g / 2; Q6_K splits a position's columns
    // over the two runs of 16, and the run-0 columns belong to the lanes with t < 2)
    const uint32_t own = FX ? (KIND == KIND_Q6_K ? (((t >> 1) == ((g >> 1) & 1u)) ? (g >> 2) : 9u) : (g >> 1))
                            : (HI && (g & 1u)) ? 4u : (g >> 1);
    const uint8_t *xlane = FX ? xrow + (g & 1u) * 32u + t * ((KIND == KIND_Q4_K || KIND == KIND_Q6_K) ? 8u : 4u)
                              : xrow + (HI ? t : (g & 1u) * 4u + t) * 8u;
    const uint8_t *zlane = FX ? zeros + lane * 8u : zeros + ((g & 1u) * 4u + t) * 8u;
    const float nibf = (t & 1u) ? 0.0625f : 1.0f;                  // Q4_K int8 steps: odd sub-blocks keep their nibbles in place (16 q)
    float *y = a.y + (tile ? (size_t)tile->first * p.rows : a.ids ? (size_t)pair * p.rows : 0);       // row of the first activation row in work
    const uint32_t kmask = (1u << p.kw_log2) - 1u;

    // Sum of a finished tile's partials over the K warps -> y.  The warp that sums rotates with
    // the tile, and it sums tile T only after its own work on tile T + 1, when the partials are
    // long complete: no warp falls behind the others at a tile boundary.
    const uint32_t tile_base = run.tiles;          // position of this projection's first tile in the partial-sum ring
    const uint32_t out_tag = LINK && a.tp.n_out ? *reinterpret_cast<const volatile uint32_t *>(a.tp.step) * a.tp.tag_mul + a.tp.out_tag : 0u;
    auto sum_tile = [&](uint32_t tile) -> bool {
        const uint32_t ring = tile_base + tile;
        if (((ring ^ kw) & kmask) != 0u) return true;                  // another warp's turn
        const uint32_t slot_id = ring % p.red_slots;
        const float *slot = red + (size_t)slot_id * MMA_WARPS * TK * 2u * 16u;
        if (!ptx::mbar_wait_sleep<20>(&tbar[slot_id], (ring / p.red_slots) & 1u)) {
            if (lane == 0) set_status_word(a.status, KERNEL_ERR_CONSUMER_TIMEOUT);
            return false;
        }
        const uint32_t row0 = r_begin + tile * stage_rows;
        const uint32_t nrows = (r_end - row0) < stage_rows ? (r_end - row0) : stage_rows;
        const uint32_t lrow = rt * 16u + (lane & 15u), first = rt << p.kw_log2;
        // NMAT == 2: lanes 0..15 sum matrix 0 and lanes 16..31 matrix 1, then exchange
        const uint32_t m = NMAT == 2 ? (lane >> 4) : 0u;
#pragma unroll
        for (uint32_t ti = 0; ti < (uint32_t)TK; ++ti) {
            if (ti >= ntok) break;
            float sum = 0.f;
            if (lrow < nrows && (NMAT == 2 || lane < 16u))
                for (uint32_t k = 0; k <= kmask; ++k) sum = add_rn(sum, slot[(((first + k) * TK + ti) * 2u + m) * 16u + (lane & 15u)]);
            sum = mul_rn(sum, unscale);
            const float other = NMAT == 2 ? __shfl_xor_sync(0xffffffffu, sum, 16) : 0.f;
            if (lrow < nrows && lane < 16u) {
                const float out = NMAT == 2 ? glu_f(sum, other, a.glu == 2) : sum;
                y[(size_t)ti * p.rows + row0 + lrow] = out;
                if (LINK && a.tp.n_out) {              // the row's tagged word, whole, into every rank's twin (NVLink stores)
                    const uint64_t word = ((uint64_t)out_tag << 32) | __float_as_uint(out);
                    for (uint32_t pr = 0; pr < a.tp.n_out; ++pr)
                        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(a.tp.out[pr] + (size_t)ti * p.rows + row0 + lrow), "l"(word) : "memory");
                }
            }
        }
        return true;
    };

    const uint32_t sg = p.stages / GROUPS;             // slots of this group's ring
    uint32_t it = run.itg[grp];
    for (uint32_t tile = grp; tile < n_tiles; tile += GROUPS) {
        const uint32_t row0 = r_begin + tile * stage_rows;
        const uint32_t nrows = (r_end - row0) < stage_rows ? (r_end - row0) : stage_rows;
        const uint32_t lr0 = rt * 16u + g, lr1 = lr0 + 8u;             // rows of this lane inside the stage
        const uint32_t ur0 = lr0 < nrows ? lr0 : rt * 16u;              // rows past the end read the tile's first row
        const uint32_t ur1 = lr1 < nrows ? lr1 : rt * 16u;
        float acc[TK][NMAT][2];
#pragma unroll
        for (int ti = 0; ti < TK; ++ti)
#pragma unroll
            for (int m = 0; m < NMAT; ++m) acc[ti][m][0] = acc[ti][m][1] = 0.f;
        for (uint32_t c = 0; c < p.chunks; ++c) {
            const uint32_t gs0 = c * (p.spw << p.kw_log2) + kw;                // first step inside the row
#pragma unroll
            for (int m = 0; m < NMAT; ++m, ++it) {
                const uint32_t s = grp * sg + it % sg, ph = (it / sg) & 1u;
                if (!ptx::mbar_wait_sleep<20>(&full[s], ph)) {
                    if (lane == 0) set_status_word(a.status, KERNEL_ERR_CONSUMER_TIMEOUT);
                    return false;
                }
                const uint8_t *st = stages + (size_t)s * p.stage_bytes;
                if (rt * 16u < nrows) {
#pragma unroll
                  for (uint32_t ti = 0; ti < (uint32_t)TK; ++ti) {
                    if (ti >= ntok) break;
                    const uint8_t *b0 = st + (size_t)ur0 * p.row_pitch + kw * STEP_BYTES;
                    const uint8_t *b1 = st + (size_t)ur1 * p.row_pitch + kw * STEP_BYTES;
                    const uint8_t *xs = xlane + (size_t)ti * xrs + (size_t)gs0 * MMAS * XS;
                    const float *ss = reinterpret_cast<const float *>(reinterpret_cast<const uint8_t *>(sx) + (size_t)ti * xrs) + gs0 * MMAS * (FX ? 2u : 1u);
                    for (uint32_t i = 0; i < p.spw; ++i) {
                        if constexpr (FX) {
                            // chain position p of this lane: its own digits at the sub-block of that position, zeros elsewhere
                            constexpr uint32_t PS = ImmaStep<KIND>::POS_STRIDE * ND * 32u;
                            const uint8_t *const xb[4] = {own == 0 ? xs : zlane, own == 1 ? xs + PS : zlane, own == 2 ? xs + 2u * PS : zlane,
                                                          own == 3 ? xs + 3u * PS : zlane};
                            // rows start on 16-byte boundaries in the stage: a Q6_K block (210 bytes) starts 2 (block mod 4)
                            // bytes past an 8-byte boundary (warp-uniform; the other formats ignore it)
                            ImmaStep<KIND>::template run<ND>(b0, b1, xb, reinterpret_cast<const uint8_t *>(ss), t, nibf, acc[ti][m][0], acc[ti][m][1],
                                                             (kw + (i << p.kw_log2)) & 3u);
                        } else {
                            const uint8_t *const xb[4] = {own == 0 ? xs : zlane, own == 1 ? xs : zlane, own == 2 ? xs : zlane,
                                                          own == 3 ? xs : zlane};
                            // rows start on 16-byte boundaries in the stage: an odd Q6_K block (210 bytes) starts
                            // 2 bytes past a 4-byte boundary (warp-uniform; the other formats ignore it)
                            if (KIND == KIND_Q6_K && (((kw + (i << p.kw_log2)) & 1u) != 0u))
                                MmaStep<KIND>::template run<XS>(b0, b1, xb, ss, t, acc[ti][m][0], acc[ti][m][1], true);
                            else
                                MmaStep<KIND>::template run<XS>(b0, b1, xb, ss, t, acc[ti][m][0], acc[ti][m][1], false);
                        }
                        b0 += step_stride; b1 += step_stride;
                        xs += x_stride; ss += s_stride * (FX ? 2u : 1u);
                    }
                  }
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&empty[s]);
            }
        }
        // quad reduce (the four lanes hold different scale groups), then across the K warps
        const uint32_t slot_id = (tile_base + tile) % p.red_slots;
        float *slot = red + (size_t)slot_id * MMA_WARPS * TK * 2u * 16u;
#pragma unroll
        for (int ti = 0; ti < TK; ++ti)
#pragma unroll
            for (int m = 0; m < NMAT; ++m)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float v = acc[ti][m][h];
                    v = add_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
                    v = add_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
                    if (t == 0) slot[((wg * TK + ti) * 2u + m) * 16u + g + 8u * h] = v;
                }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&tbar[slot_id]);
        if (tile >= GROUPS && !sum_tile(tile - GROUPS)) return false;
    }
    if (n_tiles > grp) {                               // the group's last tile
        const uint32_t last = grp + (n_tiles - 1u - grp) / GROUPS * GROUPS;
        if (!sum_tile(last)) return false;
    }
    run.itg[grp] = it;
    run.tiles = tile_base + n_tiles;
    return true;
}

template <uint32_t KIND, int NMAT, int OCC, int XM, int LINK = LINK_NONE>
__global__ void __launch_bounds__(MMA_THREADS, OCC) gemv_mma_kernel(const __grid_constant__ MmaArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    MmaRun run;
    gemv_mma_body<KIND, NMAT, XM, MMA_WARPS, 1, LINK>(a, smem, blockIdx.x, gridDim.x, blockIdx.y, false, run);
}

// Routed projections grouped by expert (the reference's packed MoE path for more than four tokens:
// Generic::moe_packed, src/generic.rs:578-660, with quant_expert_gather / quant_expert_packed /
// quant_expert_gate_up, kernels/qwen.metal:953-1081): grid.y walks the tiles of the expert grouping
// (expert, first packed position, up to 32 pairs); the CTAs of a tile stream the expert's rows ONCE per
// pass and multiply them with up to MMA_TILE_TOKENS activation rows held side by side in shared memory,
// instead of once per pair.  Activation rows are gathered through pairs[] (gate/up: row pair / top of x)
// or taken in packed order (down); results go to packed rows.
struct MmaTileArgs {
    MmaArgs a;
    const uint32_t *tiles;       // [capacity][4] = expert, first, pairs, mode; null: ONE tile of dense rows (below)
    const uint32_t *pairs;       // packed position -> pair index
    uint32_t gather;
    uint32_t dense_expert, dense_rows;     // without a table: rows 0 .. dense_rows - 1 of x against this expert
    uint32_t per_pass;                     // activation rows per pass over the weights (at most MMA_TILE_TOKENS)
};

template <uint32_t KIND, int NMAT>
__global__ void __launch_bounds__(MMA_THREADS, 2) gemv_mma_tiles_kernel(const __grid_constant__ MmaTileArgs ta) {
    extern __shared__ __align__(128) uint8_t smem[];
    ptx::pdl_wait();                                   // the grouping tables come from the kernels before
    uint32_t expert = ta.dense_expert, first = 0u, n = ta.dense_rows;
    if (ta.tiles) {
        const uint32_t *tl = ta.tiles + 4u * blockIdx.y;
        expert = tl[0]; first = tl[1]; n = tl[2];
    }
    if (n == 0) return;                                // unused tile
    if (expert >= ta.a.n_experts) {
        if (threadIdx.x == 0) set_status_word(ta.a.status, KERNEL_ERR_EXPERT_RANGE);
        return;
    }
    MmaRun run;
    for (uint32_t tok0 = 0; tok0 < n; tok0 += ta.per_pass) {
        // the rows of the pass before are rebuilt: every consumer warp must be through with them
        if (tok0 && threadIdx.x < MMA_WARPS * 32) ptx::named_bar_sync(5, MMA_WARPS * 32);
        MmaTile tile = {expert, first + tok0, n - tok0 < ta.per_pass ? n - tok0 : ta.per_pass, ta.gather, ta.pairs};
        if (!gemv_mma_body<KIND, NMAT, XM_FX4, MMA_WARPS, (int)MMA_TILE_TOKENS>(ta.a, smem, blockIdx.x, gridDim.x, blockIdx.y, false, run, &tile)) return;
    }
}

template <uint32_t KIND, int NMAT>
static cudaError_t launch_tiles_t(const MmaTileArgs &ta, dim3 grid, cudaStream_t stream, bool pdl) {
    auto kernel = gemv_mma_tiles_kernel<KIND, NMAT>;
    static DeviceOnce once;
    {
        const cudaError_t e = once.smem(kernel, (int)MMA_SMEM_MAX);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(MMA_THREADS);
    cfg.dynamicSmemBytes = ta.a.plan.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, ta);
}

// y_packed[pos][rows] = W[expert of pos] . x[row of pos] (nmat == 2: glu(gate . x, up . x)) for the packed positions
// of every tile.  False when the call is not one this kernel handles (the caller then projects pair by pair).
bool try_launch_gemv_tiles(const GemvCall &c, const uint32_t *tiles, const uint32_t *pairs, uint32_t tile_capacity, bool gather,
                           const LaunchCtx &ctx, cudaError_t &err) {
    if (!mma_kind(c.kind) || c.cols % 64u || c.x_packed || c.x_bf16 || ((uintptr_t)c.x % 16u) || !tiles || !pairs || tile_capacity == 0) return false;
    if (((uintptr_t)c.w[0] % 16u) || (c.nmat == 2 && ((uintptr_t)c.w[1] % 16u)) || ((size_t)c.rows * c.stride) % 16u) return false;
    MmaPlan plan;
    if (!plan_mma(c.kind, c.cols, c.rows, c.stride, c.nmat, 1u, MMA_SMEM_BUDGET, XM_FX4, plan, nullptr, MMA_TILE_TOKENS) &&
        !plan_mma(c.kind, c.cols, c.rows, c.stride, c.nmat, 1u, MMA_SMEM_MAX, XM_FX4, plan, nullptr, MMA_TILE_TOKENS))
        return false;
    // CTAs per tile: about as many live tiles as there are experts touched (at most min(pairs, experts))
    // (several waves on purpose: a tile's passes are bound by latency and issue, not by bytes, and tiles differ in
    // their number of passes, so more and shorter CTAs balance better: 32 tokens of the Qwen3-30B-A3B shape
    // 17.3 ms with two CTAs per SM worth of CTAs, 15.4 with four, 13.6 with six, 13.9 with ten)
    const uint32_t live = c.pairs < c.n_experts ? (c.pairs ? c.pairs : 1u) : c.n_experts;
    uint32_t ctas = (8u * ctx.sm_count + live - 1) / live;
    const uint32_t row_tiles = (c.rows + 16u * plan.row_tiles - 1) / (16u * plan.row_tiles);
    if (ctas > row_tiles) ctas = row_tiles;
    if (ctas < 1) ctas = 1;
    plan.ctas = ctas;
    MmaTileArgs ta = {};
    MmaArgs &a = ta.a;
    a.plan = plan;
    a.w[0] = c.w[0]; a.w[1] = c.w[1]; a.y = c.y;
    a.n_experts = c.n_experts; a.top = c.top ? c.top : 1u; a.glu = c.glu; a.status = ctx.status;
    a.na = static_cast<const float *>(c.x); a.npack = 1u;
    ta.tiles = tiles; ta.pairs = pairs; ta.gather = gather ? 1u : 0u; ta.per_pass = MMA_TILE_TOKENS;
    const dim3 grid(ctas, tile_capacity);
    switch (c.kind) {
    case KIND_Q4_K: err = c.nmat == 2 ? launch_tiles_t<KIND_Q4_K, 2>(ta, grid, ctx.stream, ctx.pdl) : launch_tiles_t<KIND_Q4_K, 1>(ta, grid, ctx.stream, ctx.pdl); break;
    case KIND_Q6_K: err = c.nmat == 2 ? launch_tiles_t<KIND_Q6_K, 2>(ta, grid, ctx.stream, ctx.pdl) : launch_tiles_t<KIND_Q6_K, 1>(ta, grid, ctx.stream, ctx.pdl); break;
    case KIND_Q4_0: err = c.nmat == 2 ? launch_tiles_t<KIND_Q4_0, 2>(ta, grid, ctx.stream, ctx.pdl) : launch_tiles_t<KIND_Q4_0, 1>(ta, grid, ctx.stream, ctx.pdl); break;
    default: err = c.nmat == 2 ? launch_tiles_t<KIND_Q8_0, 2>(ta, grid, ctx.stream, ctx.pdl) : launch_tiles_t<KIND_Q8_0, 1>(ta, grid, ctx.stream, ctx.pdl); break;
    }
    return true;
}

// Two or more float32 activation rows against ONE dense matrix: the rows are a single tile of the kernel above, so
// the weights stream once per four rows and every row's result has the bits the one-token kernel gives it (the
// reference's property that a token's projection does not depend on its batch: src/expert_bench.rs:698-712).
bool try_launch_gemv_rows(const GemvCall &c, const LaunchCtx &ctx, cudaError_t &err) {
    if (c.ids || c.count < 2 || !mma_kind(c.kind) || c.cols % 64u || c.x_packed || c.x_bf16 || ((uintptr_t)c.x % 16u) || c.norm_a) return false;
    if (((uintptr_t)c.w[0] % 16u) || (c.nmat == 2 && ((uintptr_t)c.w[1] % 16u)) || ((size_t)c.rows * c.stride) % 16u) return false;
    MmaPlan plan;
    // as many rows per pass as fit beside the ring (wide rows: 12288 columns take 55 KB each): four, two or one
    uint32_t per_pass = c.count < MMA_TILE_TOKENS ? c.count : MMA_TILE_TOKENS;
    bool ok = false, one_per_sm = false;
    for (; per_pass >= 1 && !ok; per_pass = ok ? per_pass : per_pass / 2u) {
        ok = plan_mma(c.kind, c.cols, c.rows, c.stride, c.nmat, 1u, MMA_SMEM_BUDGET, XM_FX4, plan, nullptr, MMA_TILE_TOKENS, per_pass);
        if (!ok && (ok = plan_mma(c.kind, c.cols, c.rows, c.stride, c.nmat, 1u, MMA_SMEM_MAX, XM_FX4, plan, nullptr, MMA_TILE_TOKENS, per_pass)))
            one_per_sm = true;
    }
    if (!ok) return false;
    const uint32_t row_tiles = (c.rows + 16u * plan.row_tiles - 1) / (16u * plan.row_tiles);
    uint32_t ctas = (one_per_sm ? 1u : 2u) * ctx.sm_count;
    if (ctas > row_tiles) ctas = row_tiles;
    plan.ctas = ctas;
    MmaTileArgs ta = {};
    MmaArgs &a = ta.a;
    a.plan = plan;
    a.w[0] = c.w[0]; a.w[1] = c.w[1]; a.y = c.y;
    a.n_experts = c.expert + 1u; a.top = 1u; a.glu = c.glu; a.status = ctx.status;
    a.na = static_cast<const float *>(c.x); a.npack = 1u;
    ta.dense_expert = c.expert; ta.dense_rows = c.count; ta.per_pass = per_pass;
    const dim3 grid(ctas, 1);
    switch (c.kind) {
    case KIND_Q4_K: err = c.nmat == 2 ? launch_tiles_t<KIND_Q4_K, 2>(ta, grid, ctx.stream, ctx.pdl) : launch_tiles_t<KIND_Q4_K, 1>(ta, grid, ctx.stream, ctx.pdl); break;
    case KIND_Q6_K: err = c.nmat == 2 ? launch_tiles_t<KIND_Q6_K, 2>(ta, grid, ctx.stream, ctx.pdl) : launch_tiles_t<KIND_Q6_K, 1>(ta, grid, ctx.stream, ctx.pdl); break;
    case KIND_Q4_0: err = c.nmat == 2 ? launch_tiles_t<KIND_Q4_0, 2>(ta, grid, ctx.stream, ctx.pdl) : launch_tiles_t<KIND_Q4_0, 1>(ta, grid, ctx.stream, ctx.pdl); break;
    default: err = c.nmat == 2 ? launch_tiles_t<KIND_Q8_0, 2>(ta, grid, ctx.stream, ctx.pdl) : launch_tiles_t<KIND_Q8_0, 1>(ta, grid, ctx.stream, ctx.pdl); break;
    }
    return true;
}

// Several independent one-token projections in one launch (what the reference's
// independent_projections scope expresses, e.g. q, k and v of one layer): CTAs
// [first[i], first[i + 1]) work on part i, each part with its own weight type, shape,
// inputs and plan.  Parts are ordered by size so that the long ones start first.
static constexpr uint32_t MMA_GROUP_MAX = 4;
struct MmaGroupArgs {
    MmaArgs part[MMA_GROUP_MAX];
    uint32_t first[MMA_GROUP_MAX + 1];
    uint32_t n;
};

// Two CTAs per SM: the Q6_K step needs the registers, and a three-per-SM form without it (smaller
// rings, a few spills) measured slower on an all-Q4_0 group (11.2 us against 6.7 us).
template <int XM, int LINK = LINK_NONE>
__global__ void __launch_bounds__(MMA_THREADS, 2) gemv_mma_group_kernel(const __grid_constant__ MmaGroupArgs ga) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint32_t i = 0;
    while (i + 1 < ga.n && blockIdx.x >= ga.first[i + 1]) ++i;
    const MmaArgs &a = ga.part[i];
    const uint32_t cta = blockIdx.x - ga.first[i], nctas = ga.first[i + 1] - ga.first[i];
    MmaRun run;
    switch (a.plan.kind) {
    case KIND_Q4_K: gemv_mma_body<KIND_Q4_K, 1, XM, MMA_WARPS, 1, LINK>(a, smem, cta, nctas, 0u, true, run); break;
    case KIND_Q6_K: gemv_mma_body<KIND_Q6_K, 1, XM, MMA_WARPS, 1, LINK>(a, smem, cta, nctas, 0u, true, run); break;
    case KIND_Q4_0: gemv_mma_body<KIND_Q4_0, 1, XM, MMA_WARPS, 1, LINK>(a, smem, cta, nctas, 0u, true, run); break;
    default: gemv_mma_body<KIND_Q8_0, 1, XM, MMA_WARPS, 1, LINK>(a, smem, cta, nctas, 0u, true, run); break;
    }
}

// ---------------------------------------------------------------------------
// Two to eight tokens at once (bfloat16 activations as high-part rows).
//
// The eight columns of the B operand are eight TOKENS: lane (g, t) supplies token g's
// activations, and the accumulator of an MMA holds rows g, g+8 for tokens 2t, 2t+1.
// A sub-block's MMAs chain into one accumulator, which is then scaled by that row's
// sub-block scale in fp32 and added to the lane's per-token sums; no group masking,
// every lane needs the scales of all sub-blocks of its two rows.  The weight bytes are
// streamed once for all tokens: about 1.3 times the instructions of the one-token kernel
// for eight times the work.  Q4_K and Q6_K, dense, rows whose step count is a multiple
// of eight (the eight warps split K), one CTA per SM.
// ---------------------------------------------------------------------------

static constexpr uint32_t MT_TOKENS = 8;
static constexpr uint32_t MT_RED_SLOTS = 6;
static constexpr int MT_MAX_STAGES = 4;

struct MtPlan {
    uint32_t kind, cols, rows, stride, nmat;
    uint32_t step_bytes, nsteps, spw, chunks, chunk_bytes, row_pitch;
    uint32_t stages, stage_bytes;
    uint32_t xrow_bytes;     // one token's packed row
    uint32_t xrow_pitch;     // its pitch in shared memory (32 mod 128: the eight token rows of a B-operand load hit different banks)
    uint32_t ntok;           // token rows held in shared memory (a multiple of 2, at most 8)
    uint32_t red_bytes, smem_bytes, ctas;
};

struct MtArgs {
    MtPlan p;
    const uint8_t *w[2];
    const uint8_t *xp;       // `count` high-part rows
    float *y;                // [count][rows]
    uint32_t count, expert, glu;
    int *status;
};

static bool plan_mt(uint32_t kind, uint32_t cols, uint32_t rows, uint32_t stride, uint32_t nmat, uint32_t count, uint32_t sm_count,
                    MtPlan &p) {
    if (kind != KIND_Q4_K && kind != KIND_Q6_K) return false;
    if (cols == 0 || rows == 0 || cols % 2048u || stride % 16u) return false;
    p.kind = kind; p.cols = cols; p.rows = rows; p.stride = stride; p.nmat = nmat;
    p.step_bytes = kind == KIND_Q4_K ? 144u : 210u;
    if (stride != cols / 256u * p.step_bytes) return false;
    p.nsteps = cols / 256u;
    p.xrow_bytes = packed_hi_bytes(cols);
    p.xrow_pitch = p.xrow_bytes + ((32u + 128u - (p.xrow_bytes % 128u)) % 128u);
    p.red_bytes = MT_RED_SLOTS * MMA_WARPS * 2u * 16u * MT_TOKENS * 4u;
    const uint32_t per_warp = p.nsteps / MMA_WARPS;
    // as many token rows as fit beside two stages
    for (p.ntok = MT_TOKENS; p.ntok >= 2; p.ntok -= 2) {
        const uint32_t fixed = MMA_BAR_BYTES + ((p.ntok * p.xrow_pitch + 127u) & ~127u) + p.red_bytes;
        if (fixed >= MMA_SMEM_MAX) continue;
        const uint32_t room = MMA_SMEM_MAX - fixed;
        uint32_t pick = 0;
        for (uint32_t spw = 1; spw <= per_warp; ++spw) {
            if (per_warp % spw) continue;
            const uint32_t cb = spw * MMA_WARPS * p.step_bytes;
            if (cb % 16u) continue;
            const uint32_t sb = (pitch_of(cb) * 16u + 127u) & ~127u;
            if (room / sb < 2) break;
            if (pick == 0 || sb <= MMA_STAGE_TARGET) pick = spw;
        }
        if (!pick) continue;
        p.spw = pick;
        p.chunks = per_warp / pick;
        p.chunk_bytes = pick * MMA_WARPS * p.step_bytes;
        p.row_pitch = pitch_of(p.chunk_bytes);
        p.stage_bytes = (p.row_pitch * 16u + 127u) & ~127u;
        p.stages = room / p.stage_bytes;
        if (p.stages > (uint32_t)MT_MAX_STAGES) p.stages = MT_MAX_STAGES;
        p.smem_bytes = fixed + p.stages * p.stage_bytes;
        break;
    }
    if (p.ntok < 2) return false;
    if (p.ntok > ((count + 1u) & ~1u)) p.ntok = (count + 1u) & ~1u;       // no more rows than there are tokens
    const uint32_t want = (rows + 15u) / 16u;
    p.ctas = want < sm_count ? want : sm_count;
    return true;
}

template <uint32_t KIND> struct MtStep;

// xs: this lane's token row at the step, plus 8 t (its k slots); s0 / s1: the 16-column sums of
// tokens 2t and 2t+1 at the step; acc: rows g, g+8 x tokens 2t, 2t+1
template <> struct MtStep<KIND_Q4_K> {
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, const uint8_t *xs, const float *s0, const float *s1,
                                               uint32_t t, float (&acc)[4], bool) {
        const U4 h0 = *reinterpret_cast<const U4 *>(r0), h1 = *reinterpret_cast<const U4 *>(r1);
        const float2 d0 = __half22float2(*reinterpret_cast<const __half2 *>(&h0.x)), d1 = __half22float2(*reinterpret_cast<const __half2 *>(&h1.x));
        // six-bit scales and mins of sub-blocks 0..3 (lo words) and 4..7 (hi words), one per byte
        const uint32_t sc0[2] = {h0.y & 0x3f3f3f3fu, (h0.w & 0x0f0f0f0fu) | ((h0.y >> 2) & 0x30303030u)};
        const uint32_t mn0[2] = {h0.z & 0x3f3f3f3fu, ((h0.w >> 4) & 0x0f0f0f0fu) | ((h0.z >> 2) & 0x30303030u)};
        const uint32_t sc1[2] = {h1.y & 0x3f3f3f3fu, (h1.w & 0x0f0f0f0fu) | ((h1.y >> 2) & 0x30303030u)};
        const uint32_t mn1[2] = {h1.z & 0x3f3f3f3fu, ((h1.w >> 4) & 0x0f0f0f0fu) | ((h1.z >> 2) & 0x30303030u)};
        const uint8_t *q0 = r0 + 16u + 4u * t, *q1 = r1 + 16u + 4u * t;
        float p[4] = {0.f, 0.f, 0.f, 0.f}, m[4] = {0.f, 0.f, 0.f, 0.f};     // scaled products and min terms of the step
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            float lo[4], hi[4];
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h) {
                const uint32_t a = lds32(q0 + 32u * j + 16u * h), b = lds32(q1 + 32u * j + 16u * h);
                const uint32_t as = a >> 8, bs = b >> 8;
                const uint2 bl = *reinterpret_cast<const uint2 *>(xs + (4u * j + h) * 32u);
                const uint2 bh = *reinterpret_cast<const uint2 *>(xs + (4u * j + 2u + h) * 32u);
                if (h == 0) {
                    mma16816_first(lo, a & 0x000f000fu, b & 0x000f000fu, as & 0x000f000fu, bs & 0x000f000fu, bl.x, bl.y);
                    mma16816_first(hi, a & 0x00f000f0u, b & 0x00f000f0u, as & 0x00f000f0u, bs & 0x00f000f0u, bh.x, bh.y);
                } else {
                    mma16816(lo, a & 0x000f000fu, b & 0x000f000fu, as & 0x000f000fu, bs & 0x000f000fu, bl.x, bl.y);
                    mma16816(hi, a & 0x00f000f0u, b & 0x00f000f0u, as & 0x00f000f0u, bs & 0x00f000f0u, bh.x, bh.y);
                }
            }
            // sub-blocks 2j (low nibbles) and 2j+1 (high nibbles, kept in place as 16 q)
            const uint32_t wsel = j >> 1, bsel = 16u * (j & 1u);
            const float a_lo = (float)((sc0[wsel] >> bsel) & 0xffu), a_hi = mul_rn((float)((sc0[wsel] >> (bsel + 8u)) & 0xffu), 0.0625f);
            const float b_lo = (float)((sc1[wsel] >> bsel) & 0xffu), b_hi = mul_rn((float)((sc1[wsel] >> (bsel + 8u)) & 0xffu), 0.0625f);
            const float am_lo = (float)((mn0[wsel] >> bsel) & 0xffu), am_hi = (float)((mn0[wsel] >> (bsel + 8u)) & 0xffu);
            const float bm_lo = (float)((mn1[wsel] >> bsel) & 0xffu), bm_hi = (float)((mn1[wsel] >> (bsel + 8u)) & 0xffu);
            const float4 u0 = *reinterpret_cast<const float4 *>(s0 + 4u * j), u1 = *reinterpret_cast<const float4 *>(s1 + 4u * j);
            const float x0l = add_rn(u0.x, u0.y), x0h = add_rn(u0.z, u0.w), x1l = add_rn(u1.x, u1.y), x1h = add_rn(u1.z, u1.w);
            p[0] = fma_rn(a_hi, hi[0], fma_rn(a_lo, lo[0], p[0]));
            p[1] = fma_rn(a_hi, hi[1], fma_rn(a_lo, lo[1], p[1]));
            p[2] = fma_rn(b_hi, hi[2], fma_rn(b_lo, lo[2], p[2]));
            p[3] = fma_rn(b_hi, hi[3], fma_rn(b_lo, lo[3], p[3]));
            m[0] = fma_rn(am_hi, x0h, fma_rn(am_lo, x0l, m[0]));
            m[1] = fma_rn(am_hi, x1h, fma_rn(am_lo, x1l, m[1]));
            m[2] = fma_rn(bm_hi, x0h, fma_rn(bm_lo, x0l, m[2]));
            m[3] = fma_rn(bm_hi, x1h, fma_rn(bm_lo, x1l, m[3]));
        }
        const float e0 = mul_rn(d0.x, SUBNORMAL_SCALE), e1 = mul_rn(d1.x, SUBNORMAL_SCALE);
        acc[0] = add_rn(acc[0], sub_rn(mul_rn(e0, p[0]), mul_rn(d0.y, m[0])));
        acc[1] = add_rn(acc[1], sub_rn(mul_rn(e0, p[1]), mul_rn(d0.y, m[1])));
        acc[2] = add_rn(acc[2], sub_rn(mul_rn(e1, p[2]), mul_rn(d1.y, m[2])));
        acc[3] = add_rn(acc[3], sub_rn(mul_rn(e1, p[3]), mul_rn(d1.y, m[3])));
    }
};

template <> struct MtStep<KIND_Q6_K> {
    template <int Q>
    static __device__ __forceinline__ uint32_t six(uint32_t L, uint32_t H) { return MmaStep<KIND_Q6_K>::six<Q>(L, H); }
    template <int Q>
    static __device__ __forceinline__ void run16(uint32_t la, uint32_t lb, uint32_t ha, uint32_t hb, uint2 bf, float sa, float sb, float x0,
                                                 float x1, float (&p)[4]) {
        float c[4];
        mma16816_first(c, six<Q>(la, ha), six<Q>(lb, hb), six<Q>(la >> 8, ha >> 8), six<Q>(lb >> 8, hb >> 8), bf.x, bf.y);
        constexpr float up = (Q < 2) ? SUBNORMAL_SCALE : SUBNORMAL_SCALE * 0.0625f;       // x16 of the in-place high nibble undone
        p[0] = fma_rn(sa, fma_rn(c[0], up, x0), p[0]);
        p[1] = fma_rn(sa, fma_rn(c[1], up, x1), p[1]);
        p[2] = fma_rn(sb, fma_rn(c[2], up, x0), p[2]);
        p[3] = fma_rn(sb, fma_rn(c[3], up, x1), p[3]);
    }
    // mis: the block starts 2 bytes past a 4-byte boundary
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, const uint8_t *xs, const float *s0, const float *s1,
                                               uint32_t t, float (&acc)[4], bool mis) {
        const float d0 = lds_half(r0 + 208u), d1 = lds_half(r1 + 208u);
        float p[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (uint32_t n = 0; n < 2; ++n) {
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h) {
                const uint32_t o = 64u * n + 16u * h + 4u * t;
                const uint32_t oh = 128u + 32u * n + 16u * h + 4u * t;
                const uint32_t a_lo = lds32_known(r0 + o, mis), a_hi = lds32_known(r0 + o + 32u, mis), a_h = lds32_known(r0 + oh, mis);
                const uint32_t b_lo = lds32_known(r1 + o, mis), b_hi = lds32_known(r1 + o + 32u, mis), b_h = lds32_known(r1 + oh, mis);
#pragma unroll
                for (uint32_t q = 0; q < 4; ++q) {
                    // run (n, q, h): 16 columns, MMA index 8n + 2q + h, its own int8 scale and activation sum
                    const uint32_t idx = 8u * n + 2u * q + h;
                    const float sa = (float)(int)*reinterpret_cast<const int8_t *>(r0 + 192u + idx);
                    const float sb = (float)(int)*reinterpret_cast<const int8_t *>(r1 + 192u + idx);
                    const float x0 = mul_rn(s0[idx], -32.0f), x1 = mul_rn(s1[idx], -32.0f);
                    const uint2 bf = *reinterpret_cast<const uint2 *>(xs + idx * 32u);
                    if (q == 0) run16<0>(a_lo, b_lo, a_h, b_h, bf, sa, sb, x0, x1, p);
                    else if (q == 1) run16<1>(a_hi, b_hi, a_h, b_h, bf, sa, sb, x0, x1, p);
                    else if (q == 2) run16<2>(a_lo, b_lo, a_h, b_h, bf, sa, sb, x0, x1, p);
                    else run16<3>(a_hi, b_hi, a_h, b_h, bf, sa, sb, x0, x1, p);
                }
            }
        }
        acc[0] = fma_rn(d0, p[0], acc[0]);
        acc[1] = fma_rn(d0, p[1], acc[1]);
        acc[2] = fma_rn(d1, p[2], acc[2]);
        acc[3] = fma_rn(d1, p[3], acc[3]);
    }
};

template <uint32_t KIND, int NMAT>
__global__ void __launch_bounds__(MMA_THREADS, 1) gemv_mt_kernel(const __grid_constant__ MtArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const MtPlan &p = a.p;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + MT_MAX_STAGES;
    uint64_t *xbar = empty + MT_MAX_STAGES;
    uint64_t *tbar = xbar + 1;                                   // [MT_RED_SLOTS]
    uint8_t *xrows = smem + MMA_BAR_BYTES;
    float *red = reinterpret_cast<float *>(xrows + ((p.ntok * p.xrow_pitch + 127u) & ~127u));
    uint8_t *stages = reinterpret_cast<uint8_t *>(red) + p.red_bytes;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], MMA_WARPS);
        }
        ptx::mbar_init(xbar, 1);
        for (uint32_t i = 0; i < MT_RED_SLOTS; ++i) ptx::mbar_init(&tbar[i], MMA_WARPS);
        ptx::mbar_init_fence();
    }
    __syncthreads();
    ptx::pdl_launch_dependents();

    uint32_t r_begin, r_end;
    cta_rows(p.rows, blockIdx.x, gridDim.x, r_begin, r_end);
    const uint32_t n_tiles = (r_end - r_begin + 15u) / 16u;
    const uint32_t live = a.count < p.ntok ? a.count : p.ntok;          // token rows to fetch

    if (warp == MMA_WARPS) {
        // ---- producer warp ----
        const size_t mat_off = (size_t)a.expert * p.rows * p.stride;
        bool x_sent = false;
        uint32_t it = 0;
        auto send_x = [&]() {
            ptx::pdl_wait();
            if (lane == 0) ptx::mbar_expect_tx(xbar, live * p.xrow_bytes);
            __syncwarp();
            if (lane < live) ptx::bulk_g2s(xrows + (size_t)lane * p.xrow_pitch, a.xp + (size_t)lane * p.xrow_bytes, p.xrow_bytes, xbar);
            x_sent = true;
        };
        for (uint32_t tile = 0; tile < n_tiles; ++tile) {
            const uint32_t row0 = r_begin + tile * 16u;
            const uint32_t nrows = (r_end - row0) < 16u ? (r_end - row0) : 16u;
            for (uint32_t cm = 0; cm < p.chunks * NMAT; ++cm, ++it) {
                const uint32_t c = cm / NMAT, m = cm - c * NMAT;
                if (!x_sent && it == p.stages) send_x();
                const uint32_t s = it % p.stages, ph = (it / p.stages) & 1u;
                bool ok = true;
                if (lane == 0) ok = ptx::mbar_wait_sleep<128>(&empty[s], ph ^ 1u);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { if (lane == 0) set_status_word(a.status, KERNEL_ERR_PRODUCER_TIMEOUT); return; }
                uint8_t *dst = stages + (size_t)s * p.stage_bytes;
                if (lane == 0) ptx::mbar_expect_tx(&full[s], p.chunk_bytes * nrows);
                __syncwarp();
                if (lane < nrows)
                    ptx::bulk_g2s(dst + (size_t)lane * p.row_pitch, a.w[m] + mat_off + (size_t)(row0 + lane) * p.stride + (size_t)c * p.chunk_bytes,
                                  p.chunk_bytes, &full[s]);
            }
        }
        if (!x_sent) send_x();
        return;
    }

    // ---- consumer warps: warp kw takes steps kw, kw + 8, ... of the row ----
    if (!ptx::mbar_wait(xbar, 0)) {
        if (lane == 0) set_status_word(a.status, KERNEL_ERR_CONSUMER_TIMEOUT);
        return;
    }
    ptx::pdl_wait();
    const uint32_t g = lane >> 2, t = lane & 3u, kw = warp;
    // the lane's own token row (token g) for the B operand, the rows of tokens 2t and 2t+1 for their sums;
    // tokens past the fetched rows read row 0 (their results are never stored)
    const uint32_t tg = g < live ? g : 0u, t0 = 2u * t < live ? 2u * t : 0u, t1 = 2u * t + 1u < live ? 2u * t + 1u : 0u;
    const uint8_t *xlane = xrows + (size_t)tg * p.xrow_pitch + t * 8u;
    const float *sum0 = reinterpret_cast<const float *>(xrows + (size_t)t0 * p.xrow_pitch + (size_t)p.cols * 2u);
    const float *sum1 = reinterpret_cast<const float *>(xrows + (size_t)t1 * p.xrow_pitch + (size_t)p.cols * 2u);
    const uint32_t step_stride = p.step_bytes * MMA_WARPS;

    auto sum_tile = [&](uint32_t tile) -> bool {
        if (((tile ^ kw) & 7u) != 0u) return true;                     // another warp's turn
        const uint32_t slot_id = tile % MT_RED_SLOTS;
        const float *slot = red + (size_t)slot_id * MMA_WARPS * 2u * 16u * MT_TOKENS;
        if (!ptx::mbar_wait_sleep<20>(&tbar[slot_id], (tile / MT_RED_SLOTS) & 1u)) {
            if (lane == 0) set_status_word(a.status, KERNEL_ERR_CONSUMER_TIMEOUT);
            return false;
        }
        const uint32_t row0 = r_begin + tile * 16u;
        const uint32_t nrows = (r_end - row0) < 16u ? (r_end - row0) : 16u;
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {                               // 128 (row, token) outputs, four per lane
            const uint32_t o = lane + 32u * j, row = o >> 3, tok = o & 7u;
            float v[NMAT];
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                float sum = 0.f;
#pragma unroll
                for (uint32_t k = 0; k < (uint32_t)MMA_WARPS; ++k) sum = add_rn(sum, slot[((k * 2u + m) * 16u + row) * MT_TOKENS + tok]);
                v[m] = sum;
            }
            if (row < nrows && tok < live) {
                const float unscale = *reinterpret_cast<const float *>(xrows + (size_t)tok * p.xrow_pitch + (size_t)p.cols * 2u + p.cols / 4u);
                const float y0 = mul_rn(v[0], unscale);
                a.y[(size_t)tok * p.rows + row0 + row] = NMAT == 2 ? glu_f(y0, mul_rn(v[NMAT - 1], unscale), a.glu == 2) : y0;
            }
        }
        return true;
    };

    uint32_t it = 0;
    for (uint32_t tile = 0; tile < n_tiles; ++tile) {
        const uint32_t row0 = r_begin + tile * 16u;
        const uint32_t nrows = (r_end - row0) < 16u ? (r_end - row0) : 16u;
        const uint32_t ur0 = g < nrows ? g : 0u, ur1 = g + 8u < nrows ? g + 8u : 0u;      // rows past the end read the tile's first row
        float acc[NMAT][4];
#pragma unroll
        for (int m = 0; m < NMAT; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
        for (uint32_t c = 0; c < p.chunks; ++c) {
            const uint32_t gs0 = c * (p.spw * MMA_WARPS) + kw;                 // first step of this warp in the chunk
#pragma unroll
            for (int m = 0; m < NMAT; ++m, ++it) {
                const uint32_t s = it % p.stages, ph = (it / p.stages) & 1u;
                if (!ptx::mbar_wait_sleep<20>(&full[s], ph)) {
                    if (lane == 0) set_status_word(a.status, KERNEL_ERR_CONSUMER_TIMEOUT);
                    return;
                }
                const uint8_t *st = stages + (size_t)s * p.stage_bytes;
                const uint8_t *b0 = st + (size_t)ur0 * p.row_pitch + kw * p.step_bytes;
                const uint8_t *b1 = st + (size_t)ur1 * p.row_pitch + kw * p.step_bytes;
                for (uint32_t i = 0; i < p.spw; ++i) {
                    const uint32_t step = gs0 + i * MMA_WARPS;                 // 256 columns: 16 MMAs of 32 packed bytes, 16 sums
                    // rows start on 16-byte boundaries in the stage and this warp's steps are kw, kw + 8, ...:
                    // its Q6_K blocks (210 bytes) all start 2 bytes past a 4-byte boundary when kw is odd
                    if (KIND == KIND_Q6_K && (kw & 1u))
                        MtStep<KIND>::run(b0, b1, xlane + (size_t)step * 512u, sum0 + step * 16u, sum1 + step * 16u, t, acc[m], true);
                    else
                        MtStep<KIND>::run(b0, b1, xlane + (size_t)step * 512u, sum0 + step * 16u, sum1 + step * 16u, t, acc[m], false);
                    b0 += step_stride; b1 += step_stride;
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&empty[s]);
            }
        }
        const uint32_t slot_id = tile % MT_RED_SLOTS;
        float *slot = red + (size_t)slot_id * MMA_WARPS * 2u * 16u * MT_TOKENS;
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
            float *dst = slot + (size_t)(warp * 2u + m) * 16u * MT_TOKENS;
            *reinterpret_cast<float2 *>(dst + g * MT_TOKENS + 2u * t) = make_float2(acc[m][0], acc[m][1]);
            *reinterpret_cast<float2 *>(dst + (g + 8u) * MT_TOKENS + 2u * t) = make_float2(acc[m][2], acc[m][3]);
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&tbar[slot_id]);
        if (tile > 0 && !sum_tile(tile - 1)) return;
    }
    if (n_tiles > 0) sum_tile(n_tiles - 1);
}

template <uint32_t KIND, int NMAT>
static cudaError_t launch_mt_t(const MtArgs &a, cudaStream_t stream, bool pdl) {
    auto kernel = gemv_mt_kernel<KIND, NMAT>;
    static DeviceOnce once;
    {
        const cudaError_t e = once.smem(kernel, (int)MMA_SMEM_MAX);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.p.ctas);
    cfg.blockDim = dim3(MMA_THREADS);
    cfg.dynamicSmemBytes = a.p.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, a);
}

// Dense projection of `count` (2..) tokens whose activations are high-part rows; tokens go through in
// groups of as many rows as fit in shared memory.  False when the call is not one it handles.
bool try_launch_gemv_mt(const GemvCall &c, const LaunchCtx &ctx, cudaError_t &err) {
    if (c.ids || c.x_packed != 4u || c.count < 1) return false;
    MtPlan plan;
    if (!plan_mt(c.kind, c.cols, c.rows, c.stride, c.nmat, c.count, ctx.sm_count, plan)) return false;
    err = cudaSuccess;
    for (uint32_t first = 0; first < c.count && err == cudaSuccess; first += plan.ntok) {
        MtArgs a = {};
        a.p = plan;
        a.w[0] = c.w[0]; a.w[1] = c.w[1];
        a.xp = static_cast<const uint8_t *>(c.x) + (size_t)first * plan.xrow_bytes;
        a.y = c.y + (size_t)first * c.rows;
        a.count = c.count - first < plan.ntok ? c.count - first : plan.ntok;
        a.expert = c.expert; a.glu = c.glu; a.status = ctx.status;
        if (c.kind == KIND_Q4_K) err = c.nmat == 2 ? launch_mt_t<KIND_Q4_K, 2>(a, ctx.stream, ctx.pdl) : launch_mt_t<KIND_Q4_K, 1>(a, ctx.stream, ctx.pdl);
        else err = c.nmat == 2 ? launch_mt_t<KIND_Q6_K, 2>(a, ctx.stream, ctx.pdl) : launch_mt_t<KIND_Q6_K, 1>(a, ctx.stream, ctx.pdl);
    }
    return true;
}

// ---------------------------------------------------------------------------
// launch
// ---------------------------------------------------------------------------

template <uint32_t KIND, int NMAT, int OCC, int XM, int LINK = LINK_NONE>
static cudaError_t launch_mma_t(const MmaArgs &a, dim3 grid, cudaStream_t stream, bool pdl) {
    auto kernel = gemv_mma_kernel<KIND, NMAT, OCC, XM, LINK>;
    static DeviceOnce once;
    {
        const cudaError_t e = once.smem(kernel, (int)(OCC == 3 ? MMA_SMEM_SMALL : MMA_SMEM_MAX));
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(MMA_THREADS);
    cfg.dynamicSmemBytes = a.plan.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, a);
}

template <uint32_t KIND, int XM, int LINK = LINK_NONE>
static cudaError_t launch_mma_h(const MmaArgs &a, dim3 grid, cudaStream_t stream, bool pdl, int occ) {
    if (occ == 3)
        return a.plan.nmat == 2 ? launch_mma_t<KIND, 2, 3, XM, LINK>(a, grid, stream, pdl) : launch_mma_t<KIND, 1, 3, XM, LINK>(a, grid, stream, pdl);
    return a.plan.nmat == 2 ? launch_mma_t<KIND, 2, 2, XM, LINK>(a, grid, stream, pdl) : launch_mma_t<KIND, 1, 2, XM, LINK>(a, grid, stream, pdl);
}
// Which form of the exchange a projection needs (the specialised forms exist for the K-quant matrices with
// bfloat16-rounded rows, what a sharded decode step runs; everything else takes the run-time form).
static int link_of(const MmaArgs &a) {
    if (!a.tp.n_out && !a.tp.in[0] && !a.tp.in[1]) return LINK_NONE;
    if (a.plan.xm != XM_FX2 || (a.plan.kind != KIND_Q4_K && a.plan.kind != KIND_Q6_K)) return LINK_ANY;
    if (a.tp.in[0] && a.tp.in[1]) return LINK_ANY;
    return a.tp.in[0] ? LINK_A : a.tp.in[1] ? LINK_B : LINK_OUT;
}
template <uint32_t KIND>
static cudaError_t launch_mma_k(const MmaArgs &a, dim3 grid, cudaStream_t stream, bool pdl, int occ) {
    const int link = link_of(a);
    if (link != LINK_NONE) {              // the exchange lives in the fused-norm (fixed-point row) forms only
        if constexpr (KIND == KIND_Q4_K || KIND == KIND_Q6_K) {
            if (link == LINK_OUT) return launch_mma_h<KIND, XM_FX2, LINK_OUT>(a, grid, stream, pdl, occ);
            if (link == LINK_A) return launch_mma_h<KIND, XM_FX2, LINK_A>(a, grid, stream, pdl, occ);
            if (link == LINK_B) return launch_mma_h<KIND, XM_FX2, LINK_B>(a, grid, stream, pdl, occ);
        }
        if (a.plan.xm == XM_FX2) return launch_mma_h<KIND, XM_FX2, LINK_ANY>(a, grid, stream, pdl, occ);
        if (a.plan.xm == XM_FX4) return launch_mma_h<KIND, XM_FX4, LINK_ANY>(a, grid, stream, pdl, occ);
        return cudaErrorInvalidValue;
    }
    switch (a.plan.xm) {
    case XM_F16: return launch_mma_h<KIND, XM_F16>(a, grid, stream, pdl, occ);
    case XM_F16_HI: return launch_mma_h<KIND, XM_F16_HI>(a, grid, stream, pdl, occ);
    case XM_FX2: return launch_mma_h<KIND, XM_FX2>(a, grid, stream, pdl, occ);
    default: return launch_mma_h<KIND, XM_FX4>(a, grid, stream, pdl, occ);
    }
}

// The activation row form of a call: the CTAs build fixed-point rows themselves when they norm or
// pack the activations; rows packed beforehand are binary16.
static uint32_t x_mode_of(const GemvCall &c, bool pack_inside) {
    if (c.norm_a) return (c.norm_round_bf16 && !c.norm_wide) ? XM_FX2 : XM_FX4;
    if (pack_inside) return XM_FX4;
    return c.x_packed == 4u ? XM_F16_HI : XM_F16;
}

// True when this call was taken (launched or failed); false to let the caller use
// another kernel.  Unpacked activations are packed into the handle's workspace first.
bool try_launch_gemv_mma(const GemvCall &c, const LaunchCtx &ctx, cudaError_t &err) {
    const bool routed = c.ids != nullptr;
    if (!mma_kind(c.kind)) return false;
    if (!routed && c.count != 1) return false;
    if (c.cols % 64u) return false;
    const uint32_t gy = routed ? c.pairs : 1u;
    // CTAs per pair are sized for the pairs that are live on this device
    const uint32_t ep = routed && ctx.ep_world > 1 ? ctx.ep_world : 1u;
    const uint32_t gy_live = (gy + ep - 1) / ep;
    // bfloat16 activations are exact in the high binary16 part alone: the fused norm with bfloat16
    // rounding, and rows packed that way, carry no low part
    // plain float32 rows are packed by the CTAs themselves (one launch, as the reference's matmul is)
    const bool pack_inside = !c.norm_a && !c.x_packed && !c.x_bf16 && ((uintptr_t)c.x % 16u) == 0;
    const uint32_t xmode = x_mode_of(c, pack_inside);
    MmaPlan plan;
    int occ = 3;
    uint32_t max_ctas = (3u * ctx.sm_count + gy_live - 1) / gy_live;
    // (many live pairs: two waves of shorter CTAs, for the same reason as in the expert-grouped kernel; 128 live
    // pairs per device 10.8 -> 10.0 ms per step, 32 live pairs 4.4 -> 4.1 ms; with a handful of pairs it costs time,
    // and so it does when most of the grid is pairs of other devices, whose CTAs only leave: 32 live pairs of 256
    // on eight devices 6.1 -> 6.9 ms)
    if (routed && gy_live >= 16u && gy <= 2u * gy_live) max_ctas = (6u * ctx.sm_count + gy_live - 1) / gy_live;
    // Two or three CTAs per SM (dense launches).  Two have deeper rings: a matrix whose 16-row tiles all fit in one
    // wave of two holds a CTA's whole share in its ring, so the copies of one launch run under the tail of the launch
    // before it (4096 x 4096 Q4_K: 6.3 us against 7.6 us back to back).  Three pay only in the steady state of a
    // long stream (the 151936-row head: 93 us against 100 us with two); with a few tiles per CTA (gate/up: 3.5) two
    // give the same launch time and a shorter token step (2.25 against 2.30 ms: the next launch's CTAs find room
    // earlier).  Measured exceptions that keep three: the 18- and 34-byte block formats, which issue more
    // instructions per byte (Gemma's Q4_0 step 1.97 ms with two against 1.79 ms), and projections that exchange
    // their rows with other GPUs (two-GPU step 2.30 ms with two against 2.23 ms).
    const uint64_t tiles16 = (c.rows + 15u) / 16u;
    const bool exchanges = c.tp.n_out || c.tp.in[0] || c.tp.in[1];
    const bool k_quant = c.kind == KIND_Q4_K || c.kind == KIND_Q6_K;
    const bool prefers_two = tiles16 <= 2ull * ctx.sm_count || (k_quant && !exchanges && tiles16 * c.nmat < 24ull * ctx.sm_count);
    const bool long_stream = !prefers_two;
    bool ok = !(gy_live == 1 && !long_stream) &&
              plan_mma(c.kind, c.cols, c.rows, c.stride, c.nmat, max_ctas, MMA_SMEM_SMALL, xmode, plan);
    if (!ok) {
        occ = 2;
        max_ctas = (2u * ctx.sm_count + gy_live - 1) / gy_live;
        if (max_ctas < 1) max_ctas = 1;
        ok = plan_mma(c.kind, c.cols, c.rows, c.stride, c.nmat, max_ctas, MMA_SMEM_BUDGET, xmode, plan);
    }
    if (!ok) {
        max_ctas = (ctx.sm_count + gy_live - 1) / gy_live;
        ok = plan_mma(c.kind, c.cols, c.rows, c.stride, c.nmat, max_ctas ? max_ctas : 1, MMA_SMEM_MAX, xmode, plan);
    }
    if (!ok) return false;
    if (gy_live == 1) {
        // A one-wave grid that leaves every CTA with part of a 16-row tile pays the whole tile's
        // arithmetic in each of them.  When one full tile per CTA puts fewer tiles on the busiest
        // SM, take that grid instead (4096 rows: 256 CTAs, two per SM at most, instead of 444
        // CTAs of 9 or 10 rows, three per SM).
        const uint32_t tile_rows = 16u * plan.row_tiles;
        const uint32_t tiles = (c.rows + tile_rows - 1) / tile_rows;
        const uint32_t rows_per_cta = (c.rows + plan.ctas - 1) / plan.ctas;
        const uint32_t load_now = ((plan.ctas + ctx.sm_count - 1) / ctx.sm_count) * ((rows_per_cta + tile_rows - 1) / tile_rows);
        const uint32_t load_full = (tiles + ctx.sm_count - 1) / ctx.sm_count;
        if (tiles <= plan.ctas && load_full < load_now) plan.ctas = tiles;
    }
    const uint8_t *xp = static_cast<const uint8_t *>(c.x);
    if (c.norm_a) {
        if (routed || c.cols % 64u) return false;
        xp = nullptr;
    } else if (pack_inside) {
        xp = nullptr;
    } else if (!c.x_packed) {
        const uint32_t x_rows = routed ? (c.per_pair ? c.pairs : (c.pairs + (c.top ? c.top : 1u) - 1) / (c.top ? c.top : 1u)) : 1u;
        const size_t need = (size_t)x_rows * packed_x_bytes(c.cols);
        if (!ctx.workspace || need > ctx.workspace_bytes) return false;
        err = launch_pack_x(c.x, c.x_bf16, x_rows, c.cols, ctx.workspace, ctx);
        if (err != cudaSuccess) return true;
        xp = static_cast<const uint8_t *>(ctx.workspace);
    }
    MmaArgs a = {};
    a.plan = plan;
    a.w[0] = c.w[0]; a.w[1] = c.w[1]; a.xp = xp; a.y = c.y;
    a.ids = c.ids; a.expert = c.expert; a.n_experts = c.n_experts;
    a.per_pair = c.per_pair; a.top = c.top ? c.top : 1u; a.glu = c.glu;
    a.status = ctx.status;
    a.na = c.norm_a; a.nb = c.norm_b; a.nw = c.norm_w; a.ns = c.norm_s; a.neps = c.norm_eps; a.nround_bf16 = c.norm_round_bf16;
    a.tp = c.tp;
    if ((a.tp.n_out || a.tp.in[0] || a.tp.in[1]) && !a.na) return false;      // the exchange is built into the fused-norm form only
    if (pack_inside) { a.na = static_cast<const float *>(c.x); a.npack = 1u; }
    const dim3 grid(plan.ctas, gy);
    switch (c.kind) {
    case KIND_Q4_K: err = launch_mma_k<KIND_Q4_K>(a, grid, ctx.stream, ctx.pdl, occ); break;
    case KIND_Q6_K: err = launch_mma_k<KIND_Q6_K>(a, grid, ctx.stream, ctx.pdl, occ); break;
    case KIND_Q4_0: err = launch_mma_k<KIND_Q4_0>(a, grid, ctx.stream, ctx.pdl, occ); break;
    default: err = launch_mma_k<KIND_Q8_0>(a, grid, ctx.stream, ctx.pdl, occ); break;
    }
    return true;
}

// One-token dense projections that can share a launch: the checks of try_launch_gemv_mma for a
// call whose activations need no packing pass (packed rows, or the fused norm).
bool gemv_mma_group_eligible(const GemvCall &c, const LaunchCtx &ctx) {
    if (c.ids || c.count != 1 || c.nmat != 1 || !mma_kind(c.kind) || c.cols % 64u) return false;
    if (!c.norm_a && c.x_packed != 1u && c.x_packed != 4u) return false;
    MmaPlan plan;
    return plan_mma(c.kind, c.cols, c.rows, c.stride, 1, 2u * ctx.sm_count, MMA_SMEM_BUDGET, x_mode_of(c, false), plan);
}

template <int XM, int LINK = LINK_NONE>
static cudaError_t launch_mma_group_t(const MmaGroupArgs &ga, uint32_t smem_bytes, cudaStream_t stream, bool pdl) {
    auto kernel = gemv_mma_group_kernel<XM, LINK>;
    static DeviceOnce once;
    {
        const cudaError_t e = once.smem(kernel, (int)MMA_SMEM_BUDGET);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ga.first[ga.n]);
    cfg.blockDim = dim3(MMA_THREADS);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, ga);
}

// Loads the exchange forms of the kernels onto the current device.  A module is otherwise loaded at a kernel's
// first launch, which can take longer than a peer's bounded wait for this rank's rows in the very first step.
template <uint32_t KIND, int XM, int LINK>
static cudaError_t preload_link_kind() {
    cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel<KIND, 1, 3, XM, LINK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MMA_SMEM_SMALL);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_mma_kernel<KIND, 2, 3, XM, LINK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MMA_SMEM_SMALL);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_mma_kernel<KIND, 1, 2, XM, LINK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MMA_SMEM_MAX);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_mma_kernel<KIND, 2, 2, XM, LINK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MMA_SMEM_MAX);
    return e;
}
cudaError_t preload_exchange_kernels() {
    cudaError_t e = preload_link_kind<KIND_Q4_K, XM_FX2, LINK_OUT>();
    if (e == cudaSuccess) e = preload_link_kind<KIND_Q4_K, XM_FX2, LINK_A>();
    if (e == cudaSuccess) e = preload_link_kind<KIND_Q4_K, XM_FX2, LINK_B>();
    if (e == cudaSuccess) e = preload_link_kind<KIND_Q6_K, XM_FX2, LINK_OUT>();
    if (e == cudaSuccess) e = preload_link_kind<KIND_Q6_K, XM_FX2, LINK_A>();
    if (e == cudaSuccess) e = preload_link_kind<KIND_Q6_K, XM_FX2, LINK_B>();
    if (e == cudaSuccess) e = preload_link_kind<KIND_Q4_K, XM_FX2, LINK_ANY>();
    if (e == cudaSuccess) e = preload_link_kind<KIND_Q6_K, XM_FX2, LINK_ANY>();
    if (e == cudaSuccess) e = preload_link_kind<KIND_Q4_K, XM_FX4, LINK_ANY>();
    if (e == cudaSuccess) e = preload_link_kind<KIND_Q6_K, XM_FX4, LINK_ANY>();
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_mma_group_kernel<XM_FX2, LINK_OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MMA_SMEM_BUDGET);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_mma_group_kernel<XM_FX2, LINK_A>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MMA_SMEM_BUDGET);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_mma_group_kernel<XM_FX2, LINK_B>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MMA_SMEM_BUDGET);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_mma_group_kernel<XM_FX2, LINK_ANY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MMA_SMEM_BUDGET);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_mma_group_kernel<XM_FX4, LINK_ANY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MMA_SMEM_BUDGET);
    return e;
}

// Launches 2..MMA_GROUP_MAX eligible calls as one grid.  False (nothing launched) when they
// cannot share one: different activation row forms, or a part that does not plan.
bool try_launch_gemv_mma_group(const GemvCall *calls, uint32_t n, const LaunchCtx &ctx, cudaError_t &err) {
    if (n < 2 || n > MMA_GROUP_MAX) return false;
    uint32_t xm0 = 0;
    uint32_t order[MMA_GROUP_MAX];
    size_t bytes[MMA_GROUP_MAX];
    for (uint32_t i = 0; i < n; ++i) {
        const GemvCall &c = calls[i];
        if (!gemv_mma_group_eligible(c, ctx)) return false;
        const uint32_t hi = x_mode_of(c, false);
        if (i == 0) xm0 = hi;
        else if (hi != xm0) return false;
        bytes[i] = (size_t)c.rows * c.stride;
        order[i] = i;
    }
    for (uint32_t i = 1; i < n; ++i)                     // largest part first
        for (uint32_t j = i; j > 0 && bytes[order[j]] > bytes[order[j - 1]]; --j) { const uint32_t t = order[j]; order[j] = order[j - 1]; order[j - 1] = t; }
    // one tile per CTA while all of them are resident at once (two CTAs per SM); beyond that every
    // part gets its share of one wave, in whole tiles: a CTA's latency, not its arithmetic, sets
    // the time of these short launches, so a second wave would double it
    MmaGroupArgs ga = {};
    ga.n = n;
    uint32_t smem_bytes = 0, tiles_total = 0;
    MmaPlan plans[MMA_GROUP_MAX];
    const uint32_t slots = 2u * ctx.sm_count;
    for (uint32_t k = 0; k < n; ++k) {
        const GemvCall &c = calls[order[k]];
        if (!plan_mma(c.kind, c.cols, c.rows, c.stride, 1, slots, MMA_SMEM_BUDGET, xm0, plans[k])) return false;
        tiles_total += (c.rows + 16u * plans[k].row_tiles - 1) / (16u * plans[k].row_tiles);
    }
    for (uint32_t k = 0; k < n; ++k) {
        const GemvCall &c = calls[order[k]];
        MmaPlan &plan = plans[k];
        const uint32_t tiles = (c.rows + 16u * plan.row_tiles - 1) / (16u * plan.row_tiles);
        uint32_t ctas = tiles;
        if (tiles_total > slots) {
            ctas = (uint32_t)((uint64_t)slots * tiles / tiles_total);
            if (ctas < 1) ctas = 1;
        }
        plan.ctas = ctas;
        MmaArgs &a = ga.part[k];
        a.plan = plan;
        a.w[0] = c.w[0]; a.w[1] = nullptr;
        a.xp = c.norm_a ? nullptr : static_cast<const uint8_t *>(c.x);
        a.y = c.y;
        a.ids = nullptr; a.expert = c.expert; a.n_experts = c.n_experts; a.per_pair = 0; a.top = 1; a.glu = 0;
        a.status = ctx.status;
        a.na = c.norm_a; a.nb = c.norm_b; a.nw = c.norm_w; a.ns = c.norm_s; a.neps = c.norm_eps; a.nround_bf16 = c.norm_round_bf16;
        a.tp = c.tp;
        ga.first[k + 1] = ga.first[k] + ctas;
        if (plan.smem_bytes > smem_bytes) smem_bytes = plan.smem_bytes;
    }
    // the parts of a scope read the same inputs (q, k, v of a layer): one form of the exchange when every part has
    // the same input tagged, else the run-time form (a part without an output side just has n_out = 0)
    bool linked = false, any_a = false, any_b = false, all_a = true, all_b = true;
    for (uint32_t i = 0; i < ga.n; ++i) {
        const TpLink &t = ga.part[i].tp;
        linked = linked || t.n_out || t.in[0] || t.in[1];
        any_a = any_a || t.in[0]; all_a = all_a && t.in[0];
        any_b = any_b || t.in[1]; all_b = all_b && t.in[1];
    }
    const int link = !linked ? LINK_NONE : (any_a && any_b) ? LINK_ANY : any_a ? (all_a ? LINK_A : LINK_ANY)
                                         : any_b ? (all_b ? LINK_B : LINK_ANY) : LINK_OUT;
    if (link != LINK_NONE) {
        if (xm0 == XM_FX2 && link == LINK_OUT) err = launch_mma_group_t<XM_FX2, LINK_OUT>(ga, smem_bytes, ctx.stream, ctx.pdl);
        else if (xm0 == XM_FX2 && link == LINK_A) err = launch_mma_group_t<XM_FX2, LINK_A>(ga, smem_bytes, ctx.stream, ctx.pdl);
        else if (xm0 == XM_FX2 && link == LINK_B) err = launch_mma_group_t<XM_FX2, LINK_B>(ga, smem_bytes, ctx.stream, ctx.pdl);
        else if (xm0 == XM_FX2) err = launch_mma_group_t<XM_FX2, LINK_ANY>(ga, smem_bytes, ctx.stream, ctx.pdl);
        else if (xm0 == XM_FX4) err = launch_mma_group_t<XM_FX4, LINK_ANY>(ga, smem_bytes, ctx.stream, ctx.pdl);
        else err = cudaErrorInvalidValue;
        return true;
    }
    switch (xm0) {
    case XM_F16: err = launch_mma_group_t<XM_F16>(ga, smem_bytes, ctx.stream, ctx.pdl); break;
    case XM_F16_HI: err = launch_mma_group_t<XM_F16_HI>(ga, smem_bytes, ctx.stream, ctx.pdl); break;
    case XM_FX2: err = launch_mma_group_t<XM_FX2>(ga, smem_bytes, ctx.stream, ctx.pdl); break;
    default: err = launch_mma_group_t<XM_FX4>(ga, smem_bytes, ctx.stream, ctx.pdl); break;
    }
    return true;
}

// ---------------------------------------------------------------------------
// A sequence of one-token fused-norm projections run by ONE persistent kernel.
//
// A decode step is a chain of short, dependent projections; launched one by one, each pays a launch,
// a ramp of its copy ring and a tail, and HBM idles in between.  Here every SM keeps one resident CTA
// for the whole sequence (a cooperative launch: all CTAs are co-resident).  The producer warp of a
// CTA walks the list of projections and keeps streaming weight rows into the ring — weights depend
// on nothing, so it runs ahead into the next projection while the consumer warps still finish the
// current one or wait for its inputs.  The consumer warps take the projections in order: wait until
// every CTA has finished the projection this one depends on (a counter per projection in global
// memory, raised with a fence by each CTA and polled, with a time limit, by one thread), build the
// activation row (add + RMS norm + fixed point, read through L2), multiply their share of the rows,
// store.  Projections that read the same normalised input (k, v and q of a layer) build it once.
// ---------------------------------------------------------------------------

static constexpr uint32_t CHAIN_NO_WAIT = 0xffffffffu;

struct alignas(16) ChainOp {
    MmaArgs a;
    uint32_t wait_op;        // the projection whose completion (by every CTA) this one waits for, or CHAIN_NO_WAIT
    uint32_t reuse_x;        // the activation row of the previous projection is this one's as well
};
static_assert(sizeof(ChainOp) % 16 == 0, "copied as 16-byte words");

struct ChainArgs {
    const ChainOp *ops;
    uint32_t *done;          // [n_ops] CTAs that have finished each projection (zero at launch)
    uint32_t n_ops;
    int *status;
    unsigned long long *trace;     // debugging (INGOT_CHAIN_TRACE): [n_ops][4] times of CTA 0: start, inputs ready, row built, done
};

__device__ __forceinline__ bool chain_wait(const uint32_t *counter, uint32_t target) {
    uint64_t t0 = 0;
    for (;;) {
        for (int i = 0; i < 1024; ++i) {
            uint32_t v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
            if (v >= target) return true;
        }
        const uint64_t now = ptx::global_timer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > ptx::WAIT_LIMIT_NS) return false;
    }
}

// FAMILY 0: Q4_K and Q6_K weights; 1: Q4_0 and Q8_0.  OCC resident CTAs per SM of CW consumer warps each.
template <int FAMILY, int XM, int OCC, int CW>
__global__ void __launch_bounds__((CW + 1) * 32, OCC) gemv_chain_kernel(const __grid_constant__ ChainArgs c) {
    extern __shared__ __align__(128) uint8_t smem[];
    // projection descriptors, two per role (the next one is fetched while the current one runs):
    // [0], [1] the consumers', [2], [3] the producer's (it runs ahead of them)
    __shared__ __align__(16) ChainOp op_slot[4];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const bool producer = warp == (uint32_t)CW;
    constexpr uint32_t WORDS = sizeof(ChainOp) / 16u;
    static_assert(WORDS <= 32u, "one descriptor word per lane");
    // the copier of a role: the producer warp's lanes, or the consumers' first warp
    const bool copier = producer || warp == 0u;
    ChainOp *slots = &op_slot[producer ? 2 : 0];
    const uint4 *src = reinterpret_cast<const uint4 *>(c.ops);
    if (copier && lane < WORDS) {
        reinterpret_cast<uint4 *>(&slots[0])[lane] = __ldg(src + lane);
        if (c.n_ops > 1) reinterpret_cast<uint4 *>(&slots[1])[lane] = __ldg(src + WORDS + lane);
    }
    // A wait that runs out (the status word says which) must not leave the CTA's other warps at a barrier
    // for ever: the CTA is marked dead, skips the arithmetic of this and every later projection — all its
    // warps decide that together, right after a barrier — and still raises its counters, so that the other
    // CTAs run to their end as well.
    __shared__ uint32_t cta_dead, wait_ok;
    if (threadIdx.x == 0) cta_dead = 0u;
    MmaRun run;
    uint4 ahead = make_uint4(0u, 0u, 0u, 0u);
    for (uint32_t i = 0; i < c.n_ops; ++i) {
        if (producer) {
            __syncwarp();
        } else {
            // every consumer warp is through with the previous projection: its outputs are complete, the
            // activation row may be rebuilt, and this projection's descriptor is in place
            ptx::named_bar_sync(3, CW * 32);
            if (i > 0 && threadIdx.x == 0)             // (a release: the CTA's stores, ordered before it by the barrier, are visible to whoever sees the count)
                asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(c.done + (i - 1)), "r"(1u) : "memory");
            if (c.trace && blockIdx.x == 0 && threadIdx.x == 0) {
                const unsigned long long now = ptx::global_timer_ns();
                c.trace[8u * i] = now;
                if (i > 0) c.trace[8u * (i - 1u) + 3u] = now;
            }
        }
        if (copier && lane < WORDS) {
            // the slot of the projection just finished takes the next one (fetched while that one ran), and
            // the one after it starts its way from global memory now
            if (i >= 1 && i + 1 < c.n_ops) reinterpret_cast<uint4 *>(&slots[(i + 1) & 1u])[lane] = ahead;
            if (i + 2 < c.n_ops) ahead = __ldg(src + (size_t)(i + 2) * WORDS + lane);
        }
        const ChainOp *mine = &slots[i & 1u];
        if (!producer) {
            if (threadIdx.x == 0) {
                bool ok = true;
                const uint32_t dep = mine->wait_op;
                if (dep != CHAIN_NO_WAIT && !*(volatile uint32_t *)&cta_dead) {
                    ok = chain_wait(c.done + dep, gridDim.x);
                    if (!ok) set_status_word(c.status, KERNEL_ERR_CHAIN_TIMEOUT);
                }
                if (!ok) cta_dead = 1u;
                wait_ok = *(volatile uint32_t *)&cta_dead ? 0u : 1u;
            }
            ptx::named_bar_sync(4, CW * 32);
            if (!*(volatile uint32_t *)&wait_ok) continue;             // the whole CTA skips (barriers and counters go on)
            if (c.trace && blockIdx.x == 0 && threadIdx.x == 0) c.trace[8u * i + 1u] = ptx::global_timer_ns();
        }
        run.trace = (c.trace && blockIdx.x == 0) ? c.trace + 8u * i + 2u : nullptr;
        const MmaArgs &a = mine->a;
        run.build_x = mine->reuse_x == 0u;
        const uint32_t kind = a.plan.kind, nmat = a.plan.nmat;
        bool ok;
        if (FAMILY == 0) {
            if (kind == KIND_Q4_K)
                ok = nmat == 2 ? gemv_mma_body<KIND_Q4_K, 2, XM, CW>(a, smem, blockIdx.x, gridDim.x, 0u, false, run)
                               : gemv_mma_body<KIND_Q4_K, 1, XM, CW>(a, smem, blockIdx.x, gridDim.x, 0u, false, run);
            else
                ok = gemv_mma_body<KIND_Q6_K, 1, XM, CW>(a, smem, blockIdx.x, gridDim.x, 0u, false, run);
        } else {
            if (kind == KIND_Q4_0)
                ok = nmat == 2 ? gemv_mma_body<KIND_Q4_0, 2, XM, CW>(a, smem, blockIdx.x, gridDim.x, 0u, false, run)
                               : gemv_mma_body<KIND_Q4_0, 1, XM, CW>(a, smem, blockIdx.x, gridDim.x, 0u, false, run);
            else
                ok = gemv_mma_body<KIND_Q8_0, 1, XM, CW>(a, smem, blockIdx.x, gridDim.x, 0u, false, run);
        }
        if (!ok) {
            if (producer) return;                  // the producer meets nobody at a barrier; the consumers' waits for its stages run out
            if (lane == 0) *(volatile uint32_t *)&cta_dead = 1u;
        }
    }
}

static bool ranges_overlap(const void *p, size_t np, const void *q, size_t nq) {
    if (!p || !q) return false;
    const uintptr_t a = (uintptr_t)p, b = (uintptr_t)q;
    return a < b + nq && b < a + np;
}

bool chain_call_eligible(const GemvCall &c) {
    if (c.ids || !c.norm_a || !mma_kind(c.kind) || c.cols % 64u || (c.nmat != 1 && c.nmat != 2)) return false;
    if (c.nmat == 2 && (c.kind == KIND_Q6_K || c.kind == KIND_Q8_0)) return false;
    if (((uintptr_t)c.w[0] % 16u) || (c.nmat == 2 && ((uintptr_t)c.w[1] % 16u)) || ((size_t)c.rows * c.stride) % 16u) return false;
    return true;
}

cudaError_t chain_build(const GemvCall *calls, uint32_t n, const LaunchCtx &ctx, ChainLaunch &out, const char *&why) {
    out = ChainLaunch();
    why = "";
    if (n == 0) { why = "no projections were recorded"; return cudaErrorInvalidValue; }
    std::vector<GemvCall> cs(calls, calls + n);
    const bool family1 = cs[0].kind == KIND_Q4_0 || cs[0].kind == KIND_Q8_0;
    const uint32_t xm = x_mode_of(cs[0], false);
    for (const GemvCall &c : cs) {
        if (!chain_call_eligible(c)) { why = "a recorded projection has no fused tensor-core form (type, alignment or shape)"; return cudaErrorNotSupported; }
        if ((c.kind == KIND_Q4_0 || c.kind == KIND_Q8_0) != family1) { why = "K-quant and legacy weight types cannot share one chain"; return cudaErrorNotSupported; }
        if (x_mode_of(c, false) != xm) { why = "all projections of a chain round their activations the same way"; return cudaErrorNotSupported; }
    }
    // projections that read the same normalised input build it once: the first of the group takes the
    // group's residual-sum store
    std::vector<uint32_t> reuse(n, 0u);
    auto same_input = [](const GemvCall &p, const GemvCall &q) {
        return p.norm_a == q.norm_a && p.norm_b == q.norm_b && p.norm_w == q.norm_w && p.cols == q.cols && p.norm_eps == q.norm_eps;
    };
    for (uint32_t j = 1; j < n; ++j) {
        uint32_t first = j - 1;
        while (reuse[first]) --first;
        GemvCall &f = cs[first], &c = cs[j];
        if (!same_input(f, c)) continue;
        if (c.norm_s && f.norm_s && c.norm_s != f.norm_s) continue;
        // nothing the group writes may touch what a slower CTA is still reading to build the row
        bool clash = false;
        for (uint32_t k = first; k <= j && !clash; ++k) {
            const GemvCall &m = cs[k];
            const void *outs[2] = {m.y, m.norm_s ? (const void *)m.norm_s : (const void *)c.norm_s};
            const size_t lens[2] = {(size_t)m.rows * 4u, (size_t)m.cols * 4u};
            for (int o = 0; o < 2; ++o)
                clash = clash || ranges_overlap(outs[o], lens[o], c.norm_a, (size_t)c.cols * 4u) || ranges_overlap(outs[o], lens[o], c.norm_b, (size_t)c.cols * 4u);
        }
        // ... and what this projection writes must not be written by another member (members run unordered across CTAs)
        for (uint32_t k = first; k < j && !clash; ++k) {
            const GemvCall &m = cs[k];
            clash = ranges_overlap(c.y, (size_t)c.rows * 4u, m.y, (size_t)m.rows * 4u) ||
                    ranges_overlap(c.y, (size_t)c.rows * 4u, m.norm_s, (size_t)m.cols * 4u) ||
                    ranges_overlap(c.norm_s, (size_t)c.cols * 4u, m.y, (size_t)m.rows * 4u);
        }
        if (clash) continue;
        if (c.norm_s) { f.norm_s = c.norm_s; c.norm_s = nullptr; }
        reuse[j] = 1u;
    }
    // the projection each one waits for: the latest earlier one that wrote what it reads, or that read
    // or wrote what it writes.  CTAs take the projections in order, so "all CTAs finished i" covers all before i.
    std::vector<uint32_t> wait(n, CHAIN_NO_WAIT);
    for (uint32_t j = 0; j < n; ++j) {
        const GemvCall &c = cs[j];
        const void *rd[2] = {c.norm_a, c.norm_b};
        const void *wr[2] = {c.y, c.norm_s};
        const size_t wl[2] = {(size_t)c.rows * 4u, (size_t)c.cols * 4u};
        for (uint32_t i = 0; i < j; ++i) {
            const GemvCall &e = cs[i];
            const void *er[2] = {e.norm_a, e.norm_b};
            const void *ew[2] = {e.y, e.norm_s};
            const size_t el[2] = {(size_t)e.rows * 4u, (size_t)e.cols * 4u};
            bool dep = false;
            for (int x = 0; x < 2; ++x)
                for (int y = 0; y < 2; ++y) {
                    dep = dep || ranges_overlap(rd[x], (size_t)c.cols * 4u, ew[y], el[y]);      // read after write
                    dep = dep || ranges_overlap(wr[x], wl[x], er[y], (size_t)e.cols * 4u);      // write after read
                    dep = dep || ranges_overlap(wr[x], wl[x], ew[y], el[y]);                    // write after write
                }
            if (dep) wait[j] = i;
        }
    }
    for (uint32_t j = 0; j < n; ++j) {          // a group waits, at its first projection, for everything any member needs
        if (!reuse[j]) continue;
        uint32_t first = j;
        while (reuse[first]) --first;
        if (wait[j] != CHAIN_NO_WAIT && wait[j] >= first) { why = "internal: a projection depends on a member of its own group"; return cudaErrorNotSupported; }
        if (wait[j] != CHAIN_NO_WAIT && (wait[first] == CHAIN_NO_WAIT || wait[j] > wait[first])) wait[first] = wait[j];
        wait[j] = CHAIN_NO_WAIT;
    }
    // common shared-memory geometry: the widest activation row, a ring of equal slots that holds every
    // projection's smallest stage, one CTA per SM
    MmaFixed fx = {0u, 0u, 0u, (uint32_t)MMA_WARPS};
    for (const GemvCall &c : cs) {
        const uint32_t xb = x_row_bytes(xm, c.cols);
        if (xb > fx.x_bytes) fx.x_bytes = xb;
    }
    const char *occ_env = getenv("INGOT_CHAIN_OCC");                // experiments: resident CTAs per SM (1 or 2)
    const uint32_t occ = occ_env && atoi(occ_env) == 2 ? 2u : 1u;
    const char *cw_env = getenv("INGOT_CHAIN_WARPS");               // experiments: consumer warps per CTA (8 or 16)
    const uint32_t cw = occ == 2 ? 8u : (cw_env && atoi(cw_env) == 8 ? 8u : 16u);
    fx.warps = cw;
    const uint32_t budget = occ == 2 ? 113u * 1024u : MMA_SMEM_MAX;
    const uint32_t red_slots = budget <= MMA_SMEM_SMALL ? 4u : MMA_RED_SLOTS;      // as plan_mma sizes it
    const uint32_t red_bytes = red_slots * MMA_WARPS * 2u * 16u * 4u + MMA_ZERO_BYTES;
    const uint32_t fixed_bytes = MMA_BAR_BYTES + ((fx.x_bytes + 127u) & ~127u) + red_bytes;
    if (fixed_bytes + 2u * 16384u > budget) { why = "activation rows too wide for the chain kernel"; return cudaErrorNotSupported; }
    for (const GemvCall &c : cs) {              // smallest stage of each projection: one step per warp
        uint32_t step_cols, step_bytes;
        step_geometry(c.kind, step_cols, step_bytes);
        if (c.cols % step_cols) { why = "a recorded projection does not plan"; return cudaErrorNotSupported; }
        const uint32_t nsteps = c.cols / step_cols;
        uint32_t kw = 3;
        while (kw > 0 && (nsteps % (1u << kw))) --kw;
        const uint32_t per_warp = nsteps >> kw, row_tiles = (uint32_t)MMA_WARPS >> kw;
        const uint32_t lead = (c.kind == KIND_Q4_K || c.kind == KIND_Q6_K) ? 32u : 16u;
        uint32_t sb = 0;
        for (uint32_t spw = 1; spw <= per_warp; ++spw) {
            const uint32_t cb = spw * (1u << kw) * step_bytes;
            if (per_warp % spw || cb % 16u) continue;
            sb = (pitch_of(cb, lead) * 16u * row_tiles + 64u + 127u) & ~127u;
            break;
        }
        if (sb == 0) { why = "a recorded projection does not plan"; return cudaErrorNotSupported; }
        if (sb > fx.slot_bytes) fx.slot_bytes = sb;
    }
    const char *slot_env = getenv("INGOT_CHAIN_SLOT_BYTES");        // experiments: a larger slot lets narrow rows take more steps per stage
    if (slot_env && (uint32_t)atoi(slot_env) > fx.slot_bytes) fx.slot_bytes = ((uint32_t)atoi(slot_env) + 127u) & ~127u;
    fx.slots = (budget - fixed_bytes) / fx.slot_bytes;
    if (fx.slots > (uint32_t)MMA_MAX_STAGES) fx.slots = MMA_MAX_STAGES;
    const uint32_t groups = cw / (uint32_t)MMA_WARPS;                // every consumer group has a ring of its own
    fx.slots -= fx.slots % groups;
    if (fx.slots < 2 * groups) { why = "the chain's stages do not fit in shared memory"; return cudaErrorNotSupported; }
    const uint32_t ctas = ctx.sm_count * occ;
    std::vector<ChainOp> ops(n);
    std::vector<CUtensorMap> maps(2u * n);
    cudaError_t e = cudaMalloc(&out.maps_dev, sizeof(CUtensorMap) * 2u * n);
    if (e != cudaSuccess) return e;
    const bool use_tma = !(getenv("INGOT_CHAIN_TMA") && atoi(getenv("INGOT_CHAIN_TMA")) == 0);      // experiments: 0 = one bulk copy per row
    uint32_t smem_bytes = 0;
    for (uint32_t j = 0; j < n; ++j) {
        const GemvCall &c = cs[j];
        ChainOp &o = ops[j];
        memset(&o, 0, sizeof(o));
        if (!plan_mma(c.kind, c.cols, c.rows, c.stride, c.nmat, ctas, budget, xm, o.a.plan, &fx)) {
            why = "a recorded projection does not plan";
            chain_free(out);
            return cudaErrorNotSupported;
        }
        o.a.plan.ctas = ctas;
        if (o.a.plan.smem_bytes > smem_bytes) smem_bytes = o.a.plan.smem_bytes;
        o.a.w[0] = c.w[0]; o.a.w[1] = c.nmat == 2 ? c.w[1] : nullptr;
        o.a.y = c.y; o.a.expert = c.expert; o.a.n_experts = 0; o.a.top = 1; o.a.glu = c.glu;
        o.a.status = ctx.status;
        o.a.na = c.norm_a; o.a.nb = c.norm_b; o.a.nw = c.norm_w; o.a.ns = c.norm_s; o.a.neps = c.norm_eps; o.a.nround_bf16 = c.norm_round_bf16;
        o.wait_op = wait[j];
        o.reuse_x = reuse[j];
        // the stage as one box: rows of 8-byte elements, row_pitch / 8 of them (at most 256) by 16 row_tiles rows
        const MmaPlan &pl = o.a.plan;
        for (uint32_t m = 0; m < c.nmat && use_tma; ++m) {
            const uint8_t *base = c.w[m] + (size_t)c.expert * c.rows * c.stride;
            if (pl.row_pitch % 16u || pl.row_pitch / 8u > 256u || c.stride % 16u || ((uintptr_t)base % 16u)) break;
            if (!make_tensor_map_2d(maps[2u * j + m], CU_TENSOR_MAP_DATA_TYPE_UINT64, base, c.stride / 8u, c.rows, c.stride,
                                    pl.row_pitch / 8u, 16u * pl.row_tiles, CU_TENSOR_MAP_SWIZZLE_NONE))
                break;
            o.a.tmap[m] = static_cast<const CUtensorMap *>(out.maps_dev) + (2u * j + m);
        }
        if (c.nmat == 2 && !o.a.tmap[1]) o.a.tmap[0] = nullptr;       // both matrices or neither
        if (o.a.tmap[0]) o.a.expert = 0;                               // the maps start at the expert's first row
    }
    e = cudaMemcpy(out.maps_dev, maps.data(), sizeof(CUtensorMap) * 2u * n, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMalloc(&out.ops_dev, sizeof(ChainOp) * n);
    if (e == cudaSuccess) e = cudaMalloc(&out.done_dev, sizeof(uint32_t) * n);
    if (e == cudaSuccess) e = cudaMemcpy(out.ops_dev, ops.data(), sizeof(ChainOp) * n, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { chain_free(out); return e; }
    out.n_ops = n; out.ctas = ctas; out.smem_bytes = smem_bytes; out.xm = xm; out.family = family1 ? 1u : 0u;
    out.slots = fx.slots; out.slot_bytes = fx.slot_bytes; out.occ = occ; out.warps = cw;
    if (getenv("INGOT_CHAIN_TRACE") && atoi(getenv("INGOT_CHAIN_TRACE")) != 0 &&
        cudaMalloc(&out.trace_dev, 64u * n) == cudaSuccess)
        cudaMemset(out.trace_dev, 0, 64u * n);
    uint32_t waits = 0;
    for (uint32_t j = 0; j < n; ++j) waits += wait[j] != CHAIN_NO_WAIT;
    out.waits = waits;
    return cudaSuccess;
}

void chain_free(ChainLaunch &c) {
    if (c.ops_dev) cudaFree(c.ops_dev);
    if (c.done_dev) cudaFree(c.done_dev);
    if (c.maps_dev) cudaFree(c.maps_dev);
    if (c.trace_dev) {
        // debugging: the last launch's times of CTA 0, one line per projection
        std::vector<unsigned long long> t(8u * c.n_ops);
        if (cudaDeviceSynchronize() == cudaSuccess && cudaMemcpy(t.data(), c.trace_dev, t.size() * 8u, cudaMemcpyDeviceToHost) == cudaSuccess) {
            fprintf(stderr, "chain trace (CTA 0, microseconds): projection  start  wait  build (loads, reduce, pack)  rows  total\n");
            for (uint32_t i = 0; i + 1 < c.n_ops; ++i) {
                const unsigned long long *q = &t[8u * i];
                const double t0 = (double)q[0], t1 = (double)q[1], t2 = (double)q[2], t3 = (double)q[3];
                const bool built = q[2] >= q[1] && q[2] <= q[3];
                fprintf(stderr, "%4u %10.2f %7.2f %7.2f (%5.2f %5.2f %5.2f) %7.2f %7.2f\n", i, (t0 - (double)t[0]) * 1e-3, (t1 - t0) * 1e-3,
                        built ? (t2 - t1) * 1e-3 : 0.0, built ? ((double)q[4] - t1) * 1e-3 : 0.0, built ? ((double)q[5] - (double)q[4]) * 1e-3 : 0.0,
                        built ? (t2 - (double)q[5]) * 1e-3 : 0.0, (t3 - (built ? t2 : t1)) * 1e-3, (t3 - t0) * 1e-3);
            }
        }
        cudaFree(c.trace_dev);
    }
    c = ChainLaunch();
}

template <int FAMILY, int XM, int OCC, int CW>
static cudaError_t chain_launch_t(const ChainLaunch &c, const ChainArgs &args, cudaStream_t stream) {
    auto kernel = gemv_chain_kernel<FAMILY, XM, OCC, CW>;
    static DeviceOnce once;
    const cudaError_t e = once.smem(kernel, (int)MMA_SMEM_MAX);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(c.ctas);
    cfg.blockDim = dim3((CW + 1) * 32);
    cfg.dynamicSmemBytes = c.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;          // every CTA resident at once: they wait for one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args);
}

cudaError_t chain_launch(const ChainLaunch &c, const LaunchCtx &ctx) {
    cudaError_t e = cudaMemsetAsync(c.done_dev, 0, sizeof(uint32_t) * c.n_ops, ctx.stream);
    if (e != cudaSuccess) return e;
    ChainArgs args = {static_cast<const ChainOp *>(c.ops_dev), c.done_dev, c.n_ops, ctx.status, static_cast<unsigned long long *>(c.trace_dev)};
    const bool fx2 = c.xm == XM_FX2;
    if (c.occ == 2) {
        if (c.family == 0) return fx2 ? chain_launch_t<0, XM_FX2, 2, 8>(c, args, ctx.stream) : chain_launch_t<0, XM_FX4, 2, 8>(c, args, ctx.stream);
        return fx2 ? chain_launch_t<1, XM_FX2, 2, 8>(c, args, ctx.stream) : chain_launch_t<1, XM_FX4, 2, 8>(c, args, ctx.stream);
    }
    if (c.warps == 8) {
        if (c.family == 0) return fx2 ? chain_launch_t<0, XM_FX2, 1, 8>(c, args, ctx.stream) : chain_launch_t<0, XM_FX4, 1, 8>(c, args, ctx.stream);
        return fx2 ? chain_launch_t<1, XM_FX2, 1, 8>(c, args, ctx.stream) : chain_launch_t<1, XM_FX4, 1, 8>(c, args, ctx.stream);
    }
    if (c.family == 0) return fx2 ? chain_launch_t<0, XM_FX2, 1, 16>(c, args, ctx.stream) : chain_launch_t<0, XM_FX4, 1, 16>(c, args, ctx.stream);
    return fx2 ? chain_launch_t<1, XM_FX2, 1, 16>(c, args, ctx.stream) : chain_launch_t<1, XM_FX4, 1, 16>(c, args, ctx.stream);
}

}  // namespace ingot
