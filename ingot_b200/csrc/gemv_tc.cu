// One-token GEMV over Q4_K rows on the 5th-generation tensor cores (tcgen05, int8).  Opt-in
// (INGOT_OPT_TCGEN05_GEMV, or activations passed as digit rows): at the benchmark shapes it is
// not yet faster than the mma.sync kernel of gemv_mma.cu, see "Status" below.
//
// Idea: with mma.sync every weight costs a register-level extraction AND the lane-level
// bookkeeping of a 16-row fragment (about 330 issued instructions per 4096 weights), and the
// SM's issue slots run out near half of HBM bandwidth.  Here a THREAD owns a ROW:
//   * a 2-D TMA copy brings 128 rows x one 256-column block (a "unit") into shared memory;
//   * unpack warps (thread = row, each of two warp sets takes one 128-column half) turn the
//     row's quants into unsigned bytes with one logic op per four weights and store them
//     straight into tensor memory (tcgen05.st) as the A operand of eight int8 MMAs (M 128,
//     N 8, K 32 each: one per 32-column sub-block);
//   * the B operand is the activation row as three signed base-256 digits of round(x * S)
//     (a 22-bit fixed-point value, S a power of two), resident in shared memory for the
//     whole kernel; the MMA gives, per row and sub-block, the exact integer dot product
//     with each digit (D in tensor memory, int32);
//   * epilogue warps (thread = row and half) read D (tcgen05.ld), recombine the digits in
//     int32, apply the row's sub-block scales in fp32 in the reference's factored form
//     (kernels/iq3_mix.metal:104-123) and keep the row's sum in a register; the min term
//     (dmin * min * sum of x) is added by the unpack thread, which needs no MMA result.
//     No cross-lane or cross-warp reduction exists; a flush warp adds the two halves.
// The integer part is exact; rounding happens only in the fp32 scale-and-add.
//
// Work split ("stream-K"): the units of all 128-row tiles are numbered (tile, matrix, block)
// and cut into equal contiguous ranges, one per CTA (one CTA per SM), so every SM streams
// the same number of bytes whatever the row count.  A tile finished by one CTA is written
// directly; a tile shared by several CTAs goes through per-CTA partial rows in a scratch
// buffer, and the LAST CTA to arrive (one atomic counter per tile, no waiting) adds the
// partials in CTA order — the result does not depend on arrival order.
//
// Status (measured on B200, fused gate/up 4096 -> 2 x 12288): 22.7 us per launch against
// 19.1 us for the mma.sync kernel; about 1400 cycles per unit where HBM would allow 800.
// What the measurements showed: issuing one tcgen05.mma costs the issuing thread about 100
// cycles whatever its shape or operand source (so four threads issue two MMAs each); the
// tensor-memory rings hold only four units (A 64 + D 64 columns each of 512), and with
// every unit crossing four hand-offs (copy -> unpack -> MMA -> epilogue) the pipeline is
// latency-bound rather than issue- or bandwidth-bound.
//
// Every wait is bounded; a timeout sets the status word and the CTA drains and exits.
#include <cuda.h>
#include <cuda_fp16.h>

#include "dev_common.cuh"
#include "gemv_core.cuh"
#include "kernels.h"
#include "pack.cuh"
#include "ptx.cuh"
#include "tensor_map.h"

namespace ingot {


static constexpr uint32_t TC_THREADS = 704;        // 8 unpack, 8 epilogue, 1 copy, 4 MMA, 1 flush warp
static constexpr uint32_t TC_TILE = 128;           // rows per tile = TMEM lanes
static constexpr uint32_t TC_MAX_STAGES = 8;
static constexpr uint32_t TC_SLOTS = 4;            // A and D rings in tensor memory
static constexpr uint32_t TC_TMEM_COLS = 512;      // A: 4 x 64 columns, D: 4 x 64 columns
static constexpr uint32_t TC_BAR_BYTES = 512;
static constexpr uint32_t TC_HAND_BYTES = 2u * TC_TILE * 20u;   // per slot and half: a row's block header (16 bytes) and its min term (fp32)
static constexpr uint32_t TC_DEPOSIT_BYTES = 2u * 2u * 2u * TC_TILE * 4u;      // [2 buffers][2 groups][2 matrices][128 rows] fp32
static constexpr uint32_t TC_SMEM_MAX = 226u * 1024u;

struct TcPlan {
    uint32_t kind, cols, rows, stride, nmat;
    uint32_t kb;            // 256-column blocks per row
    uint32_t ut;            // units per tile = nmat * kb
    uint32_t tiles, units;
    uint32_t ctas;
    uint32_t box_bytes;     // bytes per row of one unit in shared memory
    uint32_t stages, stage_bytes;
    uint32_t x_bytes;       // digit image + sums + scale
    uint32_t smem_bytes;
    uint32_t maxc;          // most CTAs that can share one tile
};

struct TcArgs {
    TcPlan p;
    const uint8_t *xq;      // packed digits of the activation row (launch_pack_digits)
    float *y;
    float *partials;        // [tiles][maxc][nmat][128]
    uint32_t *counters;     // [tiles], zero between launches
    uint32_t glu;
    int *status;
};

// ---- host: geometry --------------------------------------------------------------------

static bool plan_tc(uint32_t kind, uint32_t cols, uint32_t rows, uint32_t stride, uint32_t nmat, uint32_t sm_count, TcPlan &p) {
    if (kind != KIND_Q4_K) return false;
    if (cols == 0 || rows == 0 || cols % 256u || stride % 16u || stride != cols / 256u * 144u) return false;
    p.kind = kind; p.cols = cols; p.rows = rows; p.stride = stride; p.nmat = nmat;
    p.kb = cols / 256u;
    p.ut = nmat * p.kb;
    p.tiles = (rows + TC_TILE - 1) / TC_TILE;
    const uint64_t units = (uint64_t)p.tiles * p.ut;
    if (units > 0x7fffffffull) return false;
    p.units = (uint32_t)units;
    p.ctas = p.units < sm_count ? p.units : sm_count;
    p.box_bytes = 144u;
    p.stage_bytes = p.box_bytes * TC_TILE;
    p.x_bytes = packed_digits_bytes(cols);
    const uint32_t fixed = TC_BAR_BYTES + TC_SLOTS * TC_HAND_BYTES + TC_DEPOSIT_BYTES + ((p.x_bytes + 127u) & ~127u);
    if (fixed + 2u * p.stage_bytes > TC_SMEM_MAX) return false;
    p.stages = (TC_SMEM_MAX - fixed) / p.stage_bytes;
    if (p.stages > TC_MAX_STAGES) p.stages = TC_MAX_STAGES;
    p.smem_bytes = fixed + p.stages * p.stage_bytes;
    const uint32_t per_cta = p.units / p.ctas;            // floor: the shortest range
    p.maxc = (p.ut + per_cta - 1) / per_cta + 1;
    return true;
}

// first unit of CTA c
__host__ __device__ __forceinline__ uint32_t tc_range_begin(uint32_t c, uint32_t units, uint32_t ctas) {
    return (uint32_t)(((uint64_t)c * units) / ctas);
}
// the CTA whose range holds unit u
__device__ __forceinline__ uint32_t tc_cta_of(uint32_t u, uint32_t units, uint32_t ctas) {
    uint32_t c = (uint32_t)(((uint64_t)u * ctas) / units);
    while (c + 1 < ctas && tc_range_begin(c + 1, units, ctas) <= u) ++c;
    while (c > 0 && tc_range_begin(c, units, ctas) > u) --c;
    return c;
}

// ---- packing the activation row into digits ----------------------------------------------
// Row image for `cols` activations (a multiple of 256):
//   [cols/16 chunks][8 rows][16 bytes]: rows 0..2 = digits d0, d1, d2 of q = round(x * S)
//     (q = d0 + 256 d1 + 65536 d2, each digit in [-128, 127]) for the chunk's 16 columns;
//     rows 3..5 = the same digits in odd chunks and zero in even ones (the sum over the second
//     half of every 32 columns, for formats with 16-column groups); rows 6, 7 zero.
//     This is the K-major, unswizzled shared-memory layout of an N = 8 B operand.
//   [cols/16] fp32: sum of q over the chunk
//   16 bytes: 1/S.  S is the power of two that puts max|x| * S in [2^21, 2^22).

struct DigitArgs {
    const void *x;
    uint8_t *out;
    uint32_t cols, bf16;
};

__global__ void __launch_bounds__(256) pack_digits_kernel(const __grid_constant__ DigitArgs a) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    __shared__ float part_max[8];
    const uint32_t tid = threadIdx.x;
    const size_t base = (size_t)blockIdx.x * a.cols;
    uint8_t *row = a.out + (size_t)blockIdx.x * packed_digits_bytes(a.cols);
    float mx = 0.f;
    for (uint32_t c = tid; c < a.cols; c += 256) mx = fmaxf(mx, fabsf(load_x(a.x, base + c, a.bf16)));
    for (uint32_t off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if ((tid & 31u) == 0) part_max[tid >> 5] = mx;
    __syncthreads();
    mx = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) mx = fmaxf(mx, part_max[i]);
    const float scale = digits_scale(mx);
    const uint32_t n4 = a.cols / 4u;
    for (uint32_t q0 = 0; q0 < n4; q0 += 256) {        // every thread runs the same rounds: the sum uses quad shuffles
        const uint32_t q = q0 + tid;
        const bool live = q < n4;
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = live ? load_x(a.x, base + 4u * q + i, a.bf16) * scale : 0.f;
        digits_store_quad(row, a.cols, q, v, live);
    }
    if (tid == 0) digits_store_unscale(row, a.cols, scale);
}

cudaError_t launch_pack_digits(const void *x, uint32_t bf16, uint32_t rows, uint32_t cols, void *packed, const LaunchCtx &ctx) {
    if (rows == 0) return cudaSuccess;
    if (cols % 256u) return cudaErrorInvalidValue;
    DigitArgs a = {x, static_cast<uint8_t *>(packed), cols, bf16};
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, pack_digits_kernel, a);
}

// ---- tcgen05 wrappers --------------------------------------------------------------------

__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit_to(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ptx::smem_addr(bar)) : "memory");
}
// D[tmem] = A[tmem] * B[smem]^T: A 128 x 32 unsigned bytes (lane = row, 8 columns), B 8 x 32 signed bytes, D int32
__device__ __forceinline__ void tc_mma_i8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc)
        : "memory");
}
// K-major operand without swizzle: 8 rows x 16 bytes per 128-byte core matrix, the two 16-byte
// K halves of one MMA `lbo` bytes apart
__device__ __forceinline__ uint64_t tc_desc_kmajor_plain(uint32_t smem_byte_addr, uint32_t lbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_byte_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(128u >> 4) << 32;          // next 8-row group (unused for N = 8)
    d |= (uint64_t)1 << 46;                    // descriptor version of sm_100
    return d;
}
// kind::i8: D int32, A unsigned 8-bit, B signed 8-bit, both K-major, M 128, N 8
__device__ __forceinline__ uint32_t tc_idesc_u8s8(uint32_t m, uint32_t n) {
    return (2u << 4) | (0u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
          "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, int32_t (&v)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
                 : "r"(taddr)
                 : "memory");
}

__device__ __forceinline__ void tma_load_2d(void *dst_smem, const CUtensorMap *map, uint32_t x, uint32_t y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(ptx::smem_addr(dst_smem)), "l"(map), "r"(x), "r"(y), "r"(ptx::smem_addr(bar))
        : "memory");
}

// ---- kernel ------------------------------------------------------------------------------

// Position of a unit: (tile, matrix, block), advanced without divisions.
struct TcUnit {
    uint32_t tile, m, b;
    __device__ __forceinline__ void init(uint32_t u, uint32_t ut, uint32_t kb) {
        tile = u / ut;
        const uint32_t rem = u - tile * ut;
        m = rem / kb;
        b = rem - m * kb;
    }
    __device__ __forceinline__ void next(uint32_t kb, uint32_t nmat) {
        if (++b == kb) { b = 0; if (++m == nmat) { m = 0; ++tile; } }
    }
};
// Ring position (index, phase parity) advanced without divisions.
struct TcRing {
    uint32_t idx, phase;
    __device__ __forceinline__ TcRing(uint32_t first, uint32_t n) : idx(first % n), phase((first / n) & 1u) {}
    __device__ __forceinline__ void advance(uint32_t by, uint32_t n) {
        idx += by;
        while (idx >= n) { idx -= n; phase ^= 1u; }
    }
};

// Warp roles.  Every unit is split in two halves of 128 columns (four MMAs): each half has its own four
// unpack warps, four epilogue warps and MMA thread, which halves the time a unit spends in every phase
// of the pipeline (the tensor-memory rings hold four units).
static constexpr uint32_t TC_W_EPI = 8, TC_W_COPY = 16, TC_W_MMA = 17, TC_W_FLUSH = 21;

template <int NMAT>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemv_tc_q4k_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1, const __grid_constant__ TcArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const TcPlan &p = a.p;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);            // [stages] copy -> unpack
    uint64_t *empty = full + TC_MAX_STAGES;                           // [stages] unpack -> copy
    uint64_t *afull = empty + TC_MAX_STAGES;                          // [slots][2 halves] unpack -> MMA
    uint64_t *mdone = afull + 2 * TC_SLOTS;                               // [slots] MMA -> unpack (A slot free) and epilogue (D ready)
    uint64_t *dempty = mdone + TC_SLOTS;                              // [slots] epilogue -> MMA, unpack (hand-off area free)
    uint64_t *fl_full = dempty + TC_SLOTS;                            // [2] epilogue -> flush warp: a tile's sums are deposited
    uint64_t *fl_empty = fl_full + 2;                                 // [2] flush warp -> epilogue
    uint64_t *xbar = fl_empty + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(xbar + 1);
    uint8_t *hand = smem + TC_BAR_BYTES;                              // [slots]: uint4 header[128], float minterm[128]
    float *deposit = reinterpret_cast<float *>(hand + TC_SLOTS * TC_HAND_BYTES);     // [2 buffers][2 groups][NMAT][128]
    uint8_t *ximg = reinterpret_cast<uint8_t *>(deposit) + TC_DEPOSIT_BYTES;
    const float *sums = reinterpret_cast<const float *>(ximg + (size_t)p.cols * 8u);
    uint8_t *stages = ximg + ((p.x_bytes + 127u) & ~127u);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], 8);
        }
        for (uint32_t s = 0; s < TC_SLOTS; ++s) {
            ptx::mbar_init(&afull[2 * s], 4);
            ptx::mbar_init(&afull[2 * s + 1], 4);
            ptx::mbar_init(&mdone[s], 4);
            ptx::mbar_init(&dempty[s], 8);
        }
        for (uint32_t s = 0; s < 2; ++s) {
            ptx::mbar_init(&fl_full[s], 8);
            ptx::mbar_init(&fl_empty[s], 1);
        }
        ptx::mbar_init(xbar, 1);
        ptx::mbar_init_fence();
    }
    if (warp == TC_W_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_addr(tmem_slot)), "r"(TC_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t a_base = tmem_base, d_base = tmem_base + TC_SLOTS * 64u;
    ptx::pdl_launch_dependents();

    const uint32_t u0 = tc_range_begin(blockIdx.x, p.units, gridDim.x), u1 = tc_range_begin(blockIdx.x + 1, p.units, gridDim.x);
    const uint32_t n_units = u1 - u0;
    bool failed = false;

    if (warp == TC_W_COPY) {
        // ---- copy thread: the weights do not depend on the previous kernel ----
        if (lane == 0) {
            TcUnit un;
            un.init(u0, p.ut, p.kb);
            TcRing st(0, p.stages);
            for (uint32_t i = 0; i < n_units; ++i) {
                if (!ptx::mbar_wait_sleep<0>(&empty[st.idx], st.phase ^ 1u)) { failed = true; break; }
                ptx::mbar_expect_tx(&full[st.idx], p.stage_bytes);
                tma_load_2d(stages + (size_t)st.idx * p.stage_bytes, un.m ? &map1 : &map0, un.b * 144u, un.tile * TC_TILE, &full[st.idx]);
                un.next(p.kb, NMAT);
                st.advance(1, p.stages);
            }
            if (failed) set_status_word(a.status, KERNEL_ERR_PRODUCER_TIMEOUT);
        }
    } else if (warp >= TC_W_MMA && warp < TC_W_MMA + 4) {
        // ---- MMA threads.  Issuing one tcgen05.mma costs the issuing thread about 100 cycles whatever
        // its shape (measured), far more than these small MMAs take to run, so four threads in four
        // warps (four schedulers) each issue two of a unit's eight.  The first also brings the
        // activation image, which does depend on the previous kernel. ----
        if (lane == 0) {
            const uint32_t mt = warp - TC_W_MMA, grp = mt >> 1;
            if (mt == 0) {
                ptx::pdl_wait();
                ptx::mbar_expect_tx(xbar, p.x_bytes);
                for (uint32_t off = 0; off < p.x_bytes; off += 32768u)
                    ptx::bulk_g2s(ximg + off, a.xq + off, (p.x_bytes - off) < 32768u ? (p.x_bytes - off) : 32768u, xbar);
            }
            const uint32_t idesc = tc_idesc_u8s8(TC_TILE, 8);
            const uint32_t x_addr = ptx::smem_addr(ximg);
            if (!ptx::mbar_wait(xbar, 0)) failed = true;
            TcUnit un;
            un.init(u0, p.ut, p.kb);
            TcRing sl(0, TC_SLOTS);
            for (uint32_t i = 0; i < n_units && !failed; ++i) {
                if (!ptx::mbar_wait_sleep<0>(&afull[2u * sl.idx + grp], sl.phase)) { failed = true; break; }
                if (!ptx::mbar_wait_sleep<0>(&dempty[sl.idx], sl.phase ^ 1u)) { failed = true; break; }
                tc_fence_after_sync();
                const uint32_t bx = x_addr + un.b * (16u * 128u);
#pragma unroll
                for (uint32_t m = 2u * mt; m < 2u * mt + 2u; ++m)
                    tc_mma_i8_ts(d_base + sl.idx * 64u + m * 8u, a_base + sl.idx * 64u + m * 8u, tc_desc_kmajor_plain(bx + m * 256u, 128u), idesc);
                tc_commit_to(&mdone[sl.idx]);
                un.next(p.kb, NMAT);
                sl.advance(1, TC_SLOTS);
            }
            if (failed) set_status_word(a.status, KERNEL_ERR_GEMM_TIMEOUT);
        }
    } else if (warp < TC_W_EPI) {
        // ---- unpack warps: thread = row; quants -> unsigned bytes -> tensor memory ----
        const uint32_t grp = warp >> 2, q = warp & 3u, r = q * 32u + lane;
        TcRing st(0, p.stages), sl(0, TC_SLOTS);
        TcUnit un;
        un.init(u0, p.ut, p.kb);
        bool have_x = false;
        for (uint32_t i = 0; i < n_units && !failed; ++i) {
            if (!ptx::mbar_wait_sleep<0>(&full[st.idx], st.phase)) { failed = true; break; }
            // the A slot is free when its MMAs are done, the hand-off area when the epilogue has read it
            if (!ptx::mbar_wait_sleep<0>(&mdone[sl.idx], sl.phase ^ 1u) || !ptx::mbar_wait_sleep<0>(&dempty[sl.idx], sl.phase ^ 1u)) { failed = true; break; }
            tc_fence_after_sync();
            const uint4 *blk = reinterpret_cast<const uint4 *>(stages + (size_t)st.idx * p.stage_bytes + (size_t)r * 144u);
            const uint4 *src = blk + 1u + 4u * grp;                      // this half's 64 bytes of quants
            const uint32_t taddr = a_base + sl.idx * 64u + 32u * grp + ((q * 32u) << 16);
#pragma unroll
            for (uint32_t j = 0; j < 2; ++j) {          // 32 bytes: low nibbles = one sub-block, high nibbles = the next
                const uint4 w0 = src[2 * j], w1 = src[2 * j + 1];
                const uint32_t w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                uint32_t v[16];
#pragma unroll
                for (uint32_t k = 0; k < 8; ++k) {
                    v[k] = w[k] & 0x0f0f0f0fu;
                    v[8 + k] = (w[k] >> 4) & 0x0f0f0f0fu;
                }
                tmem_st16(taddr + 16u * j, v);
            }
            // hand the block header to the epilogue thread of this row and half, with the part of the sum
            // that needs no tensor-core result: dmin * sum over the half's sub-blocks of min * sum(x)
            {
                const uint4 hdr = blk[0];
                if (!have_x) {
                    if (!ptx::mbar_wait(xbar, 0)) { failed = true; break; }
                    have_x = true;
                }
                const uint32_t mnw = grp == 0 ? (hdr.z & 0x3f3f3f3fu) : (((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u));
                const float *sx = sums + 16u * un.b + 8u * grp;
                float tm = 0.f;
#pragma unroll
                for (uint32_t k = 0; k < 4; ++k) {
                    const float2 sq = *reinterpret_cast<const float2 *>(sx + 2u * k);
                    tm = fma_rn((float)((mnw >> (8u * k)) & 0xffu), add_rn(sq.x, sq.y), tm);
                }
                const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
                uint8_t *h = hand + sl.idx * TC_HAND_BYTES + grp * (TC_TILE * 20u);
                reinterpret_cast<uint4 *>(h)[r] = hdr;
                reinterpret_cast<float *>(h + TC_TILE * 16u)[r] = mul_rn(dmin, tm);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(&afull[2u * sl.idx + grp]);
                ptx::mbar_arrive(&empty[st.idx]);
            }
            st.advance(1, p.stages);
            sl.advance(1, TC_SLOTS);
            un.next(p.kb, NMAT);
        }
        if (failed && lane == 0) set_status_word(a.status, KERNEL_ERR_CONSUMER_TIMEOUT);
    } else if (warp < TC_W_COPY) {
        // ---- epilogue warps: thread = row; D -> scaled sums; at the end of every tile the CTA touches,
        // both groups deposit their sums for the flush warp ----
        const uint32_t grp = (warp - TC_W_EPI) >> 2, q = (warp - TC_W_EPI) & 3u, r = q * 32u + lane;
        TcRing sl(0, TC_SLOTS);
        uint32_t i = 0;                                     // next unit (index inside the CTA's range)
        const uint32_t tile_first = u0 / p.ut, tile_last = (u1 - 1) / p.ut;
        uint32_t buf = 0, buf_phase = 0;
        for (uint32_t tile = tile_first; tile <= tile_last && !failed; ++tile) {
            const uint32_t t_end = (tile + 1) * p.ut;                           // first unit after the tile
            const uint32_t i_end = (t_end < u1 ? t_end : u1) - u0;              // ... as an index in the CTA's range
            float acc[NMAT], accm[NMAT];
#pragma unroll
            for (int m = 0; m < NMAT; ++m) acc[m] = accm[m] = 0.f;
            uint32_t mb = NMAT == 2 ? (u0 + i - tile * p.ut) : 0u;              // unit inside the tile: matrix = mb / kb
            for (; i < i_end && !failed; ++i, ++mb) {
                const uint32_t m = NMAT == 2 ? (mb >= p.kb ? 1u : 0u) : 0u;
                if (!ptx::mbar_wait_sleep<0>(&mdone[sl.idx], sl.phase)) { failed = true; break; }
                tc_fence_after_sync();
                // the row's block header (d, dmin, 8 six-bit (scale, min) pairs) and min term, from the unpack thread
                const uint8_t *h = hand + sl.idx * TC_HAND_BYTES + grp * (TC_TILE * 20u);
                const uint4 hdr = reinterpret_cast<const uint4 *>(h)[r];
                const float minterm = reinterpret_cast<const float *>(h + TC_TILE * 16u)[r];
                const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
                const uint32_t scw = grp == 0 ? (hdr.y & 0x3f3f3f3fu) : ((hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u));
                int32_t c[4][4];
                const uint32_t taddr = d_base + sl.idx * 64u + 32u * grp + ((q * 32u) << 16);
#pragma unroll
                for (uint32_t k = 0; k < 4; ++k) tmem_ld4(taddr + 8u * k, c[k]);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&dempty[sl.idx]);
                float t = 0.f;
#pragma unroll
                for (uint32_t k = 0; k < 4; ++k) {
                    // |sum of q * round(x S)| <= 32 * 15 * 2^22 < 2^31: the digits recombine in int32
                    const float v = (float)(c[k][0] + (c[k][1] << 8) + (c[k][2] << 16));
                    t = fma_rn((float)((scw >> (8u * k)) & 0xffu), v, t);
                }
                if (m == 0) { acc[0] = fma_rn(d, t, acc[0]); accm[0] = add_rn(accm[0], minterm); }
                else { acc[NMAT - 1] = fma_rn(d, t, acc[NMAT - 1]); accm[NMAT - 1] = add_rn(accm[NMAT - 1], minterm); }
                sl.advance(1, TC_SLOTS);
            }
            if (failed) break;
            // deposit this half's sums
            if (!ptx::mbar_wait_sleep<0>(&fl_empty[buf], buf_phase ^ 1u)) { failed = true; break; }
            float *dst = deposit + ((size_t)buf * 2u + grp) * NMAT * TC_TILE;
#pragma unroll
            for (int m = 0; m < NMAT; ++m) dst[m * TC_TILE + r] = sub_rn(acc[m], accm[m]);
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&fl_full[buf]);
            buf ^= 1u;
            if (buf == 0) buf_phase ^= 1u;
        }
        if (failed && lane == 0) set_status_word(a.status, KERNEL_ERR_CONSUMER_TIMEOUT);
    } else if (warp == TC_W_FLUSH) {
        // ---- flush warp: lane l owns rows l, l + 32, l + 64, l + 96 of the tile.  A tile the CTA covers
        // alone goes straight to y; a shared one goes to this CTA's partial rows, and the last CTA to
        // arrive adds the partials in CTA order ----
        const uint32_t tile_first = u0 / p.ut, tile_last = (u1 - 1) / p.ut;
        uint32_t buf = 0, buf_phase = 0;
        bool have_x = false;
        float unscale = 1.f;
        for (uint32_t tile = tile_first; tile <= tile_last && !failed; ++tile) {
            if (!ptx::mbar_wait_sleep<0>(&fl_full[buf], buf_phase)) { failed = true; break; }
            if (!have_x) {
                if (!ptx::mbar_wait(xbar, 0)) { failed = true; break; }
                unscale = *reinterpret_cast<const float *>(ximg + (size_t)p.cols * 8u + p.cols / 4u);
                have_x = true;
            }
            const float *dep = deposit + (size_t)buf * 2u * NMAT * TC_TILE;
            float v[4][NMAT];
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j)
#pragma unroll
                for (int m = 0; m < NMAT; ++m)
                    v[j][m] = add_rn(dep[m * TC_TILE + j * 32u + lane], dep[(NMAT + m) * TC_TILE + j * 32u + lane]);
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&fl_empty[buf]);
            buf ^= 1u;
            if (buf == 0) buf_phase ^= 1u;
            const uint32_t t_begin = tile * p.ut, t_end = t_begin + p.ut;
            bool write_out = u0 <= t_begin && u1 >= t_end;
            if (!write_out) {
                const uint32_t first = tc_cta_of(t_begin, p.units, gridDim.x), last = tc_cta_of(t_end - 1, p.units, gridDim.x);
                float *mine = a.partials + ((size_t)tile * p.maxc + (blockIdx.x - first)) * NMAT * TC_TILE;
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j)
#pragma unroll
                    for (int m = 0; m < NMAT; ++m) mine[m * TC_TILE + j * 32u + lane] = v[j][m];
                __threadfence();
                __syncwarp();
                uint32_t arrived = 0;
                if (lane == 0) arrived = atomicAdd(&a.counters[tile], 1u);
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                if (arrived == last - first) {
                    __threadfence();
                    const float *all = a.partials + (size_t)tile * p.maxc * NMAT * TC_TILE;
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j)
#pragma unroll
                        for (int m = 0; m < NMAT; ++m) v[j][m] = 0.f;
                    for (uint32_t cc = 0; cc <= last - first; ++cc)
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j)
#pragma unroll
                            for (int m = 0; m < NMAT; ++m)
                                v[j][m] = add_rn(v[j][m], __ldcg(all + ((size_t)cc * NMAT + m) * TC_TILE + j * 32u + lane));
                    if (lane == 0) a.counters[tile] = 0u;
                    write_out = true;
                }
            }
            if (write_out) {
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) {
                    const uint32_t row = tile * TC_TILE + j * 32u + lane;
                    if (row < p.rows) {
                        const float g = mul_rn(v[j][0], unscale);
                        a.y[row] = NMAT == 2 ? glu_f(g, mul_rn(v[j][NMAT - 1], unscale), a.glu == 2) : g;
                    }
                }
            }
        }
        if (failed && lane == 0) set_status_word(a.status, KERNEL_ERR_CONSUMER_TIMEOUT);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == TC_W_MMA) {
        tc_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
    }
}

// ---- host: tensor maps and launch ----------------------------------------------------------

// rows x stride bytes, boxes of 128 rows x box_bytes
static bool make_row_map(CUtensorMap &map, const uint8_t *w, uint32_t rows, uint32_t stride, uint32_t box_bytes) {
    return make_tensor_map_2d(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, w, stride, rows, stride, box_bytes, TC_TILE, CU_TENSOR_MAP_SWIZZLE_NONE);
}

template <int NMAT>
static cudaError_t launch_tc_t(const CUtensorMap &m0, const CUtensorMap &m1, const TcArgs &a, cudaStream_t stream, bool pdl) {
    auto kernel = gemv_tc_q4k_kernel<NMAT>;
    static DeviceOnce once;
    {
        const cudaError_t e = once.smem(kernel, (int)TC_SMEM_MAX);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.p.ctas);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = a.p.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, m0, m1, a);
}

// True when this call was taken (launched or failed); false to let the caller use another kernel.
bool try_launch_gemv_tc(const GemvCall &c, const LaunchCtx &ctx, cudaError_t &err) {
    if (c.ids || c.count != 1 || c.kind != KIND_Q4_K || !ctx.tc_scratch) return false;
    if (((uintptr_t)c.w[0] % 16u) || (c.nmat == 2 && ((uintptr_t)c.w[1] % 16u))) return false;
    TcPlan p;
    if (!plan_tc(c.kind, c.cols, c.rows, c.stride, c.nmat, ctx.sm_count, p)) return false;
    const size_t counter_bytes = ((size_t)p.tiles * 4u + 255u) & ~(size_t)255u;
    const size_t partial_bytes = (size_t)p.tiles * p.maxc * p.nmat * TC_TILE * 4u;
    if (counter_bytes > TC_COUNTER_BYTES || TC_COUNTER_BYTES + partial_bytes > ctx.tc_scratch_bytes) return false;
    const uint8_t *xq = static_cast<const uint8_t *>(c.x);
    if (c.x_packed == 3u) {
        if ((uintptr_t)xq % 16u) return false;
    } else if (c.x_packed) {
        return false;
    } else {
        if (!ctx.workspace || p.x_bytes > ctx.workspace_bytes) return false;
        err = launch_pack_digits(c.x, c.x_bf16, 1, c.cols, ctx.workspace, ctx);
        if (err != cudaSuccess) return true;
        xq = static_cast<const uint8_t *>(ctx.workspace);
    }
    CUtensorMap m0, m1;
    const size_t mat_off = (size_t)c.expert * c.rows * c.stride;
    if (!make_row_map(m0, c.w[0] + mat_off, c.rows, c.stride, p.box_bytes)) return false;
    if (c.nmat == 2) {
        if (!make_row_map(m1, c.w[1] + mat_off, c.rows, c.stride, p.box_bytes)) return false;
    } else m1 = m0;
    TcArgs a = {};
    a.p = p;
    a.xq = xq;
    a.y = c.y;
    a.counters = static_cast<uint32_t *>(ctx.tc_scratch);
    a.partials = reinterpret_cast<float *>(static_cast<uint8_t *>(ctx.tc_scratch) + TC_COUNTER_BYTES);
    a.glu = c.glu;
    a.status = ctx.status;
    err = c.nmat == 2 ? launch_tc_t<2>(m0, m1, a, ctx.stream, ctx.pdl) : launch_tc_t<1>(m0, m1, a, ctx.stream, ctx.pdl);
    return true;
}

}  // namespace ingot
