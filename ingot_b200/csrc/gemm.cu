// Batched prefill: Y[T][N] = X[T][K] . W^T for block-quantised W, on the 5th-generation
// tensor cores (tcgen05) with dequantise-on-load.
//
// Replaces the reference's generic_gemm / gemm_q4k / gemm_q6k (kernels/generic.metal:315-388):
// like it, weights AND activations are rounded to binary16 before the product and the
// accumulation is fp32 (its simdgroup_half8x8 staging, :343,355-361), so results are held
// to the same expectation (f64 dot of F16-rounded operands, src/expert_bench.rs:734-749).
//
// One CTA computes a 128 (weight rows) x 256 (tokens) tile of Y^T.  Per 64-column K step:
//   * four warps decode one weight row each — the fp32 value d*sc*q - dmin*m (Q4_K) or
//     d*scale*(q-32) (Q6_K) exactly as weight_at forms it, rounded to binary16 — and store
//     the 128 x 64 tile K-major with the 128-byte swizzle the tensor core expects;
//   * two warps bring the 256 x 64 activation tile (already binary16) with 16-byte
//     cp.async into the same swizzled layout;
//   * one thread issues four tcgen05.mma (M 128, N 256, K 16) accumulating in tensor
//     memory (256 columns x 128 lanes of fp32), and a tcgen05.commit frees the stage.
// After the last step the four decode warps read the accumulator with tcgen05.ld and write
// Y (token-major) with coalesced stores.  Every wait is bounded.
#include <cuda_fp16.h>

#include "dev_common.cuh"
#include "gemv_core.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace ingot {

static constexpr uint32_t GEMM_M = 128;          // weight rows per CTA (MMA M)
static constexpr uint32_t GEMM_N = 256;          // tokens per CTA (MMA N)
static constexpr uint32_t GEMM_K = 64;           // columns per stage (4 MMAs of K 16)
static constexpr uint32_t GEMM_STAGES = 4;
static constexpr uint32_t GEMM_A_BYTES = GEMM_M * GEMM_K * 2;       // 16 KB
static constexpr uint32_t GEMM_B_BYTES = GEMM_N * GEMM_K * 2;       // 32 KB
static constexpr uint32_t GEMM_STAGE_BYTES = GEMM_A_BYTES + GEMM_B_BYTES;
static constexpr uint32_t GEMM_THREADS = 224;    // 4 decode/epilogue warps, 2 activation warps, 1 MMA warp
static constexpr uint32_t GEMM_SMEM = 1024 + GEMM_STAGES * GEMM_STAGE_BYTES + 1024;   // + alignment slack

struct GemmArgs {
    const uint8_t *w;          // [rows][stride] of expert `expert`
    const __half *x;           // [tokens][cols] binary16
    float *y;                  // [tokens][rows]
    uint32_t cols, rows, stride, kind, tokens;
    int *status;
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

// ---- decoding 64 consecutive weights of one row into a swizzled tile row ------------------

// Q4_K: K step ks covers group j = ks % 4 of block ks / 4: 32 bytes, low nibbles = sub-block 2j
// (columns 0..31 of the step), high nibbles = sub-block 2j+1 (columns 32..63).
__device__ __forceinline__ void decode64_q4k(const uint8_t *row, uint32_t ks, uint8_t *dst_row_base, uint32_t r) {
    const uint8_t *b = row + (size_t)(ks >> 2) * 144u;
    const uint32_t j = ks & 3u;
    const uint4 hdr = *reinterpret_cast<const uint4 *>(b);
    uint32_t sc0, m0, sc1, m1;
    const uint8_t *s = reinterpret_cast<const uint8_t *>(&hdr) + 4;
    q4k_scale_min(s, 2 * j, sc0, m0);
    q4k_scale_min(s, 2 * j + 1, sc1, m1);
    const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
    const float ds0 = __fmul_rn(dd.x, (float)sc0), ds1 = __fmul_rn(dd.x, (float)sc1);
    const float c0 = __fmul_rn(dd.y, (float)m0), c1 = __fmul_rn(dd.y, (float)m1);
    const uint4 q0 = *reinterpret_cast<const uint4 *>(b + 16u + 32u * j);
    const uint4 q1 = *reinterpret_cast<const uint4 *>(b + 32u + 32u * j);
    const uint32_t qs[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (uint32_t c = 0; c < 4; ++c) {           // 16-byte chunk c: columns 8c..8c+7 (low), 32+8c.. (high)
        uint32_t lo[4], hi[4];
#pragma unroll
        for (uint32_t i = 0; i < 2; ++i) {
            const uint32_t wq = qs[2 * c + i];
#pragma unroll
            for (uint32_t e = 0; e < 2; ++e) {
                const float a0 = (float)((wq >> (16 * e)) & 15u), a1 = (float)((wq >> (16 * e + 8)) & 15u);
                const float b0 = (float)((wq >> (16 * e + 4)) & 15u), b1 = (float)((wq >> (16 * e + 12)) & 15u);
                lo[2 * i + e] = pack_h2(__fsub_rn(__fmul_rn(ds0, a0), c0), __fsub_rn(__fmul_rn(ds0, a1), c0));
                hi[2 * i + e] = pack_h2(__fsub_rn(__fmul_rn(ds1, b0), c1), __fsub_rn(__fmul_rn(ds1, b1), c1));
            }
        }
        *reinterpret_cast<uint4 *>(dst_row_base + swz_off(r, c)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        *reinterpret_cast<uint4 *>(dst_row_base + swz_off(r, 4u + c)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    }
}

// Q6_K: K step ks covers half n = (ks % 4) / 2 of block ks / 4 and quarters q0 = 2 * (ks % 2), q0 + 1.
__device__ __forceinline__ void decode64_q6k(const uint8_t *row, uint32_t ks, uint8_t *dst_row_base, uint32_t r) {
    const uint8_t *b = row + (size_t)(ks >> 2) * 210u;
    const uint32_t n = (ks >> 1) & 1u, q0 = 2u * (ks & 1u);
    const float d = __half2float(*reinterpret_cast<const __half *>(b + 208));
#pragma unroll
    for (uint32_t qq = 0; qq < 2; ++qq) {
        const uint32_t q = q0 + qq;
        const uint8_t *ql = b + 64u * n + 32u * (q & 1u), *qh = b + 128u + 32u * n;
#pragma unroll
        for (uint32_t c = 0; c < 4; ++c) {       // columns 32 qq + 8c .. + 7  (l = 8c .. 8c + 7)
            const int scale = (int)(int8_t)b[192u + 8u * n + 2u * q + (c >> 1)];
            const float ds = __fmul_rn(d, (float)scale);
            uint32_t out[4];
#pragma unroll
            for (uint32_t e = 0; e < 4; ++e) {
                const uint32_t l = 8u * c + 2u * e;
                const uint32_t v0 = (((uint32_t)ql[l] >> (q >= 2 ? 4 : 0)) & 15u) | ((((uint32_t)qh[l] >> (2 * q)) & 3u) << 4);
                const uint32_t v1 = (((uint32_t)ql[l + 1] >> (q >= 2 ? 4 : 0)) & 15u) | ((((uint32_t)qh[l + 1] >> (2 * q)) & 3u) << 4);
                out[e] = pack_h2(__fmul_rn(ds, (float)((int)v0 - 32)), __fmul_rn(ds, (float)((int)v1 - 32)));
            }
            *reinterpret_cast<uint4 *>(dst_row_base + swz_off(r, 4u * qq + c)) = make_uint4(out[0], out[1], out[2], out[3]);
        }
    }
}

__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_dequant_tcgen05_kernel(const __grid_constant__ GemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte aligned tiles (the swizzle pattern repeats every 1024 bytes)
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    uint64_t *full_a = reinterpret_cast<uint64_t *>(smem);          // [STAGES] decode warps -> MMA
    uint64_t *full_b = full_a + GEMM_STAGES;                          // [STAGES] activation warps -> MMA
    uint64_t *empty = full_b + GEMM_STAGES;                           // [STAGES] MMA -> producers
    uint64_t *acc_full = empty + GEMM_STAGES;                         // accumulator complete
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
    uint8_t *tiles = smem + 1024;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t n0 = blockIdx.x * GEMM_M, t0 = blockIdx.y * GEMM_N;
    const uint32_t ksteps = a.cols / GEMM_K;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < GEMM_STAGES; ++s) {
            ptx::mbar_init(&full_a[s], 128);
            ptx::mbar_init(&full_b[s], 64);
            ptx::mbar_init(&empty[s], 1);
        }
        ptx::mbar_init(acc_full, 1);
        ptx::mbar_init_fence();
    }
    if (warp == 6) tmem_alloc(tmem_slot, GEMM_N);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();

    bool failed = false;
    if (warp < 4) {
        // ---- decode warps: one weight row per thread ----
        const uint32_t r = threadIdx.x;                               // row inside the tile = TMEM lane
        const bool live = n0 + r < a.rows;
        const uint8_t *row = a.w + (size_t)(live ? n0 + r : 0) * a.stride;
        for (uint32_t ks = 0; ks < ksteps && !failed; ++ks) {
            const uint32_t s = ks % GEMM_STAGES, ph = (ks / GEMM_STAGES) & 1u;
            if (!ptx::mbar_wait_sleep<20>(&empty[s], ph ^ 1u)) { failed = true; break; }
            uint8_t *dst = tiles + (size_t)s * GEMM_STAGE_BYTES;
            if (live) {
                if (a.kind == KIND_Q4_K) decode64_q4k(row, ks, dst, r);
                else decode64_q6k(row, ks, dst, r);
            } else {
#pragma unroll
                for (uint32_t c = 0; c < 8; ++c) *reinterpret_cast<uint4 *>(dst + swz_off(r, c)) = make_uint4(0, 0, 0, 0);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy stores -> tensor core reads
            ptx::mbar_arrive(&full_a[s]);
        }
        // ---- epilogue: this warp reads TMEM lanes 32 * warp .. + 31 ----
        if (!failed && !ptx::mbar_wait_sleep<64>(acc_full, 0)) failed = true;
        if (!failed) {
            tc_fence_after();
            const uint32_t rowg = n0 + r;
#pragma unroll 1
            for (uint32_t c0 = 0; c0 < GEMM_N; c0 += 32) {
                float v[32];
                tmem_ld32(tmem_base + ((warp * 32u) << 16) + c0, v);
                if (rowg < a.rows) {
#pragma unroll
                    for (uint32_t i = 0; i < 32; ++i) {
                        const uint32_t t = t0 + c0 + i;
                        if (t < a.tokens) a.y[(size_t)t * a.rows + rowg] = v[i];
                    }
                }
            }
        }
    } else if (warp < 6) {
        // ---- activation warps: 256 tokens x 64 columns of binary16 per stage, 16 bytes per cp.async ----
        const uint32_t tid = threadIdx.x - 128u;                       // 0..63
        for (uint32_t ks = 0; ks < ksteps && !failed; ++ks) {
            const uint32_t s = ks % GEMM_STAGES, ph = (ks / GEMM_STAGES) & 1u;
            if (!ptx::mbar_wait_sleep<20>(&empty[s], ph ^ 1u)) { failed = true; break; }
            uint8_t *dst = tiles + (size_t)s * GEMM_STAGE_BYTES + GEMM_A_BYTES;
#pragma unroll 4
            for (uint32_t i = tid; i < GEMM_N * 8u; i += 64u) {
                const uint32_t tok = i >> 3, chunk = i & 7u;
                const uint32_t t = t0 + tok;
                const __half *src = a.x + (size_t)(t < a.tokens ? t : 0) * a.cols + (size_t)ks * GEMM_K + chunk * 8u;
                const uint32_t bytes = t < a.tokens ? 16u : 0u;        // rows past the end are zero-filled
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(ptx::smem_addr(dst + swz_off(tok, chunk))), "l"(src),
                             "r"(bytes)
                             : "memory");
            }
            // the barrier gets this thread's arrival when its copies above have landed
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(ptx::smem_addr(&full_b[s])) : "memory");
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (lane == 0) {
        // ---- MMA thread ----
        const uint32_t idesc = idesc_f16(GEMM_M, GEMM_N);
        for (uint32_t ks = 0; ks < ksteps && !failed; ++ks) {
            const uint32_t s = ks % GEMM_STAGES, ph = (ks / GEMM_STAGES) & 1u;
            if (!ptx::mbar_wait_sleep<0>(&full_a[s], ph) || !ptx::mbar_wait_sleep<0>(&full_b[s], ph)) { failed = true; break; }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // tiles were written through the generic proxy
            tc_fence_after();
            const uint32_t a_addr = ptx::smem_addr(tiles + (size_t)s * GEMM_STAGE_BYTES), b_addr = a_addr + GEMM_A_BYTES;
#pragma unroll
            for (uint32_t k = 0; k < GEMM_K / 16u; ++k)
                tc_mma_f16(tmem_base, smem_desc_k128(a_addr + k * 32u), smem_desc_k128(b_addr + k * 32u), idesc, (ks | k) != 0u);
            tc_commit(&empty[s]);                                     // frees the stage when these MMAs are done
        }
        if (!failed) tc_commit(acc_full);
    }
    if (failed && lane == 0) set_status_word(a.status, KERNEL_ERR_GEMM_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 6) tmem_dealloc(tmem_base, GEMM_N);
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

cudaError_t launch_gemm_dequant(const uint8_t *w, uint32_t cols, uint32_t rows, uint32_t stride, uint32_t kind, uint32_t expert,
                                const void *x, uint32_t x_bf16, uint32_t tokens, float *y, void *x_half_scratch,
                                const LaunchCtx &ctx) {
    if (kind != KIND_Q4_K && kind != KIND_Q6_K) return cudaErrorNotSupported;
    if (cols % 256u || tokens == 0 || rows == 0) return cudaErrorInvalidValue;
    if (((uintptr_t)w % 16u) || (stride % 2u) || (kind == KIND_Q4_K && stride % 16u)) return cudaErrorNotSupported;
    ToHalfArgs h = {x, static_cast<__half *>(x_half_scratch), (uint64_t)tokens * cols, x_bf16};
    uint64_t blocks = (h.n + 255) / 256, cap = (uint64_t)ctx.sm_count * 16u;
    if (blocks > cap) blocks = cap;
    to_half_kernel<<<(uint32_t)blocks, 256, 0, ctx.stream>>>(h);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    static bool configured = false;
    if (!configured) {
        e = cudaFuncSetAttribute(gemm_dequant_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    GemmArgs a = {w + (size_t)expert * rows * stride, static_cast<const __half *>(x_half_scratch), y, cols, rows, stride, kind, tokens,
                  ctx.status};
    dim3 grid((rows + GEMM_M - 1) / GEMM_M, (tokens + GEMM_N - 1) / GEMM_N);
    gemm_dequant_tcgen05_kernel<<<grid, GEMM_THREADS, GEMM_SMEM, ctx.stream>>>(a);
    return cudaGetLastError();
}

}  // namespace ingot
