// Expert-parallel token exchange for the routed FFN: the experts of a layer are split over the GPUs of a
// node (rank r owns experts [r E / world, (r + 1) E / world)), every rank routes its OWN tokens, and the rows
// travel to the ranks that own the chosen experts and back:
//
//   dispatch  every routed pair (token, k) of this rank: the token's activation row and a word
//             {local expert id, pair index} go, with plain stores over NVLink, into region `rank` of the OWNER's
//             receive area; unused places of the region are marked ROUTE_SKIP; the launch's last CTA then stores
//             one tagged word per owner ("region `rank` is complete for this step")
//   receive   the owner polls the tagged words of all regions (bounded) and writes the expert ids of the
//             world x cap places for the routed projections, which skip the unused ones
//   return    after its experts ran, the owner stores each live place's output row into the HOME rank's return
//             rows at the pair's index, then one tagged word per home rank
//   combine   the home rank polls the tagged words (bounded) and sums its pairs' rows with the router's weights,
//             in route order (what moe_sum computes: kernels/generic.metal:17)
//
// The reference keeps every expert on its one device (src/weights.rs:55-58) and runs the pairs there
// (Generic::moe, src/generic.rs:508-574); this file replaces that residency with a split, and nothing else: a
// pair's arithmetic is the single-device one, so results are bit-identical.  No collective library is involved;
// every wait is bounded and reports through the status word.
#include <cuda_runtime.h>

#include <cstdint>

#include "dev_common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace ingot {

namespace {

constexpr uint32_t EP_THREADS = 256;

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

__device__ __forceinline__ uint32_t step_tag(const EpLink &l) {
    return *reinterpret_cast<const volatile uint32_t *>(l.step) * l.tag_mul + l.tag_add;
}

// Bounded poll of one tagged word; the low half of the word on success.
__device__ __forceinline__ bool poll_tagged(const uint64_t *word, uint32_t tag, uint32_t &low) {
    uint64_t t0 = 0;
    for (;;) {
        for (int i = 0; i < 256; ++i) {
            uint64_t w;
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(word) : "memory");
            if ((uint32_t)(w >> 32) == tag) { low = (uint32_t)w; return true; }
            __nanosleep(32);
        }
        const uint64_t now = ptx::global_timer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > ptx::WAIT_LIMIT_NS) return false;
    }
}

// All rows of this CTA are stored.  The CTA counts itself on the own device (release at device scope); the
// launch's last CTA releases at system scope and stores the tagged words: causality order carries every CTA's
// stores through the counter to whoever acquires a word.  The last CTA also sets the counter back to zero, so
// launches of different grid sizes can follow each other (the next launch's CTAs count only after their
// griddepcontrol.wait, when this launch is complete).
template <class F>
__device__ __forceinline__ void signal_when_last(uint32_t *launch_count, F store_words) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t before = atomicAdd(launch_count, 1u);
        if (before + 1u == gridDim.x) {
            atomicExch(launch_count, 0u);
            __threadfence_system();
            store_words();
        }
    }
}

__device__ __forceinline__ void store_tagged(uint64_t *word, uint32_t tag, uint32_t low) {
    const uint64_t w = ((uint64_t)tag << 32) | low;
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(word), "l"(w) : "memory");
}

__device__ __forceinline__ void copy_row(float *dst, const float *src, uint32_t width, uint32_t lane) {
    const float4 *s = reinterpret_cast<const float4 *>(src);
    float4 *d = reinterpret_cast<float4 *>(dst);
    for (uint32_t j = lane; j < (width >> 2); j += 32u) d[j] = __ldcg(s + j);
}

struct DispatchArgs {
    EpLink link;
    const float *x;              // [tokens][hidden], this rank's tokens
    const uint32_t *ids;         // [pairs] global expert ids in route order
    uint32_t pairs, top, hidden, cap, experts_per_rank;
    int *status;
};

// Every CTA works out the whole placement (a pair's place in its owner's region = the number of earlier pairs
// with the same owner: deterministic, in pair order); the copies are shared out by pair.
__global__ void __launch_bounds__(EP_THREADS) ep_dispatch_kernel(const __grid_constant__ DispatchArgs a) {
    extern __shared__ uint32_t sm[];
    uint32_t *owner = sm, *place = sm + a.pairs, *count = sm + 2u * a.pairs;        // [pairs], [pairs], [world]
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    const EpLink &l = a.link;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, nwarps = EP_THREADS / 32u;
    if (tid < l.world) count[tid] = 0u;
    for (uint32_t p = tid; p < a.pairs; p += EP_THREADS) {
        const uint32_t e = a.ids[p];
        uint32_t o = e / a.experts_per_rank;
        if (o >= l.world) { set_status_word(a.status, KERNEL_ERR_EXPERT_RANGE); o = TP_MAX_RANKS; }
        owner[p] = o;
    }
    __syncthreads();
    for (uint32_t p = tid; p < a.pairs; p += EP_THREADS) {
        const uint32_t o = owner[p];
        uint32_t n = 0;
        for (uint32_t q = 0; q < p; ++q) n += owner[q] == o ? 1u : 0u;
        place[p] = n;
        if (o < l.world) atomicAdd(&count[o], 1u);
    }
    __syncthreads();
    for (uint32_t p = blockIdx.x * nwarps + warp; p < a.pairs; p += gridDim.x * nwarps) {
        const uint32_t o = owner[p];
        if (o >= l.world) continue;
        const size_t at = (size_t)l.rank * a.cap + place[p];
        copy_row(l.rx_rows[o] + at * a.hidden, a.x + (size_t)(p / a.top) * a.hidden, a.hidden, lane);
        if (lane == 0) l.rx_meta[o][at] = (a.ids[p] - o * a.experts_per_rank) | (p << 16);
    }
    // the unused places of this rank's region on every owner
    for (uint32_t i = blockIdx.x * EP_THREADS + tid; i < l.world * a.cap; i += gridDim.x * EP_THREADS) {
        const uint32_t o = i / a.cap, k = i - o * a.cap;
        if (k >= count[o]) l.rx_meta[o][(size_t)l.rank * a.cap + k] = ROUTE_SKIP;
    }
    const uint32_t tag = step_tag(l);
    signal_when_last(l.launch_count, [&] {
        for (uint32_t o = 0; o < l.world; ++o) store_tagged(l.rx_ready[o] + l.rank, tag, count[o]);
    });
}

struct ReceiveArgs {
    EpLink link;
    uint32_t cap;
    uint32_t *ids_out;           // [world * cap] local expert id or ROUTE_SKIP
    int *status;
};

__global__ void __launch_bounds__(EP_THREADS) ep_receive_kernel(const __grid_constant__ ReceiveArgs a) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    const EpLink &l = a.link;
    const uint32_t tag = step_tag(l);
    if (threadIdx.x < l.world && !(a.status && *reinterpret_cast<const volatile int *>(a.status) != 0)) {
        uint32_t n;
        if (!poll_tagged(l.rx_ready[l.rank] + threadIdx.x, tag, n)) set_status_word(a.status, KERNEL_ERR_PEER_TIMEOUT);
    }
    __syncthreads();
    for (uint32_t i = blockIdx.x * EP_THREADS + threadIdx.x; i < l.world * a.cap; i += gridDim.x * EP_THREADS) {
        const uint32_t m = __ldcg(l.rx_meta[l.rank] + i);
        a.ids_out[i] = m == ROUTE_SKIP ? ROUTE_SKIP : (m & 0xffffu);
    }
}

struct ReturnArgs {
    EpLink link;
    const float *rows;           // [world * cap][hidden] outputs of the places
    const uint32_t *inverse;     // null, or the row of each place (outputs in the expert grouping's packed order)
    uint32_t cap, hidden;
};

__global__ void __launch_bounds__(EP_THREADS) ep_return_kernel(const __grid_constant__ ReturnArgs a) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    const EpLink &l = a.link;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, nwarps = EP_THREADS / 32u;
    for (uint32_t i = blockIdx.x * nwarps + warp; i < l.world * a.cap; i += gridDim.x * nwarps) {
        const uint32_t m = __ldcg(l.rx_meta[l.rank] + i);
        if (m == ROUTE_SKIP) continue;
        const uint32_t home = i / a.cap, pair = m >> 16;
        const size_t row = a.inverse ? a.inverse[i] : i;
        copy_row(l.ret_rows[home] + (size_t)pair * a.hidden, a.rows + row * a.hidden, a.hidden, lane);
    }
    const uint32_t tag = step_tag(l);
    signal_when_last(l.launch_count, [&] {
        for (uint32_t h = 0; h < l.world; ++h) store_tagged(l.ret_ready[h] + l.rank, tag, 0u);
    });
}

struct CombineArgs {
    EpLink link;
    const float *w;              // [tokens * top] router weights of this rank's pairs
    float *y;                    // [tokens][hidden]
    uint32_t hidden, top, tokens;
    int *status;
};

__global__ void __launch_bounds__(EP_THREADS) ep_combine_kernel(const __grid_constant__ CombineArgs a) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    const EpLink &l = a.link;
    const uint32_t tag = step_tag(l);
    if (threadIdx.x < l.world && !(a.status && *reinterpret_cast<const volatile int *>(a.status) != 0)) {
        uint32_t n;
        if (!poll_tagged(l.ret_ready[l.rank] + threadIdx.x, tag, n)) set_status_word(a.status, KERNEL_ERR_PEER_TIMEOUT);
    }
    __syncthreads();
    const float *rows = l.ret_rows[l.rank];
    const uint32_t w4 = a.hidden >> 2;
    const uint64_t total = (uint64_t)a.tokens * w4;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(idx / w4), j = (uint32_t)(idx - (uint64_t)t * w4);
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t e = 0; e < a.top; ++e) {
            const uint32_t pair = t * a.top + e;
            const float4 r = __ldcg(reinterpret_cast<const float4 *>(rows + (size_t)pair * a.hidden) + j);
            const float wt = a.w[pair];
            s.x = __fmaf_rn(r.x, wt, s.x); s.y = __fmaf_rn(r.y, wt, s.y);
            s.z = __fmaf_rn(r.z, wt, s.z); s.w = __fmaf_rn(r.w, wt, s.w);
        }
        reinterpret_cast<float4 *>(a.y + (size_t)t * a.hidden)[j] = s;
    }
}

uint32_t ctas_for(uint32_t warps_of_work, const LaunchCtx &ctx) {
    uint32_t ctas = (warps_of_work + EP_THREADS / 32u - 1u) / (EP_THREADS / 32u);
    if (ctas > ctx.sm_count) ctas = ctx.sm_count;
    return ctas ? ctas : 1u;
}

}  // namespace

cudaError_t launch_ep_dispatch(const EpLink &link, const float *x, const uint32_t *ids, uint32_t pairs, uint32_t top, uint32_t hidden,
                               uint32_t cap, uint32_t experts_per_rank, const LaunchCtx &ctx) {
    if (hidden % 4u || pairs > EP_MAX_PAIRS || pairs > cap || top == 0 || experts_per_rank == 0 || experts_per_rank > 0x10000u)
        return cudaErrorInvalidValue;
    DispatchArgs a = {link, x, ids, pairs, top, hidden, cap, experts_per_rank, ctx.status};
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas_for(pairs, ctx));
    cfg.blockDim = dim3(EP_THREADS);
    cfg.dynamicSmemBytes = (2u * pairs + TP_MAX_RANKS) * 4u;
    cfg.stream = ctx.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, ep_dispatch_kernel, a);
}

cudaError_t launch_ep_receive(const EpLink &link, uint32_t cap, uint32_t *ids_out, const LaunchCtx &ctx) {
    ReceiveArgs a = {link, cap, ids_out, ctx.status};
    return launch(ep_receive_kernel, dim3(1), dim3(EP_THREADS), ctx, a);
}

cudaError_t launch_ep_return(const EpLink &link, const float *rows, const uint32_t *inverse, uint32_t cap, uint32_t hidden,
                             const LaunchCtx &ctx) {
    if (hidden % 4u) return cudaErrorInvalidValue;
    ReturnArgs a = {link, rows, inverse, cap, hidden};
    return launch(ep_return_kernel, dim3(ctas_for(cap, ctx)), dim3(EP_THREADS), ctx, a);
}

cudaError_t launch_ep_combine(const EpLink &link, const float *w, uint32_t hidden, uint32_t top, uint32_t tokens, float *y,
                              const LaunchCtx &ctx) {
    if (hidden % 4u) return cudaErrorInvalidValue;
    CombineArgs a = {link, w, y, hidden, top, tokens, ctx.status};
    const uint64_t total = (uint64_t)tokens * (hidden >> 2);
    uint64_t blocks = (total + EP_THREADS - 1u) / EP_THREADS;
    if (blocks > ctx.sm_count) blocks = ctx.sm_count;
    return launch(ep_combine_kernel, dim3(blocks ? (uint32_t)blocks : 1u), dim3(EP_THREADS), ctx, a);
}

}  // namespace ingot
