// Inline-PTX helpers for sm_100a: mbarrier, 1-D bulk async copies (TMA without
// a tensor map), programmatic dependent launch, cache-hinted loads.
//
// Every wait is bounded: after WAIT_LIMIT_NS the caller records an error
// code in the device status word and leaves, so a lost copy or a mis-sized
// transaction can never hang the GPU.
#pragma once
#include <stdint.h>

namespace ingot {
namespace ptx {

static constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;   // two seconds of wall time

__device__ __forceinline__ uint32_t smem_addr(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}

// Makes freshly initialised barriers visible to the async proxy.
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait: polls until the phase completes or WAIT_LIMIT_NS of wall time have
// passed; false when the limit ran out.  Between polls the warp sleeps SLEEP_NS so a
// waiting warp does not take issue slots from the warps doing the arithmetic.
template <uint32_t SLEEP_NS>
__device__ __forceinline__ bool mbar_wait_sleep(uint64_t *bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    // the clock is read only every 1024 polls: reading it costs hundreds of cycles, and an
    // ordinary wait ends within a few polls
    uint64_t t0 = 0;
    for (;;) {
        for (int i = 0; i < 1024; ++i) {
            if (SLEEP_NS) __nanosleep(SLEEP_NS);
            if (mbar_try_wait(bar, parity)) return true;
        }
        const uint64_t now = global_timer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > WAIT_LIMIT_NS) return false;
    }
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) { return mbar_wait_sleep<0>(bar, parity); }

// Global -> shared bulk copy of `bytes` (multiple of 16; both addresses 16-byte
// aligned) that signals `bar` with complete_tx.  No multicast.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_addr(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
        : "memory");
}

// Tiled 2-D copy global -> shared through a tensor map (in global or parameter memory): the box at
// element coordinates (x, y), x the inner one; x times the element size must be a multiple of 16
// bytes.  Signals `bar` with the bytes of the whole box.  No multicast.
__device__ __forceinline__ void tma_load_2d(void *dst_smem, const void *tensor_map, uint32_t x, uint32_t y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_addr(dst_smem)),
                 "l"(tensor_map), "r"(x), "r"(y), "r"(smem_addr(bar))
                 : "memory");
}

// Programmatic dependent launch: let the next kernel in the stream begin its
// prologue; wait until the previous kernel's writes are visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

}  // namespace ptx
}  // namespace ingot
