// Small device helpers shared by the kernel files.
#pragma once
#include <stdint.h>

namespace ingot {

// Routed pair that this device does not own (expert-parallel sharding): its output row is zero.
static constexpr uint32_t ROUTE_SKIP = 0xffffffffu;

// Records the first error of a launch in the device status word.
__device__ __forceinline__ void set_status_word(int *status, int code) {
    if (status) atomicCAS(status, 0, code);
}

// Activation element i as float32 (bf16 widens exactly).
__device__ __forceinline__ float load_x(const void *x, size_t i, uint32_t bf16) {
    return bf16 ? __uint_as_float((uint32_t)static_cast<const uint16_t *>(x)[i] << 16) : static_cast<const float *>(x)[i];
}

}  // namespace ingot
