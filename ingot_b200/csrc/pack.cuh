// Writing activations in the order the tensor-core GEMV reads them.
// Packed row for `cols` activations (a multiple of 64):
//   [cols/16 MMAs][2 parts: xh, xl][4 lanes][4 halves]   binary16 (high, low) split
//   [cols/16] fp32 sums of each 16 (scaled) activations
//   16 bytes: 1/scale (x is pre-multiplied by a power of two when |x| would overflow binary16)
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace ingot {

// Power of two that brings max|x| = mx below 2^14 (1 when it already is).
__device__ __forceinline__ float pack_scale(float mx) {
    if (!(mx >= 16384.0f) || !(mx < INFINITY)) return 1.0f;
    int e;
    frexpf(mx, &e);                       // mx = f * 2^e, f in [0.5, 1)
    return ldexpf(1.0f, 14 - e);          // mx * scale in [2^13, 2^14)
}

// One thread stores four consecutive activations v[0..3] (already scaled) = columns
// 4q..4q+3: the word of lane t = q % 4 of MMA mi = q / 4.  All four threads of a quad
// (consecutive q) must call this together: the 16-column sum uses quad shuffles.
__device__ __forceinline__ void pack_store_quad(uint8_t *row, uint32_t cols, uint32_t q, const float (&v)[4], bool live) {
    const uint32_t mi = q >> 2, t = q & 3u;
    __half h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        h[i] = __float2half_rn(v[i]);
        l[i] = __float2half_rn(v[i] - __half2float(h[i]));
    }
    if (live) {
        // slots: byte 0 -> b0.lo, byte 2 -> b0.hi, byte 1 -> b1.lo, byte 3 -> b1.hi
        __half *xf = reinterpret_cast<__half *>(row);
        __half2 *dh = reinterpret_cast<__half2 *>(xf + ((mi * 2u + 0u) * 4u + t) * 4u);
        __half2 *dl = reinterpret_cast<__half2 *>(xf + ((mi * 2u + 1u) * 4u + t) * 4u);
        dh[0] = __halves2half2(h[0], h[2]); dh[1] = __halves2half2(h[1], h[3]);
        dl[0] = __halves2half2(l[0], l[2]); dl[1] = __halves2half2(l[1], l[3]);
    }
    float s = (v[0] + v[1]) + (v[2] + v[3]);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (live && t == 0) reinterpret_cast<float *>(row + (size_t)cols * 4u)[mi] = s;
}

__device__ __forceinline__ void pack_store_unscale(uint8_t *row, uint32_t cols, float scale) {
    *reinterpret_cast<float *>(row + (size_t)cols * 4u + cols / 4u) = 1.0f / scale;
}

}  // namespace ingot
