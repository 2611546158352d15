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

// ---- base-256 digits for the int8 tensor-core GEMV ----
// Power of two that puts max|x| = mx into [2^21, 2^22) (1 for an all-zero or non-finite row).
__device__ __forceinline__ float digits_scale(float mx) {
    if (!(mx > 0.f) || !(mx < INFINITY)) return 1.0f;
    int e;
    frexpf(mx, &e);
    return ldexpf(1.0f, 22 - e);
}

// One thread stores columns 4q..4q+3 (v already scaled) of the digit image: q = round(v) =
// d0 + 256 d1 + 65536 d2 with digits in [-128, 127]; rows 0..2 of the column's 16-column chunk
// get the digits, rows 3..5 get them again in odd chunks (zero in even ones), rows 6, 7 are zero.
// The four threads of a quad call this together: the chunk sum uses quad shuffles.
__device__ __forceinline__ void digits_store_quad(uint8_t *row, uint32_t cols, uint32_t q, const float (&v)[4], bool live) {
    uint32_t w0 = 0, w1 = 0, w2 = 0;
    int total = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int x = __float2int_rn(v[i]);
        const int r1 = (x + 128) >> 8, r2 = (r1 + 128) >> 8;
        w0 |= (uint32_t)(x & 0xff) << (8 * i);
        w1 |= (uint32_t)(r1 & 0xff) << (8 * i);
        w2 |= (uint32_t)(r2 & 0xff) << (8 * i);
        total += x;
    }
    if (live) {
        const uint32_t chunk = q >> 2;
        uint32_t *dst = reinterpret_cast<uint32_t *>(row + (size_t)chunk * 128u + (q & 3u) * 4u);
        const bool odd = chunk & 1u;
        dst[0] = w0; dst[4] = w1; dst[8] = w2;
        dst[12] = odd ? w0 : 0u; dst[16] = odd ? w1 : 0u; dst[20] = odd ? w2 : 0u;
        dst[24] = 0u; dst[28] = 0u;
    }
    total += __shfl_xor_sync(0xffffffffu, total, 1);
    total += __shfl_xor_sync(0xffffffffu, total, 2);
    if (live && (q & 3u) == 0) reinterpret_cast<float *>(row + (size_t)cols * 8u)[q >> 2] = (float)total;
}

__device__ __forceinline__ void digits_store_unscale(uint8_t *row, uint32_t cols, float scale) {
    *reinterpret_cast<float *>(row + (size_t)cols * 8u + cols / 4u) = 1.0f / scale;
}

// The same without the low part (bfloat16 activations are exact in binary16): [cols/16 MMAs][4 lanes][4 halves],
// then the sums and 1/scale: 2 * cols + cols / 4 + 16 bytes.
__device__ __forceinline__ void pack_hi_store_quad(uint8_t *row, uint32_t cols, uint32_t q, const float (&v)[4], bool live) {
    const uint32_t mi = q >> 2, t = q & 3u;
    if (live) {
        __half2 *dh = reinterpret_cast<__half2 *>(reinterpret_cast<__half *>(row) + (mi * 4u + t) * 4u);
        dh[0] = __halves2half2(__float2half_rn(v[0]), __float2half_rn(v[2]));
        dh[1] = __halves2half2(__float2half_rn(v[1]), __float2half_rn(v[3]));
    }
    float s = (v[0] + v[1]) + (v[2] + v[3]);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (live && t == 0) reinterpret_cast<float *>(row + (size_t)cols * 2u)[mi] = s;
}
__device__ __forceinline__ void pack_hi_store_unscale(uint8_t *row, uint32_t cols, float scale) {
    *reinterpret_cast<float *>(row + (size_t)cols * 2u + cols / 4u) = 1.0f / scale;
}

__device__ __forceinline__ void pack_store_unscale(uint8_t *row, uint32_t cols, float scale) {
    *reinterpret_cast<float *>(row + (size_t)cols * 4u + cols / 4u) = 1.0f / scale;
}

}  // namespace ingot
