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

// ---- fixed-point rows for the int8 mma.sync GEMV ----
// Every sub-block of 32 activations has its own power-of-two scale S: x is held as the integer
// round(x S), split into ND signed base-256 digits (most significant first; 2 digits = 16 bits for
// activations that carry a bfloat16's eight significant bits, 4 digits = 31 bits for float32).  Row:
//   [cols/32 sub-blocks][ND digit planes][32 bytes]     digit d of the sub-block's 32 activations
//   [cols/32 sub-blocks][2 runs of 16]{1/S, sum of the run's quantised activations / S}   (float2)
// = cols * ND + cols / 2 bytes.  An all-zero (or denormal) sub-block has S = 1 and zero digits; a
// sub-block with a non-finite activation stores that value as its 1/S, which makes every result that
// touches it non-finite as well.
// One thread stores four consecutive activations v[0..3] = columns 4j..4j+3.  The eight threads of a
// sub-block (consecutive j, the first a multiple of 8, in one warp) must call this together: the scale
// and the run sums use shuffles among them.
template <int ND>
__device__ __forceinline__ void fx_store(uint8_t *row, uint32_t cols, uint32_t j, const float (&v)[4], bool live) {
    static_assert(ND == 2 || ND == 4, "two or four digits");
    constexpr uint32_t LB = ND == 2 ? 15u : 30u;             // max |x| S lands in [2^(LB-1), 2^LB)
    float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
    const uint32_t e = __float_as_uint(m) >> 23;             // biased exponent (m >= 0); NaN compares through fmaxf as the other operand
    float s = 1.0f, inv = 1.0f;
    if (e >= 32u && e < 255u) {
        uint32_t se = 253u + LB - e;                         // S = 2^(LB - 1 - (e - 127))
        if (ND == 2 && m * __uint_as_float(se << 23) > 32512.0f) --se;      // keep the high digit inside int8 after rounding
        s = __uint_as_float(se << 23);
        inv = __uint_as_float((254u - se) << 23);
    } else if (e == 255u) {
        inv = m;                                             // infinity: poisons the sub-block's results
    }
    bool nan = false;
    float xq[4];
    int xi[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        nan = nan || (v[i] != v[i]);
        xq[i] = rintf(v[i] * s);
        xi[i] = __float2int_rn(xq[i]);
    }
    if (__any_sync(0xffffffffu, nan)) {                      // rare: find the sub-blocks that hold a NaN
        unsigned mask = __ballot_sync(0xffffffffu, nan);
        if ((mask >> ((threadIdx.x & 24u))) & 0xffu) inv = __uint_as_float(0x7fc00000u);
    }
    float rs = (xq[0] + xq[1]) + (xq[2] + xq[3]);
    rs += __shfl_xor_sync(0xffffffffu, rs, 1);
    rs += __shfl_xor_sync(0xffffffffu, rs, 2);
    uint32_t w[ND];
#pragma unroll
    for (int d = 0; d < ND; ++d) w[d] = 0u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int r = xi[i];
#pragma unroll
        for (int d = ND - 1; d >= 0; --d) {
            w[d] |= (uint32_t)(r & 0xff) << (8 * i);
            r = (r + 128) >> 8;
        }
    }
    if (live) {
        const uint32_t sb = j >> 3, jj = j & 7u;
        uint8_t *dst = row + (size_t)sb * (ND * 32u) + 4u * jj;
#pragma unroll
        for (int d = 0; d < ND; ++d) *reinterpret_cast<uint32_t *>(dst + 32 * d) = w[d];
        if ((jj & 3u) == 0u)
            *reinterpret_cast<float2 *>(row + (size_t)cols * ND + (size_t)sb * 16u + (jj >> 2) * 8u) = make_float2(inv, rs * inv);
    }
}

// The norm's last step and fx_store for one thread's four columns, as ONE copy of code that a row's
// unrolled loop calls: x = v * inv * w (w may be null), rounded to bfloat16 when `round_bf16`.  The
// packing code of a row runs once per projection; inlined into every iteration of an unrolled loop it
// is kilobytes of straight-line code that the instruction cache has to fetch each time, which costs
// more than the arithmetic.  All 32 lanes of a warp call it together.
template <int ND>
__device__ __noinline__ void fx_norm_store(uint8_t *row, uint32_t cols, uint32_t j, float4 v, float inv, const float *nw, uint32_t round_bf16,
                                           bool live) {
    float u[4] = {v.x, v.y, v.z, v.w};
    if (live) {
        const float4 wv = nw ? reinterpret_cast<const float4 *>(nw)[j] : make_float4(1.f, 1.f, 1.f, 1.f);
        u[0] = u[0] * inv * wv.x; u[1] = u[1] * inv * wv.y; u[2] = u[2] * inv * wv.z; u[3] = u[3] * inv * wv.w;
        if (round_bf16) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t x = __float_as_uint(u[k]);
                if ((x & 0x7fffffffu) <= 0x7f800000u) x += 0x7fffu + ((x >> 16) & 1u);       // round to nearest even
                u[k] = __uint_as_float(x & 0xffff0000u);
            }
        }
    }
    fx_store<ND>(row, cols, j, u, live);
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
