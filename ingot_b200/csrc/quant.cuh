// GGUF block formats of the decode path: geometry, the scalar decoder that
// defines "the dequantised weight", and the per-lane unit decoders the GEMV
// kernels are built from.
//
// Everything here is __host__ __device__ so that the lane arithmetic can be
// run on a CPU (tests/host_emulation.cpp) exactly as the kernels run it.
//
// Formats (GGML type ids, block elements, block bytes — the reference's
// geometry(): src/gguf.rs:470-491):
//   0 F32 (1,4)  1 F16 (1,2)  30 BF16 (1,2)
//   2 Q4_0 (32,18)  8 Q8_0 (32,34)  12 Q4_K (256,144)  14 Q6_K (256,210)
#pragma once
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#include <cuda_fp16.h>
#define IG_HD __host__ __device__ __forceinline__
#else
#include <math.h>
#define IG_HD inline
#endif

namespace ingot {

enum : uint32_t {
    KIND_F32 = 0, KIND_F16 = 1, KIND_Q4_0 = 2, KIND_Q8_0 = 8,
    KIND_Q4_K = 12, KIND_Q6_K = 14, KIND_BF16 = 30
};

// (block elements, block bytes); false for a type outside this path.
IG_HD bool geometry(uint32_t kind, uint32_t &block, uint32_t &bytes) {
    switch (kind) {
    case KIND_F32: block = 1; bytes = 4; return true;
    case KIND_F16: case KIND_BF16: block = 1; bytes = 2; return true;
    case KIND_Q4_0: block = 32; bytes = 18; return true;
    case KIND_Q8_0: block = 32; bytes = 34; return true;
    case KIND_Q4_K: block = 256; bytes = 144; return true;
    case KIND_Q6_K: block = 256; bytes = 210; return true;
    default: return false;
    }
}

IG_HD float bits_to_float(uint32_t b) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(b);
#else
    float f; memcpy(&f, &b, 4); return f;
#endif
}

// binary16 bit pattern -> float, exact (reference half_at: kernels/moe.metal:6-9).
IG_HD float half_bits_to_float(uint32_t h) {
#if defined(__CUDA_ARCH__)
    return __half2float(__ushort_as_half((unsigned short)h));
#else
    uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
    else bits = sign | ((exp + 112u) << 23) | (man << 13);
    return bits_to_float(bits);
#endif
}

IG_HD float bf16_bits_to_float(uint32_t b) { return bits_to_float(b << 16); }

IG_HD uint32_t rd16(const uint8_t *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8); }

IG_HD float fma_rn(float a, float b, float c) {
#if defined(__CUDA_ARCH__)
    return __fmaf_rn(a, b, c);
#else
    return fmaf(a, b, c);
#endif
}
IG_HD float mul_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fmul_rn(a, b);
#else
    return a * b;
#endif
}
IG_HD float sub_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fsub_rn(a, b);
#else
    return a - b;
#endif
}
IG_HD float add_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fadd_rn(a, b);
#else
    return a + b;
#endif
}

// Right funnel shift of the 64-bit value hi:lo by `s` in [0,32].
IG_HD uint32_t funnel_r(uint32_t lo, uint32_t hi, uint32_t s) {
#if defined(__CUDA_ARCH__)
    return __funnelshift_rc(lo, hi, s);
#else
    return s >= 32 ? hi : (s == 0 ? lo : ((lo >> s) | (hi << (32 - s))));
#endif
}

// Six-bit (scale, min) of sub-block g of a Q4_K block's 12 scale bytes
// (reference kquant_scale_min: kernels/iq3_mix.metal:13-15).
IG_HD void q4k_scale_min(const uint8_t *s, uint32_t g, uint32_t &sc, uint32_t &m) {
    if (g < 4) { sc = s[g] & 63u; m = s[g + 4] & 63u; }
    else {
        sc = (s[g + 4] & 15u) | ((uint32_t)(s[g - 4] >> 6) << 4);
        m = (uint32_t)(s[g + 4] >> 4) | ((uint32_t)(s[g] >> 6) << 4);
    }
}

// Element j of a row, the definition of the dequantised weight
// (reference weight_at: kernels/moe.metal:11-28,47-50; mix_weight_at:
// kernels/iq3_mix.metal:17-24).  Each product is rounded separately in fp32 in
// the order the shader writes it; NaN for a kind outside this path.
IG_HD float weight_at(const uint8_t *row, uint32_t kind, uint32_t j) {
    switch (kind) {
    case KIND_F32: {
        const uint8_t *p = row + 4u * j;
        return bits_to_float((uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) |
                             ((uint32_t)p[3] << 24));
    }
    case KIND_F16: return half_bits_to_float(rd16(row + 2u * j));
    case KIND_BF16: return bf16_bits_to_float(rd16(row + 2u * j));
    case KIND_Q4_0: {
        const uint8_t *b = row + (j / 32u) * 18u;
        uint32_t k = j % 32u;
        int q = (int)((b[2 + k % 16u] >> (4u * (k / 16u))) & 15u) - 8;
        return mul_rn(half_bits_to_float(rd16(b)), (float)q);
    }
    case KIND_Q8_0: {
        const uint8_t *b = row + (j / 32u) * 34u;
        return mul_rn(half_bits_to_float(rd16(b)), (float)(int8_t)b[2 + j % 32u]);
    }
    case KIND_Q4_K: {
        const uint8_t *b = row + (j / 256u) * 144u;
        uint32_t k = j % 256u, g = k / 32u, sc, m;
        q4k_scale_min(b + 4, g, sc, m);
        uint32_t q = (b[16u + 32u * (k / 64u) + k % 32u] >> (4u * (g % 2u))) & 15u;
        float a = mul_rn(mul_rn(half_bits_to_float(rd16(b)), (float)sc), (float)q);
        float c = mul_rn(half_bits_to_float(rd16(b + 2)), (float)m);
        return sub_rn(a, c);
    }
    case KIND_Q6_K: {
        const uint8_t *b = row + (j / 256u) * 210u;
        uint32_t k = j % 256u, n = k / 128u, l = k % 32u, t = (k % 128u) / 32u;
        uint32_t low = (b[n * 64u + l + (t % 2u) * 32u] >> (t >= 2u ? 4u : 0u)) & 15u;
        uint32_t high = (b[128u + n * 32u + l] >> (2u * t)) & 3u;
        int scale = (int8_t)b[192u + n * 8u + l / 16u + 2u * t];
        float ds = mul_rn(half_bits_to_float(rd16(b + 208)), (float)scale);
        return mul_rn(ds, (float)((int)(low | (high << 4)) - 32));
    }
    default: return bits_to_float(0x7fc00000u);
    }
}

// ---------------------------------------------------------------------------
// Per-lane units.
//
// A GEMV lane works on "units" of 32 consecutive-ish weights of one row and
// the matching 32 activations (eight float4 per token).  For every format:
//   UNITS_PER_BLOCK       units in one quant block
//   BLOCK_BYTES/BLOCK_W   block geometry
//   col(u, i)             first column of float4 `i` (0..7) of unit `u`
//   struct Aux            per-token sums of the unit's activations that the
//                         factored arithmetic needs (shared by all rows)
//   aux(x)                builds Aux from the eight float4
//   dot(chunk, u, x, aux) sum over the unit of weight * activation for ONE
//                         row and ONE token; `chunk` points at the row's first
//                         block held in (shared) memory, aligned to 16 bytes,
//                         and `u` counts units from that block.
// The factorisations are the algebraic forms the reference's vector kernels
// use (d*(sc*sum q x) - dmin*(m*sum x): kernels/iq3_mix.metal:104-123;
// d*sum sc*(sum x (q-32)): kernels/decode.metal:66-83; d*(sum q x - 8 sum x):
// kernels/generic.metal:242-269), so results agree with the f64 expectation
// to rounding, not bit for bit.
// ---------------------------------------------------------------------------

struct alignas(16) F4 { float x, y, z, w; };
struct alignas(16) U4 { uint32_t x, y, z, w; };

// Activation float4s are stored PERMUTED as (e0, e2, e1, e3): a 32-bit word of
// quants holds bytes 0..3, and the decoders below turn bytes (0,2) and (1,3)
// into pairs of floats, so (.x,.y) and (.z,.w) are the matching activation pairs.
IG_HD F4 permute_x(float e0, float e1, float e2, float e3) { F4 v = {e0, e2, e1, e3}; return v; }

IG_HD float byte_f(uint32_t w, int i) { return (float)((w >> (8 * i)) & 0xffu); }
IG_HD float sum4(const F4 &v) { return add_rn(add_rn(v.x, v.y), add_rn(v.z, v.w)); }

// Integer -> float without the conversion pipe.  `h2` holds two binary16
// "magic" numbers 0x6400 | v (= 1024 + v for v < 1024); adding `bias` in fp32
// gives the two integers (times whatever power of two v carries) exactly.
// On sm_100 this is one mixed-precision add per value.
IG_HD void halves_plus(uint32_t h2, float bias, float &lo, float &hi) {
#if defined(__CUDA_ARCH__)
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tadd.f32.f16 %0, l, %3;\n\tadd.f32.f16 %1, h, %3;\n\t}"
        : "=f"(lo), "=f"(hi)
        : "r"(h2), "f"(bias));
#else
    lo = half_bits_to_float(h2 & 0xffffu) + bias;
    hi = half_bits_to_float(h2 >> 16) + bias;
#endif
}

// Two independent fused multiply-adds, (ax, ay) += (px, py) * (qx, qy); one
// packed fma.rn.f32x2 on sm_100.
IG_HD void fma2(float &ax, float &ay, float px, float py, float qx, float qy) {
#if defined(__CUDA_ARCH__)
    asm("{\n\t.reg .b64 a, b, c;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %5};\n\tmov.b64 c, {%0, %1};\n\t"
        "fma.rn.f32x2 c, a, b, c;\n\tmov.b64 {%0, %1}, c;\n\t}"
        : "+f"(ax), "+f"(ay)
        : "f"(px), "f"(py), "f"(qx), "f"(qy));
#else
    ax = fmaf(px, qx, ax);
    ay = fmaf(py, qy, ay);
#endif
}

static constexpr uint32_t MAGIC_H2 = 0x64006400u;   // two binary16 1024.0

// (a0,a1) += low nibbles of the 4 bytes of `w` times xa; (b0,b1) += 16 * high
// nibbles times xb.  xa/xb are permuted float4s.
IG_HD void dot_nibbles(uint32_t w, const F4 &xa, const F4 &xb, float &a0, float &a1, float &b0, float &b1) {
    const uint32_t s = w >> 8;
    float f0, f1, f2, f3;
    halves_plus((w & 0x000f000fu) | MAGIC_H2, -1024.0f, f0, f2);      // bytes 0, 2
    halves_plus((s & 0x000f000fu) | MAGIC_H2, -1024.0f, f1, f3);      // bytes 1, 3
    fma2(a0, a1, f0, f2, xa.x, xa.y);
    fma2(a0, a1, f1, f3, xa.z, xa.w);
    halves_plus((w & 0x00f000f0u) | MAGIC_H2, -1024.0f, f0, f2);      // 16 * high nibble
    halves_plus((s & 0x00f000f0u) | MAGIC_H2, -1024.0f, f1, f3);
    fma2(b0, b1, f0, f2, xb.x, xb.y);
    fma2(b0, b1, f1, f3, xb.z, xb.w);
}

template <uint32_t KIND> struct Unit;

// ---- Q4_K: unit = 16 bytes of qs = 16 low nibbles (sub-block 2j) and 16 high
// nibbles (sub-block 2j+1) -------------------------------------------------
template <> struct Unit<KIND_Q4_K> {
    static constexpr int UNITS_PER_BLOCK = 8, BLOCK_BYTES = 144, BLOCK_W = 256;
    struct Aux { float sa, sb; };
    static IG_HD uint32_t col(uint32_t u, uint32_t i) {
        uint32_t blk = u >> 3, p = u & 7u;
        return blk * 256u + (p >> 1) * 64u + (p & 1u) * 16u + (i >> 2) * 32u + (i & 3u) * 4u;
    }
    // inverse of col(): unit and float4 slot holding column `c` (multiple of 4)
    static IG_HD void locate(uint32_t c, uint32_t &u, uint32_t &i) {
        uint32_t blk = c >> 8, r = c & 255u, j = r >> 6, rr = r & 63u;
        u = blk * 8u + j * 2u + ((rr & 31u) >> 4);
        i = (rr >> 5) * 4u + ((rr & 15u) >> 2);
    }
    static IG_HD Aux aux(const F4 *x) {
        Aux a;
        a.sa = add_rn(add_rn(sum4(x[0]), sum4(x[1])), add_rn(sum4(x[2]), sum4(x[3])));
        a.sb = add_rn(add_rn(sum4(x[4]), sum4(x[5])), add_rn(sum4(x[6]), sum4(x[7])));
        return a;
    }
    // Decoded once per row, used for every token.  dsc1 carries the 1/16 that
    // undoes the in-place high nibbles.
    struct W { uint32_t q[4]; float dsc0, dsc1, dm0, dm1; };
    static IG_HD W load(const uint8_t *chunk, uint32_t u) {
        const uint8_t *b = chunk + (u >> 3) * 144u;
        uint32_t p = u & 7u, j = p >> 1;
        const U4 hdr = *reinterpret_cast<const U4 *>(b);              // 16-byte aligned
        const U4 qs = *reinterpret_cast<const U4 *>(b + 16u + 16u * p);
        W w;
        w.q[0] = qs.x; w.q[1] = qs.y; w.q[2] = qs.z; w.q[3] = qs.w;
        uint32_t h0 = hdr.x, sh = (j & 1u) * 16u;
        uint32_t a = (hdr.y >> sh) & 0xffffu, bb = (hdr.z >> sh) & 0xffffu,
                 c = (hdr.w >> sh) & 0xffffu;
        uint32_t sc, m;
        if (j < 2) { sc = a & 0x3f3fu; m = bb & 0x3f3fu; }
        else {
            sc = (c & 0x0f0fu) | ((a >> 2) & 0x3030u);
            m = ((c >> 4) & 0x0f0fu) | ((bb >> 2) & 0x3030u);
        }
        float d = half_bits_to_float(h0 & 0xffffu), dmin = half_bits_to_float(h0 >> 16);
        float s0, s1, m0, m1;
        halves_plus(((sc & 0xffu) | ((sc & 0xff00u) << 8)) | MAGIC_H2, -1024.0f, s0, s1);
        halves_plus(((m & 0xffu) | ((m & 0xff00u) << 8)) | MAGIC_H2, -1024.0f, m0, m1);
        w.dsc0 = mul_rn(d, s0);
        w.dsc1 = mul_rn(mul_rn(d, s1), 0.0625f);
        w.dm0 = mul_rn(dmin, m0);
        w.dm1 = mul_rn(dmin, m1);
        return w;
    }
    static IG_HD float dot(const W &w, const F4 *x, const Aux &ax) {
        float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) dot_nibbles(w.q[i], x[i], x[4 + i], a0, a1, b0, b1);
        float pos = fma_rn(w.dsc1, add_rn(b0, b1), mul_rn(w.dsc0, add_rn(a0, a1)));
        float neg = fma_rn(w.dm1, ax.sb, mul_rn(w.dm0, ax.sa));
        return sub_rn(pos, neg);
    }
};

// ---- Q4_0: unit = one 18-byte block (2-byte aligned) -----------------------
template <> struct Unit<KIND_Q4_0> {
    static constexpr int UNITS_PER_BLOCK = 1, BLOCK_BYTES = 18, BLOCK_W = 32;
    struct Aux { float s; };
    static IG_HD uint32_t col(uint32_t u, uint32_t i) { return u * 32u + i * 4u; }
    static IG_HD void locate(uint32_t c, uint32_t &u, uint32_t &i) { u = c >> 5; i = (c & 31u) >> 2; }
    static IG_HD Aux aux(const F4 *x) {
        Aux a;
        a.s = add_rn(add_rn(add_rn(sum4(x[0]), sum4(x[1])), add_rn(sum4(x[2]), sum4(x[3]))),
                     add_rn(add_rn(sum4(x[4]), sum4(x[5])), add_rn(sum4(x[6]), sum4(x[7]))));
        return a;
    }
    struct W { uint32_t q[4]; float d; };
    static IG_HD W load(const uint8_t *chunk, uint32_t u) {
        uint32_t off = u * 18u, sh = (off & 2u) * 8u;           // 0 or 16
        const uint32_t *p = reinterpret_cast<const uint32_t *>(chunk + (off & ~3u));
        uint32_t w0 = p[0], w1 = p[1], w2 = p[2], w3 = p[3], w4 = p[4];
        W w;
        w.d = half_bits_to_float((w0 >> sh) & 0xffffu);
        w.q[0] = funnel_r(w0, w1, 16u + sh);
        w.q[1] = funnel_r(w1, w2, 16u + sh);
        w.q[2] = funnel_r(w2, w3, 16u + sh);
        w.q[3] = funnel_r(w3, w4, 16u + sh);
        return w;
    }
    static IG_HD float dot(const W &w, const F4 *x, const Aux &ax) {
        float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) dot_nibbles(w.q[i], x[i], x[4 + i], a0, a1, b0, b1);
        float sum = fma_rn(add_rn(b0, b1), 0.0625f, add_rn(a0, a1));
        return mul_rn(w.d, fma_rn(-8.0f, ax.s, sum));
    }
};

// ---- Q8_0: unit = one 34-byte block (2-byte aligned) -----------------------
template <> struct Unit<KIND_Q8_0> {
    static constexpr int UNITS_PER_BLOCK = 1, BLOCK_BYTES = 34, BLOCK_W = 32;
    struct Aux { float unused; };
    static IG_HD uint32_t col(uint32_t u, uint32_t i) { return u * 32u + i * 4u; }
    static IG_HD void locate(uint32_t c, uint32_t &u, uint32_t &i) { u = c >> 5; i = (c & 31u) >> 2; }
    static IG_HD Aux aux(const F4 *) { Aux a; a.unused = 0.f; return a; }
    struct W { uint32_t q[8]; float d; };
    static IG_HD W load(const uint8_t *chunk, uint32_t u) {
        uint32_t off = u * 34u, sh = (off & 2u) * 8u;
        const uint32_t *p = reinterpret_cast<const uint32_t *>(chunk + (off & ~3u));
        uint32_t v[9];
#pragma unroll
        for (int i = 0; i < 9; ++i) v[i] = p[i];
        W w;
        w.d = half_bits_to_float((v[0] >> sh) & 0xffffu);
#pragma unroll
        for (int i = 0; i < 8; ++i) w.q[i] = funnel_r(v[i], v[i + 1], 16u + sh);
        return w;
    }
    static IG_HD float dot(const W &w, const F4 *x, const Aux &) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            // signed byte b -> 1024 + (b ^ 0x80) = 1152 + b
            float f0, f1, f2, f3;
            halves_plus((w.q[i] & 0x00ff00ffu) ^ 0x64806480u, -1152.0f, f0, f2);
            halves_plus(((w.q[i] >> 8) & 0x00ff00ffu) ^ 0x64806480u, -1152.0f, f1, f3);
            fma2(a0, a1, f0, f2, x[i].x, x[i].y);
            fma2(a0, a1, f1, f3, x[i].z, x[i].w);
        }
        return mul_rn(w.d, add_rn(a0, a1));
    }
};

// ---- Q6_K: unit = 8 consecutive l of one 128-half: 8 bytes of ql (low),
// 8 bytes of ql+32 and 8 bytes of qh, giving 4 quarters t of 8 weights -------
template <> struct Unit<KIND_Q6_K> {
    static constexpr int UNITS_PER_BLOCK = 8, BLOCK_BYTES = 210, BLOCK_W = 256;
    struct Aux { float s[4]; };
    static IG_HD uint32_t col(uint32_t u, uint32_t i) {
        uint32_t blk = u >> 3, r = u & 7u;
        return blk * 256u + (r >> 2) * 128u + (i >> 1) * 32u + (r & 3u) * 8u + (i & 1u) * 4u;
    }
    static IG_HD void locate(uint32_t c, uint32_t &u, uint32_t &i) {
        uint32_t blk = c >> 8, r = c & 255u, n = r >> 7, rr = r & 127u, t = rr >> 5, l = rr & 31u;
        u = blk * 8u + n * 4u + (l >> 3);
        i = t * 2u + ((l & 7u) >> 2);
    }
    static IG_HD Aux aux(const F4 *x) {
        Aux a;
#pragma unroll
        for (int t = 0; t < 4; ++t) a.s[t] = add_rn(sum4(x[2 * t]), sum4(x[2 * t + 1]));
        return a;
    }
    // ds[t] = d * scale_t, times 1/16 for the quarters decoded from high nibbles
    struct W { uint32_t l0[2], l1[2], h[2]; float ds[4]; };
    // two consecutive 32-bit words starting at byte `off` (2-byte aligned) of chunk
    static IG_HD void ld64(const uint8_t *chunk, uint32_t off, uint32_t *out) {
        uint32_t sh = (off & 2u) * 8u;
        const uint32_t *p = reinterpret_cast<const uint32_t *>(chunk + (off & ~3u));
        uint32_t a = p[0], b = p[1], c = p[2];
        out[0] = funnel_r(a, b, sh);
        out[1] = funnel_r(b, c, sh);
    }
    static IG_HD W load(const uint8_t *chunk, uint32_t u) {
        uint32_t base = (u >> 3) * 210u, r = u & 7u, n = r >> 2, k8 = r & 3u;
        W w;
        ld64(chunk, base + 64u * n + 8u * k8, w.l0);
        ld64(chunk, base + 64u * n + 32u + 8u * k8, w.l1);
        ld64(chunk, base + 128u + 32u * n + 8u * k8, w.h);
        uint32_t sc[2];
        ld64(chunk, base + 192u + 8u * n, sc);            // the half's 8 signed scales
        uint32_t doff = base + 208u;
        uint32_t dw = *reinterpret_cast<const uint32_t *>(chunk + (doff & ~3u));
        float d = half_bits_to_float((dw >> ((doff & 2u) * 8u)) & 0xffffu);
        // scale index = (k8 >> 1) + 2t: bytes 0,2,4,6 or 1,3,5,7 of the eight
        uint32_t s0 = sc[0] >> ((k8 >> 1) * 8u), s1 = sc[1] >> ((k8 >> 1) * 8u);
        float f0, f1, f2, f3;
        halves_plus((s0 & 0x00ff00ffu) ^ 0x64806480u, -1152.0f, f0, f1);    // t = 0, 1
        halves_plus((s1 & 0x00ff00ffu) ^ 0x64806480u, -1152.0f, f2, f3);    // t = 2, 3
        w.ds[0] = mul_rn(d, f0);
        w.ds[1] = mul_rn(d, f1);
        w.ds[2] = mul_rn(mul_rn(d, f2), 0.0625f);
        w.ds[3] = mul_rn(mul_rn(d, f3), 0.0625f);
        return w;
    }
    // one quarter t of one word e: 4 six-bit values (x16 when t >= 2) against one permuted float4
    template <int T>
    static IG_HD void quarter(uint32_t L, uint32_t H, const F4 &x, float &a0, float &a1) {
        constexpr uint32_t nib = (T >= 2) ? 0x00f000f0u : 0x000f000fu;
        constexpr uint32_t hmask = 0x00030003u << (2 * T);
        // the two high bits land at bit 4 (t < 2) or bit 8 (t >= 2): shift by 4-2t or 8-2t
        constexpr uint32_t mult = (T == 0 || T == 2) ? 16u : 4u;
        const uint32_t Ls = L >> 8, Hs = H >> 8;
        float f0, f1, f2, f3;
        halves_plus((L & nib) | ((H & hmask) * mult + MAGIC_H2), -1024.0f, f0, f2);     // bytes 0, 2
        halves_plus((Ls & nib) | ((Hs & hmask) * mult + MAGIC_H2), -1024.0f, f1, f3);   // bytes 1, 3
        fma2(a0, a1, f0, f2, x.x, x.y);
        fma2(a0, a1, f1, f3, x.z, x.w);
    }
    static IG_HD float dot(const W &w, const F4 *x, const Aux &ax) {
        float total = 0.f;
        float a0, a1;
#define IG_Q6_QUARTER(T)                                                             \
        a0 = 0.f; a1 = 0.f;                                                          \
        quarter<T>((T & 1) ? w.l1[0] : w.l0[0], w.h[0], x[2 * T], a0, a1);           \
        quarter<T>((T & 1) ? w.l1[1] : w.l0[1], w.h[1], x[2 * T + 1], a0, a1);       \
        total = fma_rn(w.ds[T], fma_rn((T >= 2) ? -512.0f : -32.0f, ax.s[T], add_rn(a0, a1)), total);
        IG_Q6_QUARTER(0) IG_Q6_QUARTER(1) IG_Q6_QUARTER(2) IG_Q6_QUARTER(3)
#undef IG_Q6_QUARTER
        return total;
    }
};

}  // namespace ingot
