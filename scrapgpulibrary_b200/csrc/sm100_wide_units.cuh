// "Wide" units for the M = 1 streaming matvec: the 32-byte run of quants one thread owns in one weight
// row, unpacked without integer->float conversions.
//
// A masked byte b (0..127) is turned into the f32 value 128 + b by one byte permute: PRMT places b in
// bits 16..23 under the exponent byte 0x43, i.e. 0x43000000 | b << 16 = 2^7 * (1 + b / 128).  The constant
// 128 is removed for free by starting each accumulator at -128 * sum(x) instead of 0.  Products then go
// through the packed f32x2 FMA of sm_100 (two weights per instruction), f32 accumulation throughout.
// The arithmetic restates src/core/ref/quant.cpp:30-108 folded into the dot product of
// src/core/ref/ops.cpp:891-984 (reference project paths); NMSE against that reference is ~1e-12.
#pragma once

#include "sm100_quant_units.cuh"

namespace sm100 {

// 128 + byte j of w (w's bytes must be <= 127) as f32
__device__ __forceinline__ float magic_byte(uint32_t w, int j) { return __uint_as_float(__byte_perm(w, 0x43000000u, 0x7044u | (j << 8))); }

__device__ __forceinline__ float2 magic_pair(uint32_t w, int j) { return make_float2(magic_byte(w, j), magic_byte(w, j + 1)); }

// acc += (128 + bytes of w) * x[0..3], two packed FMAs
__device__ __forceinline__ void fma_word(uint32_t w, const float2 * x, float2 & a0, float2 & a1) {
    a0 = __ffma2_rn(magic_pair(w, 0), x[0], a0);
    a1 = __ffma2_rn(magic_pair(w, 2), x[1], a1);
}

__device__ __forceinline__ void ldg_stream32(const void * p, uint4 & a, uint4 & b) {
    // 32 bytes with one 256-bit load, streamed (no L1 allocation, first in line for L2 eviction)
    asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
                 : "l"(p));
}

// f16 bit pattern -> f32 without the conversion unit: shift into the f32 exponent/mantissa fields and
// rescale by 2^112 (exact for normal and subnormal halves; Inf/NaN scales do not occur in valid blocks)
__device__ __forceinline__ float half_bits_fast(uint32_t h) {
    return __uint_as_float(((h & 0x8000u) << 16) | ((h & 0x7FFFu) << 13)) * 5.192296858534828e33f;
}

// small unsigned integer (< 2^23) -> f32 on the FMA pipe
__device__ __forceinline__ float small_uint_to_float(uint32_t v) { return __uint_as_float(v | 0x4B000000u) - 8388608.0f; }

// ---------------------------------------------------------------------------------------------
// Q4_0: 32 bytes = two blocks (low nibble i -> element i, high nibble -> element 16 + i of each block)
// ---------------------------------------------------------------------------------------------
struct WideQ40 {
    static constexpr int DTYPE = DT_Q4_0;
    static constexpr int WEIGHTS = 64;
    static constexpr int UNITS_PER_BLOCK = -2;  // one unit spans two blocks
    static constexpr int XSUMS = 2;
    struct Data { uint4 a, b; uint32_t d; };

    __device__ static __forceinline__ void load(const uint8_t * base, const Planes & P, int64_t row, int64_t bpr, int cu, Data & d) {
        const int64_t t = row * bpr + 2 * cu;
        ldg_stream32(base + P.off[0] + t * 16, d.a, d.b);
        d.d = __ldg((const uint32_t *) (base + P.off[1] + t * 2));
    }
    __device__ static __forceinline__ int64_t x_index(int cu, int g) { return (int64_t) cu * 64 + g * 4; }
    __device__ static __forceinline__ int sum_slot(int g) { return g >> 3; }

    __device__ static __forceinline__ float dot(const Data & d, int, const float2 * x, const float * sums) {
        const uint32_t w[8] = {d.a.x, d.a.y, d.a.z, d.a.w, d.b.x, d.b.y, d.b.z, d.b.w};
        float r = 0.f;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            float2 a0 = make_float2(-136.f * sums[blk], 0.f), a1 = make_float2(0.f, 0.f);  // 128 (magic) + 8 (the format's offset)
            float2 b0 = make_float2(0.f, 0.f), b1 = make_float2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t ww = w[4 * blk + i];
                fma_word(ww & 0x0F0F0F0Fu, x + 16 * blk + 2 * i, a0, a1);
                fma_word((ww >> 4) & 0x0F0F0F0Fu, x + 16 * blk + 8 + 2 * i, b0, b1);
            }
            const float acc = ((a0.x + a0.y) + (a1.x + a1.y)) + ((b0.x + b0.y) + (b1.x + b1.y));
            r = fmaf(half_bits_fast((d.d >> (16 * blk)) & 0xFFFFu), acc, r);
        }
        return r;
    }
};

// ---------------------------------------------------------------------------------------------
// Q8_0: 32 bytes = one block of int8.  q + 128 = 16 * hn + ln with unsigned nibbles hn, ln, so
// sum q x = 16 * sum hn x + sum ln x - 128 sum x: two magic planes per byte.
// ---------------------------------------------------------------------------------------------
struct WideQ80 {
    static constexpr int DTYPE = DT_Q8_0;
    static constexpr int WEIGHTS = 32;
    static constexpr int UNITS_PER_BLOCK = 1;
    static constexpr int XSUMS = 1;
    struct Data { uint4 a, b; uint32_t d; };

    __device__ static __forceinline__ void load(const uint8_t * base, const Planes & P, int64_t row, int64_t bpr, int cu, Data & d) {
        const int64_t t = row * bpr + cu;
        ldg_stream32(base + P.off[0] + t * 32, d.a, d.b);
        d.d = (uint32_t) __ldg((const unsigned short *) (base + P.off[1] + t * 2));
    }
    __device__ static __forceinline__ int64_t x_index(int cu, int g) { return (int64_t) cu * 32 + g * 4; }
    __device__ static __forceinline__ int sum_slot(int) { return 0; }

    __device__ static __forceinline__ float dot(const Data & d, int, const float2 * x, const float * sums) {
        const uint32_t w[8] = {d.a.x, d.a.y, d.a.z, d.a.w, d.b.x, d.b.y, d.b.z, d.b.w};
        // low-nibble plane: starts at -(128 magic + 128 bias) * S; high-nibble plane: -128 magic * S, weighted by 16
        float2 l0 = make_float2(-256.f * sums[0], 0.f), l1 = make_float2(0.f, 0.f);
        float2 h0 = make_float2(-128.f * sums[0], 0.f), h1 = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t u = w[i] ^ 0x80808080u;  // int8 -> biased unsigned
            fma_word(u & 0x0F0F0F0Fu, x + 2 * i, l0, l1);
            fma_word((u >> 4) & 0x0F0F0F0Fu, x + 2 * i, h0, h1);
        }
        const float lo = (l0.x + l0.y) + (l1.x + l1.y), hi = (h0.x + h0.y) + (h1.x + h1.y);
        return half_bits_fast(d.d) * fmaf(16.f, hi, lo);
    }
};

// ---------------------------------------------------------------------------------------------
// Q6_K: unit u = 2h + c of a block: 32 low-nibble bytes + 16 high-bit bytes = four groups of 16 weights
// (elements 128h + 16c + {0, 32, 64, 96} + i), each with its own int8 scale; stored values are q + 32.
// ---------------------------------------------------------------------------------------------
struct WideQ6K {
    static constexpr int DTYPE = DT_Q6_K;
    static constexpr int WEIGHTS = 64;
    static constexpr int UNITS_PER_BLOCK = 4;
    static constexpr int XSUMS = 4;
    struct Data { uint4 a, b, h; uint32_t sc, d; };

    __device__ static __forceinline__ void load(const uint8_t * base, const Planes & P, int64_t row, int64_t bpr, int cu, Data & d) {
        const int64_t t = row * bpr + (cu >> 2);
        const int u = cu & 3;
        ldg_stream32(base + P.off[0] + t * 128 + u * 32, d.a, d.b);
        d.h = ldg_stream(base + P.off[1] + t * 64 + u * 16);
        d.sc = ldg_u32(base + P.off[2] + t * 16 + u * 4);
        d.d = (uint32_t) __ldg((const unsigned short *) (base + P.off[3] + t * 2));
    }
    // float4 group g (0..15): group of 16 weights g >> 2, quarter g & 3
    __device__ static __forceinline__ int64_t x_index(int cu, int g) {
        const int u = cu & 3;
        return (int64_t) (cu >> 2) * 256 + (u >> 1) * 128 + (u & 1) * 16 + (g >> 2) * 32 + (g & 3) * 4;
    }
    __device__ static __forceinline__ int sum_slot(int g) { return g >> 2; }

    __device__ static __forceinline__ float dot(const Data & d, int, const float2 * x, const float * sums) {
        const uint32_t a[4] = {d.a.x, d.a.y, d.a.z, d.a.w}, b[4] = {d.b.x, d.b.y, d.b.z, d.b.w}, h[4] = {d.h.x, d.h.y, d.h.z, d.h.w};
        float2 g0 = make_float2(-160.f * sums[0], 0.f), g1 = make_float2(-160.f * sums[1], 0.f);  // 128 magic + 32 bias
        float2 g2 = make_float2(-160.f * sums[2], 0.f), g3 = make_float2(-160.f * sums[3], 0.f);
        float2 e0 = make_float2(0.f, 0.f), e1 = e0, e2 = e0, e3 = e0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t v0 = (a[i] & 0x0F0F0F0Fu) | ((h[i] << 4) & 0x30303030u);
            const uint32_t v1 = (b[i] & 0x0F0F0F0Fu) | ((h[i] << 2) & 0x30303030u);
            const uint32_t v2 = ((a[i] >> 4) & 0x0F0F0F0Fu) | (h[i] & 0x30303030u);
            const uint32_t v3 = ((b[i] >> 4) & 0x0F0F0F0Fu) | ((h[i] >> 2) & 0x30303030u);
            fma_word(v0, x + 2 * i, g0, e0);
            fma_word(v1, x + 8 + 2 * i, g1, e1);
            fma_word(v2, x + 16 + 2 * i, g2, e2);
            fma_word(v3, x + 24 + 2 * i, g3, e3);
        }
        const float t0 = (g0.x + g0.y) + (e0.x + e0.y), t1 = (g1.x + g1.y) + (e1.x + e1.y);
        const float t2 = (g2.x + g2.y) + (e2.x + e2.y), t3 = (g3.x + g3.y) + (e3.x + e3.y);
        const float s0 = sbyte_f(d.sc, 0), s1 = sbyte_f(d.sc, 1), s2 = sbyte_f(d.sc, 2), s3 = sbyte_f(d.sc, 3);
        return half_bits_fast(d.d) * (s0 * t0 + s1 * t1 + s2 * t2 + s3 * t3);
    }
};

}  // namespace sm100
