// Per-dtype "units" of the packed layout: the 16/32-byte piece of quants one thread owns in one
// weight row, how it is loaded, which activations it multiplies, and its fused dequantize-and-dot.
//
// The arithmetic is the reference's dequantization (src/core/ref/quant.cpp:30-108) folded into the dot
// product of MUL_MAT (src/core/ref/ops.cpp:891-984): sum_k (scale * q_k - offset) * x_k is evaluated as
// scale * sum(q_k x_k) - offset * sum(x_k), with f32 accumulation.  Bit-exact element values are the
// business of the dequantize kernels (sm100_ops.cu); here only NMSE <= 1e-6 is required
// (tests/ops/ops_tests.cpp:725 of the reference).
#pragma once

#include "sm100_common.cuh"
#include "sm100_layout.h"

namespace sm100 {

__device__ __forceinline__ uint4 ldg_stream(const void * p) {
    // weights are read exactly once per launch: keep them out of L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t ldg_u32(const void * p) { return __ldg((const uint32_t *) p); }
__device__ __forceinline__ float half_bits_to_float(uint32_t h) { return __half2float(__ushort_as_half((unsigned short) h)); }
__device__ __forceinline__ float byte_f(uint32_t w, int j) { return (float) ((w >> (8 * j)) & 255u); }
__device__ __forceinline__ float sbyte_f(uint32_t w, int j) { return (float) (int) (signed char) ((w >> (8 * j)) & 255u); }

// ---------------------------------------------------------------------------------------------
// Q4_K: unit = 16 quant bytes = 16 low-nibble weights of sub-block 2p and 16 high-nibble weights of
// sub-block 2p+1 (p = pair index); 8 units per 256-weight block.
// ---------------------------------------------------------------------------------------------
struct UnitQ4K {
    static constexpr int DTYPE = DT_Q4_K;
    static constexpr int MAX_THREADS = 512;   // CTA size limit of the streaming kernel (register budget)
    static constexpr int ROWS_IN_FLIGHT = 4;  // weight rows a thread has loads outstanding for
    static constexpr int WEIGHTS = 32;        // weights per unit
    static constexpr int UNITS_PER_BLOCK = 8;
    static constexpr int XSUMS = 2;
    struct Data { uint4 q; uint4 h; };

    __device__ static __forceinline__ void load(const uint8_t * base, const Planes & P, int64_t row, int64_t blocks_per_row, int cu, Data & d) {
        const int64_t t = row * blocks_per_row + (cu >> 3);
        // the unit's 16 quant bytes are four words of the tile-ordered Q plane (one per lane slot t)
        const uint8_t * q0 = base + P.off[0] + q4k_q_offset(P, row, cu >> 3, (cu & 7) * 16);
        const int64_t step = row < (P.n_rows / 16) * 16 ? 16 : 4;
        d.q = make_uint4(ldg_u32(q0), ldg_u32(q0 + step), ldg_u32(q0 + 2 * step), ldg_u32(q0 + 3 * step));
        d.h = __ldg((const uint4 *) (base + P.off[1] + t * 16));
    }
    // element index of the i-th activation this unit multiplies (i < 32: 16 low then 16 high)
    __device__ static __forceinline__ int64_t x_index(int cu, int i) {
        const int b = cu >> 3, s = cu & 7;
        return (int64_t) b * 256 + (s >> 1) * 64 + (s & 1) * 16 + (i & 15) + (i >> 4) * 32;
    }
    // sums[0] = sum of the 16 low activations, sums[1] = sum of the 16 high ones
    __device__ static __forceinline__ int sum_slot(int i) { return i >> 4; }

    __device__ static __forceinline__ float dot(const Data & d, int cu, const float * x, const float * sums) {
        const uint32_t w[4] = {d.q.x, d.q.y, d.q.z, d.q.w};
        float lo = 0.f, hi = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t wl = w[i] & 0x0F0F0F0Fu, wh = (w[i] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                lo = fmaf(byte_f(wl, j), x[4 * i + j], lo);
                hi = fmaf(byte_f(wh, j), x[16 + 4 * i + j], hi);
            }
        }
        const float dd = half_bits_to_float(d.h.x & 0xFFFFu), dmin = half_bits_to_float(d.h.x >> 16);
        // 24-bit field of pair p inside the 96 bits h.y:h.z:h.w
        const int p = (cu & 7) >> 1;
        const uint32_t f = p == 0 ? d.h.y : p == 1 ? __funnelshift_r(d.h.y, d.h.z, 24) : p == 2 ? __funnelshift_r(d.h.z, d.h.w, 16) : (d.h.w >> 8);
        const float s0 = (float) (f & 63u), m0 = (float) ((f >> 6) & 63u), s1 = (float) ((f >> 12) & 63u), m1 = (float) ((f >> 18) & 63u);
        return dd * (s0 * lo + s1 * hi) - dmin * (m0 * sums[0] + m1 * sums[1]);
    }
};

// ---------------------------------------------------------------------------------------------
// Q6_K: unit u = 2h + c of a block = 32 low-nibble bytes + 16 high-bit bytes = 64 weights in four
// groups of 16 (elements 128h + 16c + {0, 32, 64, 96} + i), each group with its own int8 scale.
// ---------------------------------------------------------------------------------------------
struct UnitQ6K {
    static constexpr int DTYPE = DT_Q6_K;
    static constexpr int MAX_THREADS = 256;
    static constexpr int ROWS_IN_FLIGHT = 3;
    static constexpr int WEIGHTS = 64;
    static constexpr int UNITS_PER_BLOCK = 4;
    static constexpr int XSUMS = 4;
    struct Data { uint4 a; uint4 b; uint4 h; uint32_t sc; uint32_t d; };

    __device__ static __forceinline__ void load(const uint8_t * base, const Planes & P, int64_t row, int64_t blocks_per_row, int cu, Data & d) {
        const int64_t t = row * blocks_per_row + (cu >> 2);
        const int u = cu & 3;
        const uint8_t * l = base + P.off[0] + t * 128 + u * 32;
        d.a = ldg_stream(l);
        d.b = ldg_stream(l + 16);
        d.h = ldg_stream(base + P.off[1] + t * 64 + u * 16);
        d.sc = ldg_u32(base + P.off[2] + t * 16 + u * 4);
        d.d = (uint32_t) __ldg((const unsigned short *) (base + P.off[3] + t * 2));
    }
    __device__ static __forceinline__ int64_t x_index(int cu, int i) {
        const int b = cu >> 2, u = cu & 3;
        return (int64_t) b * 256 + (u >> 1) * 128 + (u & 1) * 16 + (i >> 4) * 32 + (i & 15);
    }
    __device__ static __forceinline__ int sum_slot(int i) { return i >> 4; }

    __device__ static __forceinline__ float dot(const Data & d, int cu, const float * x, const float * sums) {
        (void) cu;
        const uint32_t a[4] = {d.a.x, d.a.y, d.a.z, d.a.w}, b[4] = {d.b.x, d.b.y, d.b.z, d.b.w}, h[4] = {d.h.x, d.h.y, d.h.z, d.h.w};
        float g0 = 0.f, g1 = 0.f, g2 = 0.f, g3 = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t v0 = (a[i] & 0x0F0F0F0Fu) | ((h[i] << 4) & 0x30303030u);
            const uint32_t v1 = (b[i] & 0x0F0F0F0Fu) | ((h[i] << 2) & 0x30303030u);
            const uint32_t v2 = ((a[i] >> 4) & 0x0F0F0F0Fu) | (h[i] & 0x30303030u);
            const uint32_t v3 = ((b[i] >> 4) & 0x0F0F0F0Fu) | ((h[i] >> 2) & 0x30303030u);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                g0 = fmaf(byte_f(v0, j), x[4 * i + j], g0);
                g1 = fmaf(byte_f(v1, j), x[16 + 4 * i + j], g1);
                g2 = fmaf(byte_f(v2, j), x[32 + 4 * i + j], g2);
                g3 = fmaf(byte_f(v3, j), x[48 + 4 * i + j], g3);
            }
        }
        const float dd = half_bits_to_float(d.d);
        const float s0 = sbyte_f(d.sc, 0), s1 = sbyte_f(d.sc, 1), s2 = sbyte_f(d.sc, 2), s3 = sbyte_f(d.sc, 3);
        // stored values are q + 32
        return dd * (s0 * (g0 - 32.f * sums[0]) + s1 * (g1 - 32.f * sums[1]) + s2 * (g2 - 32.f * sums[2]) + s3 * (g3 - 32.f * sums[3]));
    }
};

// ---------------------------------------------------------------------------------------------
// Q4_0: unit = one block = 16 quant bytes (low nibble i -> element i, high nibble -> element 16 + i).
// ---------------------------------------------------------------------------------------------
struct UnitQ40 {
    static constexpr int DTYPE = DT_Q4_0;
    static constexpr int MAX_THREADS = 512;
    static constexpr int ROWS_IN_FLIGHT = 4;
    static constexpr int WEIGHTS = 32;
    static constexpr int UNITS_PER_BLOCK = 1;
    static constexpr int XSUMS = 1;
    struct Data { uint4 q; uint32_t d; };

    __device__ static __forceinline__ void load(const uint8_t * base, const Planes & P, int64_t row, int64_t blocks_per_row, int cu, Data & d) {
        const int64_t t = row * blocks_per_row + cu;
        d.q = ldg_stream(base + P.off[0] + t * 16);
        d.d = (uint32_t) __ldg((const unsigned short *) (base + P.off[1] + t * 2));
    }
    __device__ static __forceinline__ int64_t x_index(int cu, int i) { return (int64_t) cu * 32 + i; }
    __device__ static __forceinline__ int sum_slot(int) { return 0; }

    __device__ static __forceinline__ float dot(const Data & d, int cu, const float * x, const float * sums) {
        (void) cu;
        const uint32_t w[4] = {d.q.x, d.q.y, d.q.z, d.q.w};
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t wl = w[i] & 0x0F0F0F0Fu, wh = (w[i] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc = fmaf(byte_f(wl, j), x[4 * i + j], acc);
                acc = fmaf(byte_f(wh, j), x[16 + 4 * i + j], acc);
            }
        }
        return half_bits_to_float(d.d) * (acc - 8.f * sums[0]);
    }
};

// ---------------------------------------------------------------------------------------------
// Q8_0: unit = half a block = 16 int8 quants.
// ---------------------------------------------------------------------------------------------
struct UnitQ80 {
    static constexpr int DTYPE = DT_Q8_0;
    static constexpr int MAX_THREADS = 512;
    static constexpr int ROWS_IN_FLIGHT = 6;
    static constexpr int WEIGHTS = 16;
    static constexpr int UNITS_PER_BLOCK = 2;
    static constexpr int XSUMS = 1;
    struct Data { uint4 q; uint32_t d; };

    __device__ static __forceinline__ void load(const uint8_t * base, const Planes & P, int64_t row, int64_t blocks_per_row, int cu, Data & d) {
        const int64_t t = row * blocks_per_row + (cu >> 1);
        d.q = ldg_stream(base + P.off[0] + t * 32 + (cu & 1) * 16);
        d.d = (uint32_t) __ldg((const unsigned short *) (base + P.off[1] + t * 2));
    }
    __device__ static __forceinline__ int64_t x_index(int cu, int i) { return (int64_t) cu * 16 + i; }
    __device__ static __forceinline__ int sum_slot(int) { return 0; }

    __device__ static __forceinline__ float dot(const Data & d, int cu, const float * x, const float * sums) {
        (void) cu;
        (void) sums;
        const uint32_t w[4] = {d.q.x, d.q.y, d.q.z, d.q.w};
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int j = 0; j < 4; ++j) acc = fmaf(sbyte_f(w[i], j), x[4 * i + j], acc);
        }
        return half_bits_to_float(d.d) * acc;
    }
};

}  // namespace sm100
