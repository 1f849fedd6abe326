/*
 * sgref.c -- CPU restatement of the ScrapGpuLibrary reference arithmetic for the quantized
 * MUL_MAT / decode path.  TEST INFRASTRUCTURE ONLY: this file is the checker that the CUDA
 * kernels are compared against; nothing that ships (the CUDA library, the backend plugin,
 * the timed GPU legs of the benchmark) may call into it.
 *
 * Parity status: PINNED.  Every function below is checked (tests/test_oracle_*.py) against
 *   - the hand-built blocks and fp16 bit patterns of the reference's own unit tests
 *     (tests/ref/ref_quant_tests.cpp:23-105,179-223, tests/ref/ref_ops_tests.cpp:586-602,756-772),
 *     committed as tests/golden/ref_known_answers.json, and
 *   - outputs of the unmodified reference compiled from its own sources (oracle/Makefile ->
 *     oracle/_ref/libscrapgpu_ref.so), bit for bit, on seeded inputs (tests/golden/*.npz).
 *
 * Each function cites the reference file:line (paths relative to the reference project) whose
 * arithmetic it restates.  The association of every float expression is kept, and the file is
 * compiled with -ffp-contract=off so that no multiply-add is fused: the reference is built for
 * baseline x86-64 (SSE2, no FMA), and bit-exact dequantization depends on that.
 *
 * Plain C99, no dependencies beyond libm, single-threaded (callers that want more cores split the
 * weight rows over threads: rows are independent and the K order inside a row is untouched).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define SGREF_API __attribute__((visibility("default")))

/* dtype codes = scrapgpu_dtype (include/scrapgpu/tensor.h:10-22) */
enum { SG_F32 = 0, SG_F16 = 1, SG_Q4_0 = 16, SG_Q8_0 = 17, SG_Q4_K = 32, SG_Q6_K = 33 };

/* bytes per block / elements per block (src/tensor/tensor.h:26-52) */
SGREF_API int sgref_type_size(int dtype) {
    switch (dtype) {
        case SG_F32: return 4;
        case SG_F16: return 2;
        case SG_Q4_0: return 18;
        case SG_Q8_0: return 34;
        case SG_Q4_K: return 144;
        case SG_Q6_K: return 210;
        default: return 0;
    }
}

SGREF_API int sgref_block_size(int dtype) {
    switch (dtype) {
        case SG_Q4_0: case SG_Q8_0: return 32;
        case SG_Q4_K: case SG_Q6_K: return 256;
        case SG_F32: case SG_F16: return 1;
        default: return 0;
    }
}

/* ------------------------------------------------------------------------------------------
 * fp16 <-> fp32 (src/core/ref/f16.cpp:8-34 and :36-91)
 * ---------------------------------------------------------------------------------------- */

SGREF_API float sgref_half_to_float(uint16_t h) {
    uint32_t s = (uint32_t)(h >> 15) << 31;
    uint32_t e = (h >> 10) & 31u;
    uint32_t m = h & 1023u;
    uint32_t out;
    if (e == 31u) {
        out = s | 0x7F800000u | (m << 13);
    } else if (e != 0u) {
        out = s | ((e + 112u) << 23) | (m << 13);
    } else if (m == 0u) {
        out = s;
    } else {
        /* subnormal half: shift the leading one up to bit 10, lowering the exponent as we go */
        uint32_t shift = 0;
        while (!(m & 1024u)) { m <<= 1; ++shift; }
        out = s | ((113u - shift) << 23) | ((m & 1023u) << 13);
    }
    float f;
    memcpy(&f, &out, 4);
    return f;
}

/* round to nearest even, overflow to infinity, subnormals kept (f16.cpp:36-91) */
SGREF_API uint16_t sgref_float_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t s = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t a = x & 0x7FFFFFFFu;
    uint32_t e = a >> 23;
    uint32_t frac = a & 0x7FFFFFu;
    if (e == 255u) return (uint16_t)(s | 0x7C00u | (frac ? 0x0200u : 0u));
    if (e > 142u) return (uint16_t)(s | 0x7C00u);
    if (e >= 113u) {
        uint32_t keep = frac >> 13, rest = frac & 0x1FFFu;
        if (rest > 0x1000u || (rest == 0x1000u && (keep & 1u))) ++keep;
        uint32_t he = e - 112u;
        if (keep == 1024u) { keep = 0; ++he; }
        if (he >= 31u) return (uint16_t)(s | 0x7C00u);
        return (uint16_t)(s | (he << 10) | keep);
    }
    if (e < 103u) return (uint16_t)(s | ((e == 102u && frac) ? 1u : 0u));
    uint32_t sig = frac | 0x800000u;
    uint32_t drop = 126u - e;
    uint32_t rest = sig & ((1u << drop) - 1u);
    uint32_t halfway = 1u << (drop - 1u);
    uint32_t keep = sig >> drop;
    if (rest > halfway || (rest == halfway && (keep & 1u))) ++keep;
    if (keep & 1024u) return (uint16_t)(s | 0x0400u);
    return (uint16_t)(s | keep);
}

static inline uint16_t rd16(const uint8_t *p) { uint16_t v; memcpy(&v, p, 2); return v; }
static inline void wr16(uint8_t *p, uint16_t v) { memcpy(p, &v, 2); }

/* ------------------------------------------------------------------------------------------
 * dequantization (src/core/ref/quant.cpp:20-108)
 * ---------------------------------------------------------------------------------------- */

/* 6-bit (scale, min) pair j of a Q4_K super-block header (quant.cpp:20-28) */
static void k4_scale_min(int j, const uint8_t *sc12, int *scale, int *minv) {
    if (j < 4) {
        *scale = sc12[j] & 63;
        *minv = sc12[j + 4] & 63;
    } else {
        *scale = (sc12[j + 4] & 15) | ((sc12[j - 4] >> 6) << 4);
        *minv = (sc12[j + 4] >> 4) | ((sc12[j] >> 6) << 4);
    }
}

/* quant.cpp:30-42 : y = float(nibble - 8) * d */
static void deq_q4_0(const uint8_t *src, int64_t n, float *y) {
    for (int64_t b = 0; b < n / 32; ++b, src += 18, y += 32) {
        float d = sgref_half_to_float(rd16(src));
        for (int j = 0; j < 16; ++j) {
            int byte = src[2 + j];
            y[j] = (float)((byte & 15) - 8) * d;
            y[j + 16] = (float)((byte >> 4) - 8) * d;
        }
    }
}

/* quant.cpp:44-53 : y = float(int8) * d */
static void deq_q8_0(const uint8_t *src, int64_t n, float *y) {
    for (int64_t b = 0; b < n / 32; ++b, src += 34, y += 32) {
        float d = sgref_half_to_float(rd16(src));
        for (int j = 0; j < 32; ++j) y[j] = (float)(int8_t)src[2 + j] * d;
    }
}

/* quant.cpp:55-82 : per pair of 32-wide sub-blocks, d1 = d*sc, m1 = dmin*m, y = d1*q - m1
 * (a multiply then a subtract, never fused) */
static void deq_q4_k(const uint8_t *src, int64_t n, float *y) {
    for (int64_t b = 0; b < n / 256; ++b, src += 144, y += 256) {
        float d = sgref_half_to_float(rd16(src));
        float dmin = sgref_half_to_float(rd16(src + 2));
        const uint8_t *qs = src + 16;
        for (int pair = 0; pair < 4; ++pair, qs += 32) {
            int s0, m0, s1, m1;
            k4_scale_min(2 * pair, src + 4, &s0, &m0);
            k4_scale_min(2 * pair + 1, src + 4, &s1, &m1);
            float dl = d * (float)s0, ml = dmin * (float)m0;
            float dh = d * (float)s1, mh = dmin * (float)m1;
            float *o = y + 64 * pair;
            for (int l = 0; l < 32; ++l) {
                o[l] = dl * (float)(qs[l] & 15) - ml;
                o[l + 32] = dh * (float)(qs[l] >> 4) - mh;
            }
        }
    }
}

/* quant.cpp:84-108 : 6-bit value = low nibble | 2 bits of qh, minus 32; y = (d * sc) * q,
 * evaluated left to right */
static void deq_q6_k(const uint8_t *src, int64_t n, float *y) {
    for (int64_t b = 0; b < n / 256; ++b, src += 210, y += 256) {
        float d = sgref_half_to_float(rd16(src + 208));
        for (int half = 0; half < 2; ++half) {
            const uint8_t *ql = src + 64 * half;
            const uint8_t *qh = src + 128 + 32 * half;
            const int8_t *sc = (const int8_t *)(src + 192 + 8 * half);
            float *o = y + 128 * half;
            for (int l = 0; l < 32; ++l) {
                int g = l / 16;
                int q1 = ((ql[l] & 15) | (((qh[l] >> 0) & 3) << 4)) - 32;
                int q2 = ((ql[l + 32] & 15) | (((qh[l] >> 2) & 3) << 4)) - 32;
                int q3 = ((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                int q4 = ((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                o[l] = d * (float)sc[g] * (float)q1;
                o[l + 32] = d * (float)sc[g + 2] * (float)q2;
                o[l + 64] = d * (float)sc[g + 4] * (float)q3;
                o[l + 96] = d * (float)sc[g + 6] * (float)q4;
            }
        }
    }
}

/* dispatcher (quant.cpp:473-500, C entry :536-538).  Returns 0 ok, 2 invalid, 1 unsupported
 * (the reference's status codes, include/scrapgpu/status.h:10-17). */
SGREF_API int sgref_dequantize(int dtype, const void *src, float *dst, int64_t n) {
    if (!src || !dst || n <= 0) return 2;
    int bs = sgref_block_size(dtype);
    if (bs <= 1) return 1;
    if (n % bs) return 2;
    switch (dtype) {
        case SG_Q4_0: deq_q4_0((const uint8_t *)src, n, dst); return 0;
        case SG_Q8_0: deq_q8_0((const uint8_t *)src, n, dst); return 0;
        case SG_Q4_K: deq_q4_k((const uint8_t *)src, n, dst); return 0;
        case SG_Q6_K: deq_q6_k((const uint8_t *)src, n, dst); return 0;
    }
    return 1;
}

/* ------------------------------------------------------------------------------------------
 * quantization (src/core/ref/quant.cpp:111-469).  Q4_0 / Q8_0 are the simple absmax schemes;
 * Q4_K / Q6_K restate the published ggml k-quant reference algorithms (iterative scale search)
 * that the reference carries.  Host-only input generator: the same bytes feed CPU and GPU.
 * ---------------------------------------------------------------------------------------- */

/* round-half-even through the 1.5*2^23 magic constant (quant.cpp:161-166) */
static inline int near_int(float v) {
    float t = v + 12582912.f;
    int i;
    memcpy(&i, &t, 4);
    return (i & 0x007fffff) - 0x00400000;
}

static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* quant.cpp:111-136 */
static void q_q4_0(const float *x, uint8_t *dst, int64_t n) {
    for (int64_t b = 0; b < n / 32; ++b, x += 32, dst += 18) {
        float amax = 0.f, vmax = 0.f;
        for (int j = 0; j < 32; ++j) {
            float a = fabsf(x[j]);
            if (amax < a) { amax = a; vmax = x[j]; }
        }
        float d = vmax / -8.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        wr16(dst, sgref_float_to_half(d));
        for (int j = 0; j < 16; ++j) {
            float lo = x[j] * id, hi = x[j + 16] * id;
            uint8_t a = (uint8_t)(int8_t)(lo + 8.5f);
            uint8_t c = (uint8_t)(int8_t)(hi + 8.5f);
            if (a > 15) a = 15;
            if (c > 15) c = 15;
            dst[2 + j] = (uint8_t)(a | (c << 4));
        }
    }
}

/* quant.cpp:138-155 */
static void q_q8_0(const float *x, uint8_t *dst, int64_t n) {
    for (int64_t b = 0; b < n / 32; ++b, x += 32, dst += 34) {
        float amax = 0.f;
        for (int j = 0; j < 32; ++j) { float a = fabsf(x[j]); if (a > amax) amax = a; }
        float d = amax / 127.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        wr16(dst, sgref_float_to_half(d));
        for (int j = 0; j < 32; ++j) dst[2 + j] = (uint8_t)(int8_t)lroundf(x[j] * id);
    }
}

#define GROUP_MAX_EPS 1e-15f

/* symmetric scale search used by Q6_K (quant.cpp:168-241); only the call the reference makes
 * is needed: rmse_type = 1 (weights x^2), no external weights */
static float fit_symmetric(int n, int nmax, const float *x, int8_t *L) {
    float vmax = 0, amax = 0;
    for (int i = 0; i < n; ++i) {
        float a = fabsf(x[i]);
        if (a > amax) { amax = a; vmax = x[i]; }
    }
    if (amax < GROUP_MAX_EPS) {
        for (int i = 0; i < n; ++i) L[i] = 0;
        return 0.f;
    }
    float iscale = -(float)nmax / vmax;
    float sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; ++i) {
        int l = clampi(near_int(iscale * x[i]), -nmax, nmax - 1);
        L[i] = (int8_t)(l + nmax);
        float w = x[i] * x[i];
        sumlx += w * x[i] * l;
        suml2 += w * (float)l * (float)l;
    }
    float scale = suml2 ? sumlx / suml2 : 0.0f;
    float best = scale * sumlx;
    for (int is = -9; is <= 9; ++is) {
        if (is == 0) continue;
        iscale = -((float)nmax + 0.1f * (float)is) / vmax;
        sumlx = suml2 = 0;
        for (int i = 0; i < n; ++i) {
            int l = clampi(near_int(iscale * x[i]), -nmax, nmax - 1);
            float w = x[i] * x[i];
            sumlx += w * x[i] * l;
            suml2 += w * (float)l * (float)l;
        }
        if (suml2 > 0 && sumlx * sumlx > best * suml2) {
            for (int i = 0; i < n; ++i) {
                int l = clampi(near_int(iscale * x[i]), -nmax, nmax - 1);
                L[i] = (int8_t)(nmax + l);
            }
            scale = sumlx / suml2;
            best = scale * sumlx;
        }
    }
    return scale;
}

/* affine (scale, min) search used by Q4_K (quant.cpp:243-325), squared-error variant */
static float fit_affine(int n, int nmax, const float *x, const float *w, uint8_t *L, float *neg_min,
                        uint8_t *Ltmp, float rmin, float rdelta, int nstep) {
    float lo = x[0], hi = x[0];
    float sum_w = w[0];
    float sum_x = sum_w * x[0];
    for (int i = 1; i < n; ++i) {
        if (x[i] < lo) lo = x[i];
        if (x[i] > hi) hi = x[i];
        float wi = w[i];
        sum_w += wi;
        sum_x += wi * x[i];
    }
    if (lo > 0) lo = 0;
    if (hi == lo) {
        for (int i = 0; i < n; ++i) L[i] = 0;
        *neg_min = -lo;
        return 0.f;
    }
    float iscale = (float)nmax / (hi - lo);
    float scale = 1 / iscale;
    float best_err = 0;
    for (int i = 0; i < n; ++i) {
        int l = clampi(near_int(iscale * (x[i] - lo)), 0, nmax);
        L[i] = (uint8_t)l;
        float diff = scale * (float)l + lo - x[i];
        diff = diff * diff;
        best_err += w[i] * diff;
    }
    if (nstep < 1) {
        *neg_min = -lo;
        return scale;
    }
    for (int is = 0; is <= nstep; ++is) {
        iscale = (rmin + rdelta * (float)is + (float)nmax) / (hi - lo);
        float sum_l = 0, sum_l2 = 0, sum_xl = 0;
        for (int i = 0; i < n; ++i) {
            int l = clampi(near_int(iscale * (x[i] - lo)), 0, nmax);
            Ltmp[i] = (uint8_t)l;
            float wi = w[i];
            sum_l += wi * (float)l;
            sum_l2 += wi * (float)l * (float)l;
            sum_xl += wi * (float)l * x[i];
        }
        float D = sum_w * sum_l2 - sum_l * sum_l;
        if (D > 0) {
            float s = (sum_w * sum_xl - sum_x * sum_l) / D;
            float m = (sum_l2 * sum_x - sum_l * sum_xl) / D;
            if (m > 0) {
                m = 0;
                s = sum_xl / sum_l2;
            }
            float err = 0;
            for (int i = 0; i < n; ++i) {
                float diff = s * (float)Ltmp[i] + m - x[i];
                diff = diff * diff;
                err += w[i] * diff;
            }
            if (err < best_err) {
                for (int i = 0; i < n; ++i) L[i] = Ltmp[i];
                best_err = err;
                scale = s;
                lo = m;
            }
        }
    }
    *neg_min = -lo;
    return scale;
}

/* quant.cpp:327-402 */
static void q_q4_k(const float *x, uint8_t *dst, int64_t n) {
    uint8_t L[256], Ltmp[32];
    float wts[32], mins[8], scales[8];
    for (int64_t b = 0; b < n / 256; ++b, x += 256, dst += 144) {
        float max_scale = 0, max_min = 0;
        for (int j = 0; j < 8; ++j) {
            const float *xs = x + 32 * j;
            float sum_x2 = 0;
            for (int l = 0; l < 32; ++l) sum_x2 += xs[l] * xs[l];
            float av_x = sqrtf(sum_x2 / 32);
            for (int l = 0; l < 32; ++l) wts[l] = av_x + fabsf(xs[l]);
            scales[j] = fit_affine(32, 15, xs, wts, L + 32 * j, &mins[j], Ltmp, -1.f, 0.1f, 20);
            if (scales[j] > max_scale) max_scale = scales[j];
            if (mins[j] > max_min) max_min = mins[j];
        }
        float inv_scale = max_scale > 0 ? 63.f / max_scale : 0.f;
        float inv_min = max_min > 0 ? 63.f / max_min : 0.f;
        uint8_t *sc = dst + 4;
        memset(sc, 0, 12);
        for (int j = 0; j < 8; ++j) {
            uint8_t ls = (uint8_t)near_int(inv_scale * scales[j]);
            uint8_t lm = (uint8_t)near_int(inv_min * mins[j]);
            if (ls > 63) ls = 63;
            if (lm > 63) lm = 63;
            if (j < 4) {
                sc[j] = ls;
                sc[j + 4] = lm;
            } else {
                sc[j + 4] = (uint8_t)((ls & 15) | ((lm & 15) << 4));
                sc[j - 4] |= (uint8_t)((ls >> 4) << 6);
                sc[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        wr16(dst, sgref_float_to_half(max_scale / 63.f));
        wr16(dst + 2, sgref_float_to_half(max_min / 63.f));
        /* requantize against the rounded header so the stored nibbles match what a reader decodes */
        for (int j = 0; j < 8; ++j) {
            int s, m;
            k4_scale_min(j, sc, &s, &m);
            float d = sgref_half_to_float(rd16(dst)) * (float)s;
            if (d == 0.f) continue;
            float dm = sgref_half_to_float(rd16(dst + 2)) * (float)m;
            for (int i = 0; i < 32; ++i) {
                int l = clampi(near_int((x[32 * j + i] + dm) / d), 0, 15);
                L[32 * j + i] = (uint8_t)l;
            }
        }
        uint8_t *q = dst + 16;
        for (int j = 0; j < 256; j += 64, q += 32)
            for (int l = 0; l < 32; ++l) q[l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 4));
    }
}

/* quant.cpp:404-469 */
static void q_q6_k(const float *x, uint8_t *dst, int64_t n) {
    int8_t L[256];
    float scales[16];
    for (int64_t b = 0; b < n / 256; ++b, x += 256, dst += 210) {
        float max_scale = 0, max_abs = 0;
        for (int g = 0; g < 16; ++g) {
            float s = fit_symmetric(16, 32, x + 16 * g, L + 16 * g);
            scales[g] = s;
            float a = fabsf(s);
            if (a > max_abs) { max_abs = a; max_scale = s; }
        }
        if (max_abs < GROUP_MAX_EPS) {
            memset(dst, 0, 210);
            wr16(dst + 208, sgref_float_to_half(0.f));
            continue;
        }
        float iscale = -128.f / max_scale;
        wr16(dst + 208, sgref_float_to_half(1 / iscale));
        int8_t *sc = (int8_t *)(dst + 192);
        for (int g = 0; g < 16; ++g) {
            int v = near_int(iscale * scales[g]);
            sc[g] = (int8_t)(v < 127 ? v : 127);
        }
        for (int g = 0; g < 16; ++g) {
            float d = sgref_half_to_float(rd16(dst + 208)) * (float)sc[g];
            if (d == 0.f) continue;
            for (int i = 0; i < 16; ++i) {
                int l = clampi(near_int(x[16 * g + i] / d), -32, 31);
                L[16 * g + i] = (int8_t)(l + 32);
            }
        }
        uint8_t *ql = dst, *qh = dst + 128;
        for (int j = 0; j < 256; j += 128, ql += 64, qh += 32) {
            for (int l = 0; l < 32; ++l) {
                uint8_t a = (uint8_t)(L[j + l] & 15), c = (uint8_t)(L[j + l + 32] & 15);
                uint8_t e = (uint8_t)(L[j + l + 64] & 15), g = (uint8_t)(L[j + l + 96] & 15);
                ql[l] = (uint8_t)(a | (e << 4));
                ql[l + 32] = (uint8_t)(c | (g << 4));
                qh[l] = (uint8_t)((L[j + l] >> 4) | ((L[j + l + 32] >> 4) << 2) |
                                  ((L[j + l + 64] >> 4) << 4) | ((L[j + l + 96] >> 4) << 6));
            }
        }
    }
}

/* dispatcher (quant.cpp:502-531, C entry :540-542) */
SGREF_API int sgref_quantize(int dtype, const float *src, void *dst, int64_t n) {
    if (!src || !dst || n <= 0) return 2;
    int bs = sgref_block_size(dtype);
    if (bs <= 1) return 1;
    if (n % bs) return 2;
    switch (dtype) {
        case SG_Q4_0: q_q4_0(src, (uint8_t *)dst, n); return 0;
        case SG_Q8_0: q_q8_0(src, (uint8_t *)dst, n); return 0;
        case SG_Q4_K: q_q4_k(src, (uint8_t *)dst, n); return 0;
        case SG_Q6_K: q_q6_k(src, (uint8_t *)dst, n); return 0;
    }
    return 1;
}

/* rows of a matrix, each row one sgref_quantize (harness convenience) */
SGREF_API int sgref_quantize_rows(int dtype, const float *src, void *dst, int64_t k, int64_t rows) {
    int bs = sgref_block_size(dtype);
    if (bs <= 1 || k <= 0 || k % bs) return 2;
    int64_t rb = k / bs * sgref_type_size(dtype);
    int rc = 0;
    for (int64_t r = 0; r < rows; ++r) {
        int st = sgref_quantize(dtype, src + r * k, (uint8_t *)dst + r * rb, k);
        if (st) rc = st;
    }
    return rc;
}

/* ------------------------------------------------------------------------------------------
 * MUL_MAT (src/core/ref/ops.cpp:891-984): y[n,m] = sum_k W[k,n] * x[k,m], W row dequantized
 * (load_row :258-269), f32 accumulate in increasing k, multiply and add unfused.  The
 * reference's column-panel path for M >= 4 (:863-889) keeps the same per-output order, so
 * one loop restates both.  x is [K, M] with column stride ldx floats, y is [N, M] with ldy.
 * ---------------------------------------------------------------------------------------- */
SGREF_API int sgref_mul_mat(int dtype, const void *w, int64_t k, int64_t n, const float *x, int64_t m,
                            int64_t ldx, float *y, int64_t ldy) {
    int bs = sgref_block_size(dtype);
    if (bs == 0 || k <= 0 || k % bs) return 2;
    int64_t row_bytes = k / bs * sgref_type_size(dtype);
    int rc = 0;
    {
        float *row = (float *)malloc((size_t)k * sizeof(float));
        for (int64_t r = 0; r < n; ++r) {
            const uint8_t *src = (const uint8_t *)w + r * row_bytes;
            if (dtype == SG_F32) {
                memcpy(row, src, (size_t)k * 4);
            } else if (dtype == SG_F16) {
                for (int64_t i = 0; i < k; ++i) row[i] = sgref_half_to_float(rd16(src + 2 * i));
            } else if (sgref_dequantize(dtype, src, row, k)) {
                rc = 1;
            }
            for (int64_t c = 0; c < m; ++c) {
                const float *xc = x + c * ldx;
                float acc = 0.0f;
                for (int64_t i = 0; i < k; ++i) acc += row[i] * xc[i];
                y[c * ldy + r] = acc;
            }
        }
        free(row);
    }
    return rc;
}

/* ------------------------------------------------------------------------------------------
 * RMS_NORM family (ops.cpp:440-519): double sum of squares, scale = 1/sqrtf(float(sum/ne0)+eps),
 * y = (x*scale)*w.  `add` (optional) is the residual of ADD_RMS_NORM_MUL: s = a + b is written
 * to sum_out and normalised.  w may be NULL (plain RMS_NORM).
 * ---------------------------------------------------------------------------------------- */
SGREF_API void sgref_rms_norm(const float *x, const float *add, const float *w, float *sum_out, float *y,
                              int64_t ne0, int64_t rows, float eps) {
    for (int64_t r = 0; r < rows; ++r) {
        const float *xr = x + r * ne0;
        float *yr = y + r * ne0;
        double sum = 0.0;
        for (int64_t i = 0; i < ne0; ++i) {
            float v = add ? xr[i] + add[r * ne0 + i] : xr[i];
            if (sum_out) sum_out[r * ne0 + i] = v;
            sum += (double)v * (double)v;
        }
        float scale = 1.0f / sqrtf((float)(sum / (double)ne0) + eps);
        for (int64_t i = 0; i < ne0; ++i) {
            float v = add ? xr[i] + add[r * ne0 + i] : xr[i];
            float t = v * scale;
            yr[i] = w ? t * w[i] : t;
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * ROPE (ops.cpp:530-634) without yarn (ext_factor = 0) and without frequency factors:
 * theta_scale = powf(base, -2/n_dims); theta = pos multiplied j times by theta_scale;
 * th = freq_scale * theta; rotate pair (NORMAL: 2j,2j+1; NEOX: j, j+n_dims/2) by
 * (cos th * attn_factor, sin th * attn_factor); elements beyond n_dims are copied.
 * x is [ne0, heads, tokens]; positions has `tokens` entries.
 * ---------------------------------------------------------------------------------------- */
SGREF_API void sgref_rope(const float *x, const int32_t *positions, float *y, int64_t ne0, int64_t heads,
                          int64_t tokens, int n_dims, int neox, float freq_base, float freq_scale,
                          float attn_factor) {
    float theta_scale = powf(freq_base, -2.0f / (float)n_dims);
    for (int64_t t = 0; t < tokens; ++t) {
        float position = (float)positions[t];
        for (int64_t h = 0; h < heads; ++h) {
            const float *xr = x + (t * heads + h) * ne0;
            float *yr = y + (t * heads + h) * ne0;
            for (int64_t j = 0; j < ne0 / 2; ++j) {
                if (j < n_dims / 2) {
                    float theta = position;
                    for (int64_t q = 0; q < j; ++q) theta *= theta_scale;
                    float th = freq_scale * (theta / 1.0f);
                    float cs = cosf(th) * attn_factor;
                    float sn = sinf(th) * attn_factor;
                    int64_t e0 = neox ? j : 2 * j;
                    int64_t e1 = neox ? j + n_dims / 2 : 2 * j + 1;
                    float x0 = xr[e0], x1 = xr[e1];
                    yr[e0] = x0 * cs - x1 * sn;
                    yr[e1] = x0 * sn + x1 * cs;
                } else {
                    int64_t e = 2 * (j - n_dims / 2) + n_dims;
                    yr[e] = xr[e];
                    yr[e + 1] = xr[e + 1];
                }
            }
        }
    }
}

/* the (cos, sin) pair the ROPE above multiplies by, for one position and pair index: lets a
 * caller tabulate exactly the values the reference would use */
SGREF_API void sgref_rope_cos_sin(int32_t position, int j, int n_dims, float freq_base, float freq_scale,
                                  float attn_factor, float *cs, float *sn) {
    float theta_scale = powf(freq_base, -2.0f / (float)n_dims);
    float theta = (float)position;
    for (int q = 0; q < j; ++q) theta *= theta_scale;
    float th = freq_scale * (theta / 1.0f);
    *cs = cosf(th) * attn_factor;
    *sn = sinf(th) * attn_factor;
}

/* ------------------------------------------------------------------------------------------
 * SOFT_MAX (ops.cpp:636-684): v = x*scale (+ mask); subtract the row max; expf; sequential f32
 * sum; multiply by 1/sum.  mask may be NULL; rows of length ne0.
 * ---------------------------------------------------------------------------------------- */
SGREF_API void sgref_soft_max(const float *x, const float *mask, float *y, int64_t ne0, int64_t rows,
                              float scale) {
    for (int64_t r = 0; r < rows; ++r) {
        const float *xr = x + r * ne0;
        const float *mr = mask ? mask + r * ne0 : NULL;
        float *yr = y + r * ne0;
        float mx = -INFINITY;
        for (int64_t i = 0; i < ne0; ++i) {
            float v = xr[i] * scale;
            if (mr) v += mr[i];
            mx = fmaxf(mx, v);
        }
        float sum = 0.0f;
        for (int64_t i = 0; i < ne0; ++i) {
            float v = xr[i] * scale;
            if (mr) v += mr[i];
            float e = expf(v - mx);
            yr[i] = e;
            sum += e;
        }
        float inv = 1.0f / sum;
        for (int64_t i = 0; i < ne0; ++i) yr[i] = yr[i] * inv;
    }
}

/* GLU / SwiGLU with split inputs (ops.cpp:383-425): y = (x / (1 + expf(-x))) * g */
SGREF_API void sgref_swiglu(const float *x, const float *g, float *y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) y[i] = (x[i] / (1.0f + expf(-x[i]))) * g[i];
}

/* ADD (ops.cpp:280-312), same shapes */
SGREF_API void sgref_add(const float *a, const float *b, float *y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) y[i] = a[i] + b[i];
}

/* GET_ROWS over a quantized / f32 / f16 table (ops.cpp:690-722): dst row i = dequantized row ids[i] */
SGREF_API int sgref_get_rows(int dtype, const void *table, int64_t k, int64_t table_rows, const int32_t *ids,
                             int64_t n_ids, float *dst) {
    int bs = sgref_block_size(dtype);
    if (bs == 0 || k % bs) return 2;
    int64_t row_bytes = k / bs * sgref_type_size(dtype);
    for (int64_t i = 0; i < n_ids; ++i) {
        if (ids[i] < 0 || ids[i] >= table_rows) return 2;
        const uint8_t *src = (const uint8_t *)table + (int64_t)ids[i] * row_bytes;
        if (dtype == SG_F32) memcpy(dst + i * k, src, (size_t)k * 4);
        else if (dtype == SG_F16) for (int64_t j = 0; j < k; ++j) dst[i * k + j] = sgref_half_to_float(rd16(src + 2 * j));
        else if (sgref_dequantize(dtype, src, dst + i * k, k)) return 1;
    }
    return 0;
}

/* TOP_K with k = 1 (ops.cpp:1189-1228: stable descending sort, so the lowest index wins ties) */
SGREF_API int32_t sgref_argmax(const float *x, int64_t n) {
    int64_t best = 0;
    for (int64_t i = 1; i < n; ++i) if (x[i] > x[best]) best = i;
    return (int32_t)best;
}

/* ------------------------------------------------------------------------------------------
 * Scaled dot product attention as the core composes it (src/core/attention.cpp:558-678,
 * contract include/scrapgpu/attention.h:11-46) for one batch:
 *   scores[k,q] = sum_d K[d,k,hk] * Q[d,q,h]            (MUL_MAT, f32, increasing d)
 *   p = SOFT_MAX(scores * scale + mask), mask = -inf where causal and k > offset + q
 *   columns whose every key is masked are zeroed (:497-516)
 *   out[dv,q,h] = sum_k V[dv,k,hk] * p[k,q]            (MUL_MAT over V^T, increasing k)
 * with hk = h / (Hq / Hkv).  Q [D,Q,Hq], K [D,Kn,Hkv], V [Dv,Kn,Hkv], out [Dv,Q,Hq].
 * ---------------------------------------------------------------------------------------- */
SGREF_API void sgref_attention(const float *Q, const float *K, const float *V, float *out, int64_t D, int64_t Dv,
                               int64_t nq, int64_t nk, int64_t Hq, int64_t Hkv, int causal, int64_t offset,
                               float scale) {
    float *sc = (float *)malloc((size_t)nk * sizeof(float));
    int64_t group = Hq / Hkv;
    for (int64_t h = 0; h < Hq; ++h) {
        int64_t hk = h / group;
        for (int64_t q = 0; q < nq; ++q) {
            const float *qv = Q + (h * nq + q) * D;
            int any_open = 0;
            for (int64_t k = 0; k < nk; ++k) {
                const float *kv = K + (hk * nk + k) * D;
                float acc = 0.0f;
                for (int64_t d = 0; d < D; ++d) acc += kv[d] * qv[d];
                float v = acc * scale;
                if (causal && k > offset + q) v += -INFINITY; else any_open = 1;
                sc[k] = v;
            }
            float *o = out + (h * nq + q) * Dv;
            if (!any_open) {
                for (int64_t d = 0; d < Dv; ++d) o[d] = 0.0f;
                continue;
            }
            float mx = -INFINITY;
            for (int64_t k = 0; k < nk; ++k) mx = fmaxf(mx, sc[k]);
            float sum = 0.0f;
            for (int64_t k = 0; k < nk; ++k) { sc[k] = expf(sc[k] - mx); sum += sc[k]; }
            float inv = 1.0f / sum;
            for (int64_t k = 0; k < nk; ++k) sc[k] = sc[k] * inv;
            for (int64_t d = 0; d < Dv; ++d) {
                float acc = 0.0f;
                for (int64_t k = 0; k < nk; ++k) acc += V[(hk * nk + k) * Dv + d] * sc[k];
                o[d] = acc;
            }
        }
    }
    free(sc);
}
