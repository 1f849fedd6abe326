// The ops around the matvec in a decode step: bit-exact dequantization (GET_ROWS), RMS_NORM family,
// ROPE, SOFT_MAX, SwiGLU, ADD, SET_ROWS, arg-max.  Each kernel cites the CPU reference whose values it
// reproduces (src/core/ref/ops.cpp, src/core/ref/quant.cpp of the reference project).  Float expressions
// that the reference evaluates as separate multiply / add / subtract use __fmul_rn / __fadd_rn / __fsub_rn
// so that nvcc does not contract them into FMAs: the reference runs on SSE2 without FMA.
#include "sm100_common.cuh"
#include "sm100_layout.h"

namespace sm100 {

// Activation pointers are deliberately NOT __restrict__ / __ldg: kernels are launched with programmatic dependent
// launch, so a kernel may start while the kernel that produces its inputs is still running.  The non-coherent
// read-only path (ld.global.nc) is only valid for data that does not change during the kernel's lifetime, which
// under early launch includes the producer's writes; only weights (constant across the stream) use it.

// ---- dequantization of one element ---------------------------------------------------------------

__device__ __forceinline__ float h2f(const uint8_t * p) {
    return __half2float(__ushort_as_half((unsigned short) ((uint32_t) p[0] | ((uint32_t) p[1] << 8))));
}

// natural block `blk`, element j of the block (src/core/ref/quant.cpp:30-108)
__device__ float dequant_natural(int dtype, const uint8_t * blk, int j) {
    switch (dtype) {
        case DT_Q4_0: {
            const float d = h2f(blk);
            const int b = blk[2 + (j & 15)];
            const int q = j < 16 ? (b & 15) : (b >> 4);
            return __fmul_rn((float) (q - 8), d);
        }
        case DT_Q8_0:
            return __fmul_rn((float) (int) (signed char) blk[2 + j], h2f(blk));
        case DT_Q4_K: {
            const float d = h2f(blk), dmin = h2f(blk + 2);
            const uint8_t * s = blk + 4;
            const int sb = j >> 5;  // sub-block 0..7
            int sc, mn;
            if (sb < 4) {
                sc = s[sb] & 63;
                mn = s[sb + 4] & 63;
            } else {
                sc = (s[sb + 4] & 15) | ((s[sb - 4] >> 6) << 4);
                mn = (s[sb + 4] >> 4) | ((s[sb] >> 6) << 4);
            }
            const int byte = blk[16 + (j >> 6) * 32 + (j & 31)];
            const int q = (j & 32) ? (byte >> 4) : (byte & 15);
            return __fsub_rn(__fmul_rn(__fmul_rn(d, (float) sc), (float) q), __fmul_rn(dmin, (float) mn));
        }
        case DT_Q6_K: {
            const float d = h2f(blk + 208);
            const int h = j >> 7, r = j & 127, grp = r >> 5, l = r & 31;
            const int lbyte = blk[64 * h + (grp & 1) * 32 + l];
            const int lo = (grp & 2) ? (lbyte >> 4) : (lbyte & 15);
            const int hi = (blk[128 + 32 * h + l] >> (2 * grp)) & 3;
            const int q = (lo | (hi << 4)) - 32;
            const int sc = (int) (signed char) blk[192 + 8 * h + (l >> 4) + 2 * grp];
            return __fmul_rn(__fmul_rn(d, (float) sc), (float) q);
        }
    }
    return 0.f;
}

// packed tensor at `base`, block t, element j: gathers the natural block fields from the planes
__device__ float dequant_packed(int dtype, const uint8_t * base, const Planes & P, int64_t t, int j) {
    switch (dtype) {
        case DT_Q4_0: {
            const float d = h2f(base + P.off[1] + t * 2);
            const int b = base[P.off[0] + t * 16 + (j & 15)];
            const int q = j < 16 ? (b & 15) : (b >> 4);
            return __fmul_rn((float) (q - 8), d);
        }
        case DT_Q8_0:
            return __fmul_rn((float) (int) (signed char) base[P.off[0] + t * 32 + j], h2f(base + P.off[1] + t * 2));
        case DT_Q4_K: {
            const uint8_t * h = base + P.off[1] + t * 16;
            const float d = h2f(h), dmin = h2f(h + 2);
            const int sb = j >> 5, p = sb >> 1;
            const uint32_t f = (uint32_t) h[4 + 3 * p] | ((uint32_t) h[5 + 3 * p] << 8) | ((uint32_t) h[6 + 3 * p] << 16);
            const int sc = (f >> ((sb & 1) * 12)) & 63, mn = (f >> ((sb & 1) * 12 + 6)) & 63;
            const int byte = base[P.off[0] + q4k_q_offset(P, t / P.blocks_per_row, t % P.blocks_per_row, (j >> 6) * 32 + (j & 31))];
            const int q = (j & 32) ? (byte >> 4) : (byte & 15);
            return __fsub_rn(__fmul_rn(__fmul_rn(d, (float) sc), (float) q), __fmul_rn(dmin, (float) mn));
        }
        case DT_Q6_K: {
            const float d = h2f(base + P.off[3] + t * 2);
            const int h = j >> 7, r = j & 127, grp = r >> 5, l = r & 31;
            const int c = l >> 4, i = l & 15, u = 2 * h + c;
            const int lbyte = base[P.off[0] + t * 128 + 32 * u + (grp & 1) * 16 + i];
            const int lo = (grp & 2) ? (lbyte >> 4) : (lbyte & 15);
            const int hi = (base[P.off[1] + t * 64 + 16 * u + i] >> (2 * grp)) & 3;
            const int q = (lo | (hi << 4)) - 32;
            const int sc = (int) (signed char) base[P.off[2] + t * 16 + 4 * u + grp];
            return __fmul_rn(__fmul_rn(d, (float) sc), (float) q);
        }
    }
    return 0.f;
}

// GET_ROWS (src/core/ref/ops.cpp:690-722): dst row i = dequantized table row ids[i]; an index outside
// the table leaves the row untouched and raises the error flag
__global__ void get_rows_kernel(int dtype, int layout, const uint8_t * table, Planes P, int64_t row_stride, int64_t k,
                                int64_t table_rows, const int32_t * ids, int64_t n_ids, float * dst,
                                int64_t ld_dst, int * error_flag) {
    pdl_wait();
    pdl_launch_dependents();
    const int be = dtype == DT_Q4_0 || dtype == DT_Q8_0 ? 32 : dtype == DT_Q4_K || dtype == DT_Q6_K ? 256 : 1;
    const int bb = dtype == DT_Q4_0 ? 18 : dtype == DT_Q8_0 ? 34 : dtype == DT_Q4_K ? 144 : dtype == DT_Q6_K ? 210 : dtype == DT_F16 ? 2 : 4;
    const int64_t bpr = k / be;
    for (int64_t i = blockIdx.y; i < n_ids; i += gridDim.y) {
        const int64_t row = ids[i];
        if (row < 0 || row >= table_rows) {
            if (threadIdx.x == 0 && blockIdx.x == 0 && error_flag != nullptr) atomicExch(error_flag, 1);
            continue;
        }
        for (int64_t e = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; e < k; e += (int64_t) gridDim.x * blockDim.x) {
            float v;
            if (dtype == DT_F32) v = *reinterpret_cast<const float *>(table + row * row_stride + e * 4);
            else if (dtype == DT_F16) v = __half2float(*reinterpret_cast<const __half *>(table + row * row_stride + e * 2));
            else if (layout == LAYOUT_PACKED) v = dequant_packed(dtype, table, P, row * bpr + e / be, (int) (e % be));
            else v = dequant_natural(dtype, table + row * row_stride + (e / be) * bb, (int) (e % be));
            dst[i * ld_dst + e] = v;
        }
    }
}

// ---- RMS_NORM / RMS_NORM_MUL / ADD_RMS_NORM_MUL (ops.cpp:440-519) -------------------------------------
// scale = 1 / sqrtf(float(sum_double(v^2) / ne0) + eps);  y = (v * scale) * w.  One CTA per row.
__global__ void __launch_bounds__(256) rms_norm_kernel(const float * x, const float * add, const float * w,
                                                       float * sum_out, float * y, int64_t ne0, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ double red[8];
    __shared__ float s_scale;
    const int64_t row = blockIdx.x;
    const float * xr = x + row * ne0;
    const float * ar = add != nullptr ? add + row * ne0 : nullptr;
    double sum = 0.0;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) {
        float v = xr[i];
        if (ar != nullptr) {
            v = __fadd_rn(v, ar[i]);
            if (sum_out != nullptr) sum_out[row * ne0 + i] = v;
        }
        sum += (double) v * (double) v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int i = 0; i < (int) (blockDim.x >> 5); ++i) t += red[i];
        const float mean = (float) (t / (double) ne0);
        s_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
    }
    __syncthreads();
    const float scale = s_scale;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) {
        float v;
        if (ar != nullptr && sum_out != nullptr) v = sum_out[row * ne0 + i];  // written above by this thread; sum_out may alias x
        else v = ar != nullptr ? __fadd_rn(xr[i], ar[i]) : xr[i];
        const float t = __fmul_rn(v, scale);
        y[row * ne0 + i] = w != nullptr ? __fmul_rn(t, w[i]) : t;
    }
}

// Same values with the row held in registers: every thread owns up to VPT float4 pieces, so the row is read once,
// the loads are independent 16-byte loads, and the second pass needs no memory.  Used when ne0 is a multiple of 4,
// the rows are 16-byte aligned and a row fits 1024 threads x VPT pieces.
template <int VPT>
__global__ void __launch_bounds__(1024) rms_norm_vec_kernel(const float * x, const float * add, const float * w, float * sum_out, float * y,
                                                            int64_t ne0, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ double red[32];
    __shared__ float s_scale;
    const int64_t row = blockIdx.x;
    const int n4 = (int) (ne0 >> 2);
    const float4 * xr = reinterpret_cast<const float4 *>(x + row * ne0);
    const float4 * ar = add != nullptr ? reinterpret_cast<const float4 *>(add + row * ne0) : nullptr;
    float4 v[VPT];
    double sum = 0.0;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (idx < n4) {
            v[i] = xr[idx];
            if (ar != nullptr) {
                const float4 a4 = ar[idx];
                v[i] = make_float4(__fadd_rn(v[i].x, a4.x), __fadd_rn(v[i].y, a4.y), __fadd_rn(v[i].z, a4.z), __fadd_rn(v[i].w, a4.w));
                if (sum_out != nullptr) reinterpret_cast<float4 *>(sum_out + row * ne0)[idx] = v[i];
            }
        }
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i)
        sum += ((double) v[i].x * (double) v[i].x + (double) v[i].y * (double) v[i].y) + ((double) v[i].z * (double) v[i].z + (double) v[i].w * (double) v[i].w);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const int warps = (blockDim.x + 31) >> 5;
    if (warps > 1) {
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
        __syncthreads();
        if (threadIdx.x < 32) {
            double t = threadIdx.x < warps ? red[threadIdx.x] : 0.0;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            if (threadIdx.x == 0) s_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float) (t / (double) ne0), eps)));
        }
        __syncthreads();
    } else if (threadIdx.x == 0) {
        s_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float) (sum / (double) ne0), eps)));
    }
    if (warps == 1) __syncwarp();
    const float scale = *(volatile float *) &s_scale;
    const float4 * wr = reinterpret_cast<const float4 *>(w);
    float4 * yr = reinterpret_cast<float4 *>(y + row * ne0);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < n4) {
            float4 t = make_float4(__fmul_rn(v[i].x, scale), __fmul_rn(v[i].y, scale), __fmul_rn(v[i].z, scale), __fmul_rn(v[i].w, scale));
            if (w != nullptr) {
                const float4 w4 = wr[idx];
                t = make_float4(__fmul_rn(t.x, w4.x), __fmul_rn(t.y, w4.y), __fmul_rn(t.z, w4.z), __fmul_rn(t.w, w4.w));
            }
            yr[idx] = t;
        }
    }
}

// ---- one decode token's head post-processing in one launch -----------------------------------------------
// RMS_NORM_MUL per head of Q and K (optional), ROPE of Q and K from the (cos, sin) table, SET_ROWS_PAIR of K and V
// into the cache (include/scrapgpu/op.h:43-45; ops.cpp:440-519, 530-634, 690-760 of the reference): the values
// of those separate ops, one warp per head.  Q and K are updated in place.
struct HeadPostArgs {
    float * q; float * k; const float * v;
    const float * q_w; const float * k_w;     // norm weights [d] or null (no norm)
    const int32_t * positions;                // one token
    const float * table; int32_t table_first, table_n;
    float * k_cache; float * v_cache;         // [hkv][ctx_rows][d]
    int d, hq, hkv, neox;
    int64_t ctx_rows;
    float eps, theta_scale;
};

__global__ void __launch_bounds__(128) head_post_kernel(HeadPostArgs a) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int task = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (task >= a.hq + 2 * a.hkv) return;
    const int32_t pos = a.positions[0];
    const bool row_ok = pos >= 0 && pos < a.ctx_rows;
    if (task >= a.hq + a.hkv) {   // V head: copy into the cache
        const int h = task - a.hq - a.hkv;
        if (!row_ok) return;
        const float * src = a.v + (int64_t) h * a.d;
        float * dst = a.v_cache + ((int64_t) h * a.ctx_rows + pos) * a.d;
        for (int e = lane; e < a.d; e += 32) dst[e] = src[e];
        return;
    }
    const bool is_k = task >= a.hq;
    const int h = is_k ? task - a.hq : task;
    float * xr = is_k ? a.k + (int64_t) h * a.d : a.q + (int64_t) h * a.d;
    const float * w = is_k ? a.k_w : a.q_w;
    const int hp = a.d / 2;
    // this lane's pairs: j = lane, lane + 32, ...; elements (j, j + d/2) for NEOX, (2j, 2j+1) otherwise
    constexpr int MAXP = 4;   // d <= 256
    float x0[MAXP], x1[MAXP];
    double sum = 0.0;
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
        const int j = lane + 32 * i;
        x0[i] = x1[i] = 0.f;
        if (j < hp) {
            x0[i] = xr[a.neox ? j : 2 * j];
            x1[i] = xr[a.neox ? j + hp : 2 * j + 1];
            sum += (double) x0[i] * (double) x0[i] + (double) x1[i] * (double) x1[i];
        }
    }
    float scale = 1.0f;
    if (w != nullptr) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float) (sum / (double) a.d), a.eps)));
    }
    float * cache = is_k && row_ok ? a.k_cache + ((int64_t) h * a.ctx_rows + pos) * a.d : nullptr;
    const int64_t rel = (int64_t) pos - a.table_first;
    const bool in_table = a.table != nullptr && rel >= 0 && rel < a.table_n;
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
        const int j = lane + 32 * i;
        if (j < hp) {
            const int e0 = a.neox ? j : 2 * j, e1 = a.neox ? j + hp : 2 * j + 1;
            float v0 = x0[i], v1 = x1[i];
            if (w != nullptr) {
                v0 = __fmul_rn(__fmul_rn(v0, scale), w[e0]);
                v1 = __fmul_rn(__fmul_rn(v1, scale), w[e1]);
            }
            float cs, sn;
            if (in_table) {
                const float2 t = *reinterpret_cast<const float2 *>(a.table + (rel * hp + j) * 2);
                cs = t.x;
                sn = t.y;
            } else {
                float theta = (float) pos;
                for (int q = 0; q < j; ++q) theta = __fmul_rn(theta, a.theta_scale);
                cs = cosf(theta);
                sn = sinf(theta);
            }
            const float y0 = __fsub_rn(__fmul_rn(v0, cs), __fmul_rn(v1, sn));
            const float y1 = __fadd_rn(__fmul_rn(v0, sn), __fmul_rn(v1, cs));
            xr[e0] = y0;
            xr[e1] = y1;
            if (cache != nullptr) {
                cache[e0] = y0;
                cache[e1] = y1;
            }
        }
    }
}

// ---- ROPE (ops.cpp:530-634), no yarn, no frequency factors -------------------------------------------
// One thread per rotated pair / copied pair.  With a table the (cos, sin) come from the caller, who
// computed them with the reference's own recipe; positions outside the table, or no table at all, take
// the on-device recipe: theta = pos * theta_scale^j by j sequential f32 multiplies, cosf / sinf.
__global__ void rope_kernel(const float * x, const int32_t * positions, const float * table,
                            int32_t table_first, int32_t table_n, float * y, int64_t ne0, int64_t heads, int64_t tokens,
                            int n_dims, int neox, float theta_scale, float freq_scale, float attn_factor) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t hp = ne0 / 2;
    const int64_t total = tokens * heads * hp;
    for (int64_t idx = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; idx < total; idx += (int64_t) gridDim.x * blockDim.x) {
        const int64_t j = idx % hp;
        const int64_t rowi = idx / hp;  // token * heads + head
        const int64_t t = rowi / heads;
        const float * xr = x + rowi * ne0;
        float * yr = y + rowi * ne0;
        if (j < n_dims / 2) {
            const int32_t pos = positions[t];
            float cs, sn;
            const int64_t rel = (int64_t) pos - table_first;
            if (table != nullptr && rel >= 0 && rel < table_n) {
                const float2 v = *reinterpret_cast<const float2 *>(table + (rel * (n_dims / 2) + j) * 2);
                cs = v.x;
                sn = v.y;
            } else {
                float theta = (float) pos;
                for (int q = 0; q < (int) j; ++q) theta = __fmul_rn(theta, theta_scale);
                const float th = __fmul_rn(freq_scale, theta);
                cs = __fmul_rn(cosf(th), attn_factor);
                sn = __fmul_rn(sinf(th), attn_factor);
            }
            const int64_t e0 = neox ? j : 2 * j;
            const int64_t e1 = neox ? j + n_dims / 2 : 2 * j + 1;
            const float x0 = xr[e0], x1 = xr[e1];
            yr[e0] = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
            yr[e1] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
        } else {
            const int64_t e = 2 * (j - n_dims / 2) + n_dims;
            yr[e] = xr[e];
            yr[e + 1] = xr[e + 1];
        }
    }
}

// ---- SOFT_MAX (ops.cpp:636-684): one CTA per row, in place allowed ----------------------------------
__device__ __forceinline__ float block_reduce(float v, bool is_max, float * red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float u = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, u) : v + u;
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = red[0];
    for (int i = 1; i < (int) (blockDim.x >> 5); ++i) t = is_max ? fmaxf(t, red[i]) : t + red[i];
    return t;
}

__global__ void __launch_bounds__(256) soft_max_kernel(const float * x, const float * mask, int64_t mask_row_stride,
                                                       int64_t mask_rows, float * y, int64_t ne0, float scale) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float red[8];
    const int64_t row = blockIdx.x;
    const float * xr = x + row * ne0;
    const float * mr = mask != nullptr ? mask + (row % mask_rows) * mask_row_stride : nullptr;
    float * yr = y + row * ne0;
    float mx = -INFINITY;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) {
        float v = __fmul_rn(xr[i], scale);
        if (mr != nullptr) v = __fadd_rn(v, mr[i]);
        mx = fmaxf(mx, v);
    }
    mx = block_reduce(mx, true, red);
    float sum = 0.f;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) {
        float v = __fmul_rn(xr[i], scale);
        if (mr != nullptr) v = __fadd_rn(v, mr[i]);
        const float e = expf(v - mx);
        yr[i] = e;
        sum += e;
    }
    sum = block_reduce(sum, false, red);
    const float inv = __fdiv_rn(1.0f, sum);
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) yr[i] = __fmul_rn(yr[i], inv);
}

// ---- elementwise ---------------------------------------------------------------------------------
// SwiGLU with split inputs (ops.cpp:383-425): y = (x / (1 + expf(-x))) * g
__global__ void swiglu_kernel(const float * x, const float * g, float * y, int64_t n) {
    pdl_wait();
    pdl_launch_dependents();
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
        const float v = x[i];
        y[i] = __fmul_rn(__fdiv_rn(v, __fadd_rn(1.0f, expf(-v))), g[i]);
    }
}

// ADD (ops.cpp:280-312), same shapes
__global__ void add_kernel(const float * a, const float * b, float * y, int64_t n) {
    pdl_wait();
    pdl_launch_dependents();
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) y[i] = __fadd_rn(a[i], b[i]);
}

// SET_ROWS F32 -> F32 (ops.cpp:724-762): src [ne0, n_rows, heads], dst [ne0, dst_rows, heads], ids [n_rows]
__global__ void set_rows_kernel(const float * src, const int32_t * ids, float * dst, int64_t ne0,
                                int64_t n_rows, int64_t heads, int64_t dst_rows, int * error_flag) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t total = ne0 * n_rows * heads;
    for (int64_t idx = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; idx < total; idx += (int64_t) gridDim.x * blockDim.x) {
        const int64_t i0 = idx % ne0, i1 = (idx / ne0) % n_rows, i2 = idx / (ne0 * n_rows);
        const int64_t row = ids[i1];
        if (row < 0 || row >= dst_rows) {
            if (error_flag != nullptr) atomicExch(error_flag, 1);
            continue;
        }
        dst[(i2 * dst_rows + row) * ne0 + i0] = src[idx];
    }
}

// TOP_K with k = 1 (ops.cpp:1189-1228): maximum, lowest index on ties.  Single CTA.
__global__ void __launch_bounds__(1024) argmax_kernel(const float * x, int64_t n, int32_t * out) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float sv[32];
    __shared__ int si[32];
    float best;
    int bi;
    argmax_scan(x, n, (int) threadIdx.x, (int) blockDim.x, best, bi);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = blockDim.x >> 5;
        best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (threadIdx.x == 0) out[0] = bi;
    }
}

static unsigned grid_for(int64_t n, int threads) {
    int64_t g = (n + threads - 1) / threads;
    const int64_t cap = (int64_t) sm_count() * 8;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (unsigned) g;
}

}  // namespace sm100

using namespace sm100;

extern "C" {

int sm100_get_rows(sm100_stream_t s, int dtype, int layout, const void * table, int64_t table_row_stride, int64_t k, int64_t table_rows,
                   const int32_t * ids, int64_t n_ids, float * dst, int64_t ld_dst) {
    if (table == nullptr || ids == nullptr || dst == nullptr) return fail(ST_INVALID, "get_rows: null pointer");
    const int be = block_elems(dtype);
    if (be == 0 || dtype == DT_I32) return fail(ST_UNSUPPORTED, "get_rows: unsupported table dtype %d", dtype);
    if (k <= 0 || table_rows <= 0 || n_ids <= 0 || k % be != 0) return fail(ST_INVALID, "get_rows: bad shape");
    if (layout == LAYOUT_PACKED && !is_quant(dtype)) return fail(ST_UNSUPPORTED, "get_rows: only quantized tables have a packed layout");
    Planes P = {};
    if (layout == LAYOUT_PACKED) P = planes_for(dtype, table_rows, k);
    const int64_t row_stride = table_row_stride != 0 && layout != LAYOUT_PACKED ? table_row_stride : k / be * block_bytes(dtype);
    const int threads = 256;
    unsigned gx = (unsigned) ((k + threads - 1) / threads);
    if (gx > 64) gx = 64;
    const unsigned gy = (unsigned) (n_ids < 16384 ? n_ids : 16384);
    return launch(get_rows_kernel, dim3(gx, gy), dim3(threads), 0, (cudaStream_t) s, dtype, layout, (const uint8_t *) table, P, row_stride, k,
                  table_rows, ids, n_ids, dst, ld_dst, (int *) nullptr);
}

int sm100_rms_norm(sm100_stream_t s, const float * x, const float * add, const float * w, float * sum_out, float * y, int64_t ne0,
                   int64_t rows, float eps) {
    if (x == nullptr || y == nullptr) return fail(ST_INVALID, "rms_norm: null pointer");
    if (ne0 <= 0 || rows <= 0 || rows > INT32_MAX) return fail(ST_INVALID, "rms_norm: bad shape");
    const uintptr_t ptrs = (uintptr_t) x | (uintptr_t) y | (uintptr_t) add | (uintptr_t) w | (uintptr_t) sum_out;
    if (ne0 % 4 == 0 && (ptrs & 15) == 0 && ne0 <= 4 * 1024 * 4) {
        const int n4 = (int) (ne0 / 4);
        int threads = n4 < 1024 ? (n4 + 31) / 32 * 32 : 1024;
        // prefer 2 pieces per thread once a row has that many: fewer warps to reduce over
        if (n4 >= 512 && n4 <= 2048) threads = (n4 / 2 + 31) / 32 * 32;
        const int vpt = (n4 + threads - 1) / threads;
        const dim3 grid((unsigned) rows), block((unsigned) threads);
        switch (vpt) {
            case 1: return launch(rms_norm_vec_kernel<1>, grid, block, 0, (cudaStream_t) s, x, add, w, sum_out, y, ne0, eps);
            case 2: return launch(rms_norm_vec_kernel<2>, grid, block, 0, (cudaStream_t) s, x, add, w, sum_out, y, ne0, eps);
            case 3: case 4: return launch(rms_norm_vec_kernel<4>, grid, block, 0, (cudaStream_t) s, x, add, w, sum_out, y, ne0, eps);
        }
    }
    return launch(rms_norm_kernel, dim3((unsigned) rows), dim3(256), 0, (cudaStream_t) s, x, add, w, sum_out, y, ne0, eps);
}

static int rope_common(sm100_stream_t s, const float * x, const int32_t * positions, const float * table, int32_t first, int32_t count,
                       float * y, int64_t ne0, int64_t heads, int64_t tokens, int n_dims, int neox, float freq_base, float freq_scale,
                       float attn_factor) {
    if (x == nullptr || y == nullptr || positions == nullptr) return fail(ST_INVALID, "rope: null pointer");
    if (n_dims <= 0 || n_dims % 2 != 0 || n_dims > ne0 || ne0 % 2 != 0)
        return fail(ST_INVALID, "rope: n_dims must be a positive even number not above ne0 (ne0 even)");
    if (heads <= 0 || tokens <= 0) return fail(ST_INVALID, "rope: bad shape");
    const float theta_scale = powf(freq_base, -2.0f / (float) n_dims);
    const int64_t total = tokens * heads * (ne0 / 2);
    return launch(rope_kernel, dim3(grid_for(total, 256)), dim3(256), 0, (cudaStream_t) s, x, positions, table, first, count, y, ne0, heads,
                  tokens, n_dims, neox, theta_scale, freq_scale, attn_factor);
}

int sm100_rope(sm100_stream_t s, const float * x, const int32_t * positions, const float * table, int32_t table_first_position,
               int32_t table_positions, float * y, int64_t ne0, int64_t heads, int64_t tokens, int n_dims, int neox) {
    if (table == nullptr || table_positions <= 0) return fail(ST_INVALID, "rope: the (cos, sin) table is missing");
    // positions outside the table cannot be served without the frequency parameters
    return rope_common(s, x, positions, table, table_first_position, table_positions, y, ne0, heads, tokens, n_dims, neox, 10000.0f, 1.0f, 1.0f);
}

int sm100_rope_direct(sm100_stream_t s, const float * x, const int32_t * positions, float * y, int64_t ne0, int64_t heads, int64_t tokens,
                      int n_dims, int neox, float freq_base, float freq_scale, float attn_factor) {
    return rope_common(s, x, positions, nullptr, 0, 0, y, ne0, heads, tokens, n_dims, neox, freq_base, freq_scale, attn_factor);
}

int sm100_soft_max(sm100_stream_t s, const float * x, const float * mask, int64_t mask_row_stride, float * y, int64_t ne0, int64_t rows,
                   float scale) {
    if (x == nullptr || y == nullptr) return fail(ST_INVALID, "soft_max: null pointer");
    if (ne0 <= 0 || rows <= 0 || rows > INT32_MAX) return fail(ST_INVALID, "soft_max: bad shape");
    return launch(soft_max_kernel, dim3((unsigned) rows), dim3(256), 0, (cudaStream_t) s, x, mask, mask_row_stride, rows, y, ne0, scale);
}

int sm100_swiglu(sm100_stream_t s, const float * x, const float * g, float * y, int64_t n) {
    if (x == nullptr || g == nullptr || y == nullptr || n <= 0) return fail(ST_INVALID, "swiglu: bad arguments");
    return launch(swiglu_kernel, dim3(grid_for(n, 256)), dim3(256), 0, (cudaStream_t) s, x, g, y, n);
}

int sm100_add(sm100_stream_t s, const float * a, const float * b, float * y, int64_t n) {
    if (a == nullptr || b == nullptr || y == nullptr || n <= 0) return fail(ST_INVALID, "add: bad arguments");
    return launch(add_kernel, dim3(grid_for(n, 256)), dim3(256), 0, (cudaStream_t) s, a, b, y, n);
}

int sm100_set_rows(sm100_stream_t s, const float * src, const int32_t * ids, float * dst, int64_t ne0, int64_t n_rows, int64_t heads,
                   int64_t dst_rows) {
    if (src == nullptr || ids == nullptr || dst == nullptr) return fail(ST_INVALID, "set_rows: null pointer");
    if (ne0 <= 0 || n_rows <= 0 || heads <= 0 || dst_rows <= 0) return fail(ST_INVALID, "set_rows: bad shape");
    return launch(set_rows_kernel, dim3(grid_for(ne0 * n_rows * heads, 256)), dim3(256), 0, (cudaStream_t) s, src, ids, dst, ne0, n_rows, heads,
                  dst_rows, (int *) nullptr);
}

int sm100_head_post(sm100_stream_t s, float * q, float * k, const float * v, const float * q_norm_w, const float * k_norm_w,
                    const int32_t * positions, const float * table, int32_t table_first_position, int32_t table_positions, float * k_cache,
                    float * v_cache, int64_t head_dim, int64_t q_heads, int64_t kv_heads, int64_t cache_rows, float eps, float freq_base,
                    int neox) {
    if (q == nullptr || k == nullptr || v == nullptr || positions == nullptr || k_cache == nullptr || v_cache == nullptr)
        return fail(ST_INVALID, "head_post: null pointer");
    if (head_dim <= 0 || head_dim % 2 != 0 || head_dim > 256) return fail(ST_UNSUPPORTED, "head_post: head_dim must be even and at most 256");
    if (q_heads <= 0 || kv_heads <= 0 || cache_rows <= 0 || q_heads + 2 * kv_heads > (1 << 20)) return fail(ST_INVALID, "head_post: bad shape");
    HeadPostArgs a;
    a.q = q; a.k = k; a.v = v; a.q_w = q_norm_w; a.k_w = k_norm_w; a.positions = positions;
    a.table = table; a.table_first = table_first_position; a.table_n = table != nullptr ? table_positions : 0;
    a.k_cache = k_cache; a.v_cache = v_cache;
    a.d = (int) head_dim; a.hq = (int) q_heads; a.hkv = (int) kv_heads; a.neox = neox; a.ctx_rows = cache_rows;
    a.eps = eps;
    a.theta_scale = powf(freq_base, -2.0f / (float) head_dim);
    const int tasks = (int) (q_heads + 2 * kv_heads);
    return launch(head_post_kernel, dim3((unsigned) ((tasks + 3) / 4)), dim3(128), 0, (cudaStream_t) s, a);
}

int sm100_argmax(sm100_stream_t s, const float * x, int64_t n, int32_t * out) {
    if (x == nullptr || out == nullptr || n <= 0) return fail(ST_INVALID, "argmax: bad arguments");
    return launch(argmax_kernel, dim3(1), dim3(1024), 0, (cudaStream_t) s, x, n, out);
}

}  // extern "C"
