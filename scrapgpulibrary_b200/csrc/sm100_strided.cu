// Strided ("view") forms of the decode ops: every tensor is a pointer plus ggml-style extents ne[4] and byte
// strides nb[4], which is what the backend vtable receives in scrapgpu_tensor_desc.  These kernels honour
// arbitrary nb[1..3] (padded rows, slices, broadcast operands, transposed views for CPY) so that the plugin can
// serve the same descriptors the reference's CPU backend serves (src/backends/cpu/api.cpp:394-830, arithmetic
// src/core/ref/ops.cpp).  Dense shapes on the decode path are routed to the specialised kernels of sm100_ops.cu
// by the callers; what lands here is correctness-first.
#include "sm100_common.cuh"

namespace sm100 {

// Activation pointers are deliberately NOT __restrict__ / __ldg: kernels are launched with programmatic dependent
// launch, so a kernel may start while the kernel that produces its inputs is still running.  The non-coherent
// read-only path (ld.global.nc) is only valid for data that does not change during the kernel's lifetime, which
// under early launch includes the producer's writes; only weights (constant across the stream) use it.

struct V4 {
    char * p;
    int64_t ne[4];
    int64_t nb[4];
};

static V4 load_view(const sm100_view * v) {
    V4 o;
    o.p = (char *) v->data;
    for (int i = 0; i < 4; ++i) {
        o.ne[i] = v->ne[i] > 0 ? v->ne[i] : 1;
        o.nb[i] = v->nb[i];
    }
    return o;
}

__device__ __forceinline__ void unflatten(int64_t idx, const int64_t * ne, int64_t & i0, int64_t & i1, int64_t & i2, int64_t & i3) {
    i0 = idx % ne[0];
    idx /= ne[0];
    i1 = idx % ne[1];
    idx /= ne[1];
    i2 = idx % ne[2];
    i3 = idx / ne[2];
}

__device__ __forceinline__ int64_t off4(const V4 & v, int64_t i0, int64_t i1, int64_t i2, int64_t i3) {
    return i0 * v.nb[0] + i1 * v.nb[1] + i2 * v.nb[2] + i3 * v.nb[3];
}

// ADD / SUB / MUL / DIV (ops.cpp:280-312): src1 broadcasts by modulo over every dim
__global__ void binary_kernel(int op, V4 a, V4 b, V4 y, int64_t total) {
    pdl_wait();
    pdl_launch_dependents();
    for (int64_t idx = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; idx < total; idx += (int64_t) gridDim.x * blockDim.x) {
        int64_t i0, i1, i2, i3;
        unflatten(idx, y.ne, i0, i1, i2, i3);
        const float av = *(const float *) (a.p + off4(a, i0, i1, i2, i3));
        const float bv = *(const float *) (b.p + off4(b, i0 % b.ne[0], i1 % b.ne[1], i2 % b.ne[2], i3 % b.ne[3]));
        float r;
        switch (op) {
            case 0: r = __fadd_rn(av, bv); break;
            case 1: r = __fsub_rn(av, bv); break;
            case 2: r = __fmul_rn(av, bv); break;
            default: r = __fdiv_rn(av, bv); break;
        }
        *(float *) (y.p + off4(y, i0, i1, i2, i3)) = r;
    }
}

// GLU (ops.cpp:383-425): kind 0 SwiGLU x / (1 + expf(-x)) * g, kind 1 ReGLU max(x, 0) * g
__global__ void glu_kernel(int kind, V4 x, V4 g, int split, int swapped, V4 y, int64_t total) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t nc = y.ne[0];
    for (int64_t idx = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; idx < total; idx += (int64_t) gridDim.x * blockDim.x) {
        int64_t i0, i1, i2, i3;
        unflatten(idx, y.ne, i0, i1, i2, i3);
        float xv, gv;
        if (split) {
            xv = *(const float *) (x.p + off4(x, i0, i1, i2, i3));
            gv = *(const float *) (g.p + off4(g, i0, i1, i2, i3));
        } else {
            xv = *(const float *) (x.p + off4(x, i0 + (swapped ? nc : 0), i1, i2, i3));
            gv = *(const float *) (x.p + off4(x, i0 + (swapped ? 0 : nc), i1, i2, i3));
        }
        const float act = kind == 0 ? __fdiv_rn(xv, __fadd_rn(1.0f, expf(-xv))) : fmaxf(xv, 0.0f);
        *(float *) (y.p + off4(y, i0, i1, i2, i3)) = __fmul_rn(act, gv);
    }
}

// RMS_NORM family (ops.cpp:440-519), one CTA per row (i1, i2, i3)
__global__ void __launch_bounds__(256) rms_norm_view_kernel(V4 x, V4 add, int has_add, const float * w, V4 sum_out, int has_sum, V4 y, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ double red[8];
    __shared__ float s_scale;
    int64_t row = blockIdx.x;
    const int64_t i1 = row % x.ne[1];
    row /= x.ne[1];
    const int64_t i2 = row % x.ne[2], i3 = row / x.ne[2];
    const int64_t ne0 = x.ne[0];
    double sum = 0.0;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) {
        float v = *(const float *) (x.p + off4(x, i, i1, i2, i3));
        if (has_add) {
            v = __fadd_rn(v, *(const float *) (add.p + off4(add, i, i1, i2, i3)));
            if (has_sum) *(float *) (sum_out.p + off4(sum_out, i, i1, i2, i3)) = v;
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
        s_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float) (t / (double) ne0), eps)));
    }
    __syncthreads();
    const float scale = s_scale;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) {
        float v;
        if (has_add && has_sum) v = *(const float *) (sum_out.p + off4(sum_out, i, i1, i2, i3));
        else if (has_add) v = __fadd_rn(*(const float *) (x.p + off4(x, i, i1, i2, i3)), *(const float *) (add.p + off4(add, i, i1, i2, i3)));
        else v = *(const float *) (x.p + off4(x, i, i1, i2, i3));
        const float t = __fmul_rn(v, scale);
        *(float *) (y.p + off4(y, i, i1, i2, i3)) = w != nullptr ? __fmul_rn(t, w[i]) : t;
    }
}

__device__ __forceinline__ float load_as_float(const char * p, int dtype) {
    if (dtype == DT_F32) return *(const float *) p;
    if (dtype == DT_F16) return __half2float(*(const __half *) p);
    return __uint_as_float((uint32_t) (*(const unsigned short *) p) << 16);  // BF16
}

__device__ __forceinline__ void store_from_float(char * p, int dtype, float v) {
    if (dtype == DT_F32) {
        *(float *) p = v;
    } else if (dtype == DT_F16) {
        *(__half *) p = __float2half_rn(v);
    } else {
        // BF16, round to nearest even, NaN kept (ops.cpp:41-52)
        uint32_t bits = __float_as_uint(v);
        if ((bits & 0x7fffffffu) > 0x7f800000u) {
            *(unsigned short *) p = (unsigned short) ((bits >> 16) | 0x0040u);
        } else {
            bits += 0x7fffu + ((bits >> 16) & 1u);
            *(unsigned short *) p = (unsigned short) (bits >> 16);
        }
    }
}

// ROPE (ops.cpp:530-634) over a view [ne0, heads, tokens, batch]; optional frequency factors; yarn is left to
// the caller to reject
__global__ void rope_view_kernel(V4 x, const int32_t * positions, const float * table, int32_t table_first,
                                 int32_t table_n, const float * freq_factors, V4 y, int n_dims, int neox, float theta_scale,
                                 float freq_scale, float attn_factor, int64_t total, int dtype) {
    const int64_t es = dtype == DT_F16 ? 2 : 4;   // x and y share the dtype (ops.cpp:531-533)
    pdl_wait();
    pdl_launch_dependents();
    const int64_t hp = x.ne[0] / 2;
    for (int64_t idx = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; idx < total; idx += (int64_t) gridDim.x * blockDim.x) {
        int64_t r = idx;
        const int64_t j = r % hp;
        r /= hp;
        const int64_t i1 = r % x.ne[1];
        r /= x.ne[1];
        const int64_t i2 = r % x.ne[2], i3 = r / x.ne[2];
        const char * xr = x.p + off4(x, 0, i1, i2, i3);
        char * yr = y.p + off4(y, 0, i1, i2, i3);
        if (j < n_dims / 2) {
            const int32_t pos = positions[i2];
            const int64_t rel = (int64_t) pos - table_first;
            float cs, sn;
            if (table != nullptr && freq_factors == nullptr && rel >= 0 && rel < table_n) {
                const float2 v = *reinterpret_cast<const float2 *>(table + (rel * (n_dims / 2) + j) * 2);
                cs = v.x;
                sn = v.y;
            } else {
                float theta = (float) pos;
                for (int q = 0; q < (int) j; ++q) theta = __fmul_rn(theta, theta_scale);
                const float factor = freq_factors != nullptr ? freq_factors[j] : 1.0f;
                const float th = __fmul_rn(freq_scale, __fdiv_rn(theta, factor));
                cs = __fmul_rn(cosf(th), attn_factor);
                sn = __fmul_rn(sinf(th), attn_factor);
            }
            const int64_t e0 = neox ? j : 2 * j, e1 = neox ? j + n_dims / 2 : 2 * j + 1;
            const float x0 = load_as_float(xr + e0 * es, dtype), x1 = load_as_float(xr + e1 * es, dtype);
            store_from_float(yr + e0 * es, dtype, __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn)));
            store_from_float(yr + e1 * es, dtype, __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs)));
        } else {
            const int64_t e = 2 * (j - n_dims / 2) + n_dims;
            store_from_float(yr + e * es, dtype, load_as_float(xr + e * es, dtype));
            store_from_float(yr + (e + 1) * es, dtype, load_as_float(xr + (e + 1) * es, dtype));
        }
    }
}

__device__ __forceinline__ float block_reduce_v(float v, bool is_max, float * red) {
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

__device__ __forceinline__ float load_mask(const V4 & m, int f16, int64_t i0, int64_t i1, int64_t i2, int64_t i3) {
    const char * p = m.p + off4(m, i0, i1, i2 % m.ne[2], i3 % m.ne[3]);
    return f16 ? __half2float(*(const __half *) p) : *(const float *) p;
}

// SOFT_MAX (ops.cpp:636-684), one CTA per row, mask F32 or F16 broadcast over dims 2 and 3, in place allowed
__global__ void __launch_bounds__(256) soft_max_view_kernel(V4 x, V4 mask, int has_mask, int mask_f16, V4 y, float scale) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float red[8];
    int64_t row = blockIdx.x;
    const int64_t i1 = row % x.ne[1];
    row /= x.ne[1];
    const int64_t i2 = row % x.ne[2], i3 = row / x.ne[2];
    const int64_t ne0 = x.ne[0];
    float mx = -INFINITY;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) {
        float v = __fmul_rn(*(const float *) (x.p + off4(x, i, i1, i2, i3)), scale);
        if (has_mask) v = __fadd_rn(v, load_mask(mask, mask_f16, i, i1, i2, i3));
        mx = fmaxf(mx, v);
    }
    mx = block_reduce_v(mx, true, red);
    float sum = 0.f;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) {
        float v = __fmul_rn(*(const float *) (x.p + off4(x, i, i1, i2, i3)), scale);
        if (has_mask) v = __fadd_rn(v, load_mask(mask, mask_f16, i, i1, i2, i3));
        const float e = expf(v - mx);
        *(float *) (y.p + off4(y, i, i1, i2, i3)) = e;
        sum += e;
    }
    sum = block_reduce_v(sum, false, red);
    const float inv = __fdiv_rn(1.0f, sum);
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) {
        float * q = (float *) (y.p + off4(y, i, i1, i2, i3));
        *q = __fmul_rn(*q, inv);
    }
}

// SCALE / CLAMP / SQR / SQRT / UNARY (ops.cpp:314-381): y = f(x) element by element over F32 views of one shape.
// code: 0 SCALE (x * p0 + p1, two roundings as the reference's unfused expression), 1 CLAMP to [p0, p1], 2 SQR, 3 SQRT,
// 10.. = 10 + scrapgpu_unary_kind (SILU, RELU, NEG, ABS, SIGMOID, TANH)
__global__ void unary_kernel(int code, float p0, float p1, V4 x, V4 y, int64_t total) {
    pdl_wait();
    pdl_launch_dependents();
    for (int64_t idx = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; idx < total; idx += (int64_t) gridDim.x * blockDim.x) {
        int64_t i0, i1, i2, i3;
        unflatten(idx, y.ne, i0, i1, i2, i3);
        const float v = *(const float *) (x.p + off4(x, i0, i1, i2, i3));
        float r;
        switch (code) {
            case 0: r = __fadd_rn(__fmul_rn(v, p0), p1); break;
            case 1: r = fminf(fmaxf(v, p0), p1); break;
            case 2: r = __fmul_rn(v, v); break;
            case 3: r = __fsqrt_rn(v); break;
            case 10: r = __fdiv_rn(v, __fadd_rn(1.0f, expf(-v))); break;
            case 11: r = fmaxf(v, 0.0f); break;
            case 12: r = -v; break;
            case 13: r = fabsf(v); break;
            case 14: r = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-v))); break;
            default: r = tanhf(v); break;
        }
        *(float *) (y.p + off4(y, i0, i1, i2, i3)) = r;
    }
}

// CPY / DUP / CONT (ops.cpp:764-800): element k of the source in logical order goes to element k of the
// destination in logical order, through both sets of strides (so a transposed source view transposes)
__global__ void cpy_kernel(V4 s, int sdt, V4 d, int ddt, int64_t total) {
    pdl_wait();
    pdl_launch_dependents();
    for (int64_t idx = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; idx < total; idx += (int64_t) gridDim.x * blockDim.x) {
        int64_t a0, a1, a2, a3, b0, b1, b2, b3;
        unflatten(idx, s.ne, a0, a1, a2, a3);
        unflatten(idx, d.ne, b0, b1, b2, b3);
        store_from_float(d.p + off4(d, b0, b1, b2, b3), ddt, load_as_float(s.p + off4(s, a0, a1, a2, a3), sdt));
    }
}

// SET_ROWS (ops.cpp:724-762): dst[:, ids[i1, i2 % ine1, i3 % ine2], i2, i3] = src[:, i1, i2, i3]
__global__ void set_rows_view_kernel(V4 s, int sdt, V4 ids, int ids_i64, V4 d, int ddt, int64_t total, int * error_flag) {
    pdl_wait();
    pdl_launch_dependents();
    for (int64_t idx = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; idx < total; idx += (int64_t) gridDim.x * blockDim.x) {
        int64_t i0, i1, i2, i3;
        unflatten(idx, s.ne, i0, i1, i2, i3);
        const char * pi = ids.p + off4(ids, i1, i2 % ids.ne[1], i3 % ids.ne[2], 0);
        const int64_t row = ids_i64 ? *(const int64_t *) pi : (int64_t) * (const int32_t *) pi;
        if (row < 0 || row >= d.ne[1]) {
            if (error_flag != nullptr) atomicExch(error_flag, 1);
            continue;
        }
        store_from_float(d.p + off4(d, i0, row, i2, i3), ddt, load_as_float(s.p + off4(s, i0, i1, i2, i3), sdt));
    }
}

// TOP_K with k = 1 per row of a view (ops.cpp:1189-1228): one CTA per row
__global__ void __launch_bounds__(1024) top1_view_kernel(V4 x, V4 out) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float sv[32];
    __shared__ int si[32];
    int64_t row = blockIdx.x;
    const int64_t i1 = row % x.ne[1];
    row /= x.ne[1];
    const int64_t i2 = row % x.ne[2], i3 = row / x.ne[2];
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int64_t i = threadIdx.x; i < x.ne[0]; i += blockDim.x) {
        const float v = *(const float *) (x.p + off4(x, i, i1, i2, i3));
        if (v > best || bi == 0x7fffffff) { best = v; bi = (int) i; }
    }
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
        if (threadIdx.x == 0) *(int32_t *) (out.p + off4(out, 0, i1, i2, i3)) = bi;
    }
}

// CONT_MUL_MAT (include/scrapgpu/op.h:47; input order src/backends/opencl11/api.cpp:11-12; reference kernels
// attn.cl:123-237): dst[i1, 0, i2, i3] = sum_i0 a[i0, i1, i2 / r2, i3 / r3] * x[i0, 0, i2, i3] where `a` is the
// transposed view a CONT would have copied first (its dim 1 is the contiguous one: the P.V product of attention over
// a V cache stored [head][position][dim] or [position][head][dim]).  A CTA takes 32 consecutive i1 (the 32 lanes of
// a warp read 32 consecutive elements of `a`) and splits i0 over its 8 warps; f32 accumulation.
__global__ void __launch_bounds__(256) cont_mul_mat_kernel(V4 a, int a_f16, V4 x, V4 y, int64_t r2, int64_t r3) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float red[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t i1 = (int64_t) blockIdx.x * 32 + tx;
    const int64_t i2 = blockIdx.y % x.ne[2], i3 = blockIdx.y / x.ne[2];
    float acc = 0.f;
    if (i1 < a.ne[1]) {
        const char * ap = a.p + i1 * a.nb[1] + (i2 / r2) * a.nb[2] + (i3 / r3) * a.nb[3];
        const char * xp = x.p + i2 * x.nb[2] + i3 * x.nb[3];
        for (int64_t i0 = ty; i0 < a.ne[0]; i0 += 8) {
            const float av = a_f16 ? __half2float(*(const __half *) (ap + i0 * a.nb[0])) : *(const float *) (ap + i0 * a.nb[0]);
            acc = fmaf(av, *(const float *) (xp + i0 * x.nb[0]), acc);
        }
    }
    red[ty][tx] = acc;
    __syncthreads();
    if (ty == 0 && i1 < a.ne[1]) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += red[w][tx];
        *(float *) (y.p + i1 * y.nb[0] + i2 * y.nb[2] + i3 * y.nb[3]) = v;
    }
}

static unsigned grid_cap(int64_t n, int threads) {
    int64_t g = (n + threads - 1) / threads;
    const int64_t cap = (int64_t) sm_count() * 16;
    if (g > cap) g = cap;
    return (unsigned) (g < 1 ? 1 : g);
}

static int64_t count(const V4 & v) { return v.ne[0] * v.ne[1] * v.ne[2] * v.ne[3]; }

}  // namespace sm100

using namespace sm100;

extern "C" {

int sm100_binary(sm100_stream_t s, int op, const sm100_view * a, const sm100_view * b, const sm100_view * y) {
    if (a == nullptr || b == nullptr || y == nullptr || a->data == nullptr || b->data == nullptr || y->data == nullptr) return fail(ST_INVALID, "binary: null view");
    if (op < 0 || op > 3) return fail(ST_UNSUPPORTED, "binary: unknown op");
    const V4 va = load_view(a), vb = load_view(b), vy = load_view(y);
    const int64_t total = count(vy);
    return launch(binary_kernel, dim3(grid_cap(total, 256)), dim3(256), 0, (cudaStream_t) s, op, va, vb, vy, total);
}

int sm100_glu(sm100_stream_t s, int kind, const sm100_view * x, const sm100_view * g, int swapped, const sm100_view * y) {
    if (x == nullptr || y == nullptr || x->data == nullptr || y->data == nullptr) return fail(ST_INVALID, "glu: null view");
    if (kind < 0 || kind > 1) return fail(ST_UNSUPPORTED, "glu: unknown kind");
    const V4 vx = load_view(x), vy = load_view(y);
    const V4 vg = g != nullptr ? load_view(g) : vx;
    const int64_t total = count(vy);
    return launch(glu_kernel, dim3(grid_cap(total, 256)), dim3(256), 0, (cudaStream_t) s, kind, vx, vg, g != nullptr ? 1 : 0, swapped, vy, total);
}

int sm100_rms_norm_view(sm100_stream_t s, const sm100_view * x, const sm100_view * add, const float * w, const sm100_view * sum_out,
                        const sm100_view * y, float eps) {
    if (x == nullptr || y == nullptr || x->data == nullptr || y->data == nullptr) return fail(ST_INVALID, "rms_norm: null view");
    const V4 vx = load_view(x), vy = load_view(y);
    const V4 va = add != nullptr ? load_view(add) : vx, vs = sum_out != nullptr ? load_view(sum_out) : vy;
    const int64_t rows = vx.ne[1] * vx.ne[2] * vx.ne[3];
    if (rows > INT32_MAX) return fail(ST_UNSUPPORTED, "rms_norm: too many rows");
    return launch(rms_norm_view_kernel, dim3((unsigned) rows), dim3(256), 0, (cudaStream_t) s, vx, va, add != nullptr ? 1 : 0, w, vs,
                  sum_out != nullptr ? 1 : 0, vy, eps);
}

int sm100_unary(sm100_stream_t s, int code, float p0, float p1, const sm100_view * x, const sm100_view * y) {
    if (x == nullptr || y == nullptr || x->data == nullptr || y->data == nullptr) return fail(ST_INVALID, "unary: null view");
    if (!((code >= 0 && code <= 3) || (code >= 10 && code <= 15))) return fail(ST_UNSUPPORTED, "unary: unknown function code %d", code);
    const V4 vx = load_view(x), vy = load_view(y);
    const int64_t total = count(vy);
    if (total != count(vx)) return fail(ST_INVALID, "unary: src0 must have the shape of dst");
    return launch(unary_kernel, dim3(grid_cap(total, 256)), dim3(256), 0, (cudaStream_t) s, code, p0, p1, vx, vy, total);
}

int sm100_rope_view(sm100_stream_t s, const sm100_view * x, const int32_t * positions, const float * table, int32_t table_first_position,
                    int32_t table_positions, const float * freq_factors, const sm100_view * y, int n_dims, int neox, float freq_base,
                    float freq_scale, float attn_factor) {
    return sm100_rope_view_dt(s, DT_F32, x, positions, table, table_first_position, table_positions, freq_factors, y, n_dims, neox, freq_base,
                              freq_scale, attn_factor);
}

int sm100_rope_view_dt(sm100_stream_t s, int dtype, const sm100_view * x, const int32_t * positions, const float * table,
                       int32_t table_first_position, int32_t table_positions, const float * freq_factors, const sm100_view * y, int n_dims,
                       int neox, float freq_base, float freq_scale, float attn_factor) {
    if (dtype != DT_F32 && dtype != DT_F16) return fail(ST_UNSUPPORTED, "rope: F32 or F16 tensors");
    if (x == nullptr || y == nullptr || positions == nullptr || x->data == nullptr || y->data == nullptr) return fail(ST_INVALID, "rope: null view");
    const V4 vx = load_view(x), vy = load_view(y);
    if (n_dims <= 0 || n_dims % 2 != 0 || n_dims > vx.ne[0] || vx.ne[0] % 2 != 0) return fail(ST_INVALID, "rope: n_dims must be a positive even number not above ne0 (ne0 even)");
    const int64_t es = dtype == DT_F16 ? 2 : 4;
    if (vx.nb[0] != es || vy.nb[0] != es) return fail(ST_UNSUPPORTED, "rope: rows must be contiguous");
    const float theta_scale = powf(freq_base, -2.0f / (float) n_dims);
    const int64_t total = (vx.ne[0] / 2) * vx.ne[1] * vx.ne[2] * vx.ne[3];
    return launch(rope_view_kernel, dim3(grid_cap(total, 256)), dim3(256), 0, (cudaStream_t) s, vx, positions, table, table_first_position,
                  table_positions, freq_factors, vy, n_dims, neox, theta_scale, freq_scale, attn_factor, total, dtype);
}

int sm100_soft_max_view(sm100_stream_t s, const sm100_view * x, const sm100_view * mask, int mask_is_f16, const sm100_view * y, float scale) {
    if (x == nullptr || y == nullptr || x->data == nullptr || y->data == nullptr) return fail(ST_INVALID, "soft_max: null view");
    const V4 vx = load_view(x), vy = load_view(y);
    const V4 vm = mask != nullptr ? load_view(mask) : vx;
    const int64_t rows = vx.ne[1] * vx.ne[2] * vx.ne[3];
    if (rows > INT32_MAX) return fail(ST_UNSUPPORTED, "soft_max: too many rows");
    return launch(soft_max_view_kernel, dim3((unsigned) rows), dim3(256), 0, (cudaStream_t) s, vx, vm, mask != nullptr ? 1 : 0, mask_is_f16, vy, scale);
}

int sm100_cpy(sm100_stream_t s, const sm100_view * src, int src_dtype, const sm100_view * dst, int dst_dtype) {
    if (src == nullptr || dst == nullptr || src->data == nullptr || dst->data == nullptr) return fail(ST_INVALID, "cpy: null view");
    const bool ok_s = src_dtype == DT_F32 || src_dtype == DT_F16 || src_dtype == 5, ok_d = dst_dtype == DT_F32 || dst_dtype == DT_F16 || dst_dtype == 5;
    if (!ok_s || !ok_d) return fail(ST_UNSUPPORTED, "cpy: F32, F16 and BF16 only");
    const V4 vs = load_view(src), vd = load_view(dst);
    const int64_t total = count(vs);
    if (total != count(vd)) return fail(ST_INVALID, "cpy: element counts differ");
    return launch(cpy_kernel, dim3(grid_cap(total, 256)), dim3(256), 0, (cudaStream_t) s, vs, src_dtype, vd, dst_dtype, total);
}

int sm100_set_rows_view(sm100_stream_t s, const sm100_view * src, int src_dtype, const sm100_view * ids, int ids_are_i64, const sm100_view * dst,
                        int dst_dtype) {
    if (src == nullptr || ids == nullptr || dst == nullptr || src->data == nullptr || ids->data == nullptr || dst->data == nullptr)
        return fail(ST_INVALID, "set_rows: null view");
    if ((src_dtype != DT_F32 && src_dtype != DT_F16) || (dst_dtype != DT_F32 && dst_dtype != DT_F16)) return fail(ST_UNSUPPORTED, "set_rows: F32/F16 only");
    const V4 vs = load_view(src), vi = load_view(ids), vd = load_view(dst);
    const int64_t total = count(vs);
    return launch(set_rows_view_kernel, dim3(grid_cap(total, 256)), dim3(256), 0, (cudaStream_t) s, vs, src_dtype, vi, ids_are_i64, vd, dst_dtype, total,
                  (int *) nullptr);
}

int sm100_top1_view(sm100_stream_t s, const sm100_view * x, const sm100_view * out) {
    if (x == nullptr || out == nullptr || x->data == nullptr || out->data == nullptr) return fail(ST_INVALID, "top_k: null view");
    const V4 vx = load_view(x), vo = load_view(out);
    const int64_t rows = vx.ne[1] * vx.ne[2] * vx.ne[3];
    if (rows > INT32_MAX) return fail(ST_UNSUPPORTED, "top_k: too many rows");
    return launch(top1_view_kernel, dim3((unsigned) rows), dim3(1024), 0, (cudaStream_t) s, vx, vo);
}

int sm100_cont_mul_mat(sm100_stream_t s, const sm100_view * a, int a_dtype, const sm100_view * x, const sm100_view * y) {
    if (a == nullptr || x == nullptr || y == nullptr || a->data == nullptr || x->data == nullptr || y->data == nullptr) return fail(ST_INVALID, "cont_mul_mat: null view");
    if (a_dtype != DT_F16 && a_dtype != DT_F32) return fail(ST_UNSUPPORTED, "cont_mul_mat: the transposed view must be F16 or F32");
    const V4 va = load_view(a), vx = load_view(x), vy = load_view(y);
    if (vx.ne[1] != 1 || vx.ne[0] != va.ne[0] || vx.ne[2] % va.ne[2] != 0 || vx.ne[3] % va.ne[3] != 0)
        return fail(ST_INVALID, "cont_mul_mat: x must be one column [a.ne0, 1, n2, n3] with n2, n3 multiples of a's");
    if (vy.ne[0] != va.ne[1] || vy.ne[1] != 1 || vy.ne[2] != vx.ne[2] || vy.ne[3] != vx.ne[3]) return fail(ST_INVALID, "cont_mul_mat: dst must be [a.ne1, 1, x.ne2, x.ne3]");
    const int64_t outer = vx.ne[2] * vx.ne[3], tiles = (va.ne[1] + 31) / 32;
    if (outer > 65535 || tiles > INT32_MAX) return fail(ST_UNSUPPORTED, "cont_mul_mat: too many slices");
    return launch(cont_mul_mat_kernel, dim3((unsigned) tiles, (unsigned) outer), dim3(256), 0, (cudaStream_t) s, va, a_dtype == DT_F16 ? 1 : 0, vx, vy,
                  vx.ne[2] / va.ne[2], vx.ne[3] / va.ne[3]);
}

}  // extern "C"
