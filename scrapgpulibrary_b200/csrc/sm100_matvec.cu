// Decode MUL_MAT (M <= 8 activation columns): fused dequantize-and-dot matvec kernels for sm_100a.
//
// Replaces, for the `cuda_sm100` backend, the reference's k_mvr_q4_0 / k_mvr_q8_0
// (src/backends/opencl11/kernels/mul_mv_r.cl:240-323), k_mvr_q4_k / k_mvr_q6_k (mul_mv_k.cl:396-486)
// and the CPU path exec_mul_mat (src/core/ref/ops.cpp:891-984).  HBM-bound: each weight byte is read
// once with 16-byte streaming loads, unpacked in registers, accumulated in f32.
//
// Kernel A  matvec_stream<Unit>   packed layout, M = 1, K a multiple of 32 units.  A thread owns one
//           column unit (16 or 32 bytes of every row it visits) and keeps the matching activations
//           in registers for the whole launch, so the inner loop has no shared-memory or L1 traffic
//           besides the weight stream itself.  The weight loads of the first rows are issued before
//           griddepcontrol.wait, so under programmatic dependent launch they overlap the tail of the
//           previous kernel on the stream.
// Kernel B  matvec_rows<Unit, M>  any layout / shape / M <= 8: one warp per weight row, activations
//           through L1.
#include "sm100_quant_units.cuh"
#include "sm100_wide_units.cuh"

#include <cstdlib>

namespace sm100 {

int matvec_q6k_imma_tiles(cudaStream_t s, const void * w, int64_t k, int64_t n, const float * x, float * y, bool * handled);
int matvec_q6k_imma_cols(cudaStream_t s, const void * w, int64_t k, int64_t n, const float * x, int64_t ldx, int m, float * y, int64_t ldy, bool * handled);
int matvec_b32_imma_tiles(cudaStream_t s, int dtype, const void * w, int64_t k, int64_t n, const float * x, float * y, bool * handled);
int matvec_q4k_imma_cols_tiles(cudaStream_t s, const void * w, int64_t k, int64_t n, const float * x, int64_t ldx, int64_t m, float * y, int64_t ldy,
                               bool * handled);
int matvec_q4k_imma_tiles(cudaStream_t s, const void * w, int64_t k, int64_t n, const float * x, int64_t ldx, int64_t m, float * y, int64_t ldy,
                          bool * handled);
int matvec_q4k_tiles(cudaStream_t s, const void * w, int64_t k, int64_t n, const float * x, int64_t ldx, int64_t m, float * y, int64_t ldy,
                     bool * handled);
int q4k_pass_width(int64_t k, int64_t m);
int matvec_q4k_ring_multi(cudaStream_t s, int count, const void * const * ws, const int64_t * ns, int64_t k, const float * x,
                          float * const * ys, bool * handled, const Q4KPrologue * pro, const ArFuse * fuse);

// ---- natural-layout loading: assemble the packed-unit registers from GGUF blocks -----------------

__device__ __forceinline__ uint32_t ld_u32_any(const uint8_t * p) {
    const uintptr_t a = (uintptr_t) p;
    if ((a & 3) == 0) return __ldg((const uint32_t *) p);
    if ((a & 1) == 0) return (uint32_t) __ldg((const unsigned short *) p) | ((uint32_t) __ldg((const unsigned short *) (p + 2)) << 16);
    return (uint32_t) __ldg(p) | ((uint32_t) __ldg(p + 1) << 8) | ((uint32_t) __ldg(p + 2) << 16) | ((uint32_t) __ldg(p + 3) << 24);
}
__device__ __forceinline__ uint4 ld_u128_any(const uint8_t * p) {
    if (((uintptr_t) p & 15) == 0) return __ldg((const uint4 *) p);
    return make_uint4(ld_u32_any(p), ld_u32_any(p + 4), ld_u32_any(p + 8), ld_u32_any(p + 12));
}
__device__ __forceinline__ uint32_t ld_u16_any(const uint8_t * p) {
    if (((uintptr_t) p & 1) == 0) return (uint32_t) __ldg((const unsigned short *) p);
    return (uint32_t) __ldg(p) | ((uint32_t) __ldg(p + 1) << 8);
}

template <class U> struct Natural;

template <> struct Natural<UnitQ4K> {
    __device__ static __forceinline__ void load(const uint8_t * row, int cu, UnitQ4K::Data & d) {
        const uint8_t * blk = row + (int64_t) (cu >> 3) * 144;
        d.q = ld_u128_any(blk + 16 + (cu & 7) * 16);
        const uint32_t h0 = ld_u32_any(blk), s0 = ld_u32_any(blk + 4), s1 = ld_u32_any(blk + 8), s2 = ld_u32_any(blk + 12);
        // natural 12-byte scale bytes s[0..11] -> the four 24-bit fields of the packed header
        uint32_t f[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            uint32_t sc[2], mn[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = 2 * p + e;
                if (j < 4) {
                    sc[e] = (s0 >> (8 * j)) & 63u;
                    mn[e] = (s1 >> (8 * j)) & 63u;
                } else {
                    const uint32_t lo = (s2 >> (8 * (j - 4))) & 255u;
                    sc[e] = (lo & 15u) | ((((s0 >> (8 * (j - 4))) & 255u) >> 6) << 4);
                    mn[e] = (lo >> 4) | ((((s1 >> (8 * (j - 4))) & 255u) >> 6) << 4);
                }
            }
            f[p] = sc[0] | (mn[0] << 6) | (sc[1] << 12) | (mn[1] << 18);
        }
        d.h.x = h0;
        d.h.y = f[0] | (f[1] << 24);
        d.h.z = (f[1] >> 8) | (f[2] << 16);
        d.h.w = (f[2] >> 16) | (f[3] << 8);
    }
};

template <> struct Natural<UnitQ6K> {
    __device__ static __forceinline__ void load(const uint8_t * row, int cu, UnitQ6K::Data & d) {
        const uint8_t * blk = row + (int64_t) (cu >> 2) * 210;
        const int u = cu & 3, h = u >> 1, c = u & 1;
        d.a = ld_u128_any(blk + 64 * h + 16 * c);
        d.b = ld_u128_any(blk + 64 * h + 32 + 16 * c);
        d.h = ld_u128_any(blk + 128 + 16 * u);
        const uint8_t * s = blk + 192 + 8 * h + c;
        d.sc = (uint32_t) __ldg(s) | ((uint32_t) __ldg(s + 2) << 8) | ((uint32_t) __ldg(s + 4) << 16) | ((uint32_t) __ldg(s + 6) << 24);
        d.d = ld_u16_any(blk + 208);
    }
};

template <> struct Natural<UnitQ40> {
    __device__ static __forceinline__ void load(const uint8_t * row, int cu, UnitQ40::Data & d) {
        const uint8_t * blk = row + (int64_t) cu * 18;
        d.q = ld_u128_any(blk + 2);
        d.d = ld_u16_any(blk);
    }
};

template <> struct Natural<UnitQ80> {
    __device__ static __forceinline__ void load(const uint8_t * row, int cu, UnitQ80::Data & d) {
        const uint8_t * blk = row + (int64_t) (cu >> 1) * 34;
        d.q = ld_u128_any(blk + 2 + (cu & 1) * 16);
        d.d = ld_u16_any(blk);
    }
};

// unquantized weights ride the same row kernel: F32 (4 per unit) and F16 (8 per unit)
struct UnitF32 {
    static constexpr int DTYPE = DT_F32;
    static constexpr int WEIGHTS = 4;
    static constexpr int UNITS_PER_BLOCK = 1;
    static constexpr int XSUMS = 1;
    struct Data { uint4 q; };
    __device__ static __forceinline__ int64_t x_index(int cu, int i) { return (int64_t) cu * 4 + i; }
    __device__ static __forceinline__ int sum_slot(int) { return 0; }
    __device__ static __forceinline__ float dot(const Data & d, int, const float * x, const float *) {
        float acc = __uint_as_float(d.q.x) * x[0];
        acc = fmaf(__uint_as_float(d.q.y), x[1], acc);
        acc = fmaf(__uint_as_float(d.q.z), x[2], acc);
        return fmaf(__uint_as_float(d.q.w), x[3], acc);
    }
};
template <> struct Natural<UnitF32> {
    __device__ static __forceinline__ void load(const uint8_t * row, int cu, UnitF32::Data & d) { d.q = ld_u128_any(row + (int64_t) cu * 16); }
};

struct UnitF16 {
    static constexpr int DTYPE = DT_F16;
    static constexpr int WEIGHTS = 8;
    static constexpr int UNITS_PER_BLOCK = 1;
    static constexpr int XSUMS = 1;
    struct Data { uint4 q; };
    __device__ static __forceinline__ int64_t x_index(int cu, int i) { return (int64_t) cu * 8 + i; }
    __device__ static __forceinline__ int sum_slot(int) { return 0; }
    __device__ static __forceinline__ float dot(const Data & d, int, const float * x, const float *) {
        const uint32_t w[4] = {d.q.x, d.q.y, d.q.z, d.q.w};
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc = fmaf(half_bits_to_float(w[i] & 0xFFFFu), x[2 * i], acc);
            acc = fmaf(half_bits_to_float(w[i] >> 16), x[2 * i + 1], acc);
        }
        return acc;
    }
};
template <> struct Natural<UnitF16> {
    __device__ static __forceinline__ void load(const uint8_t * row, int cu, UnitF16::Data & d) { d.q = ld_u128_any(row + (int64_t) cu * 16); }
};

// ---- activations of one unit into registers ---------------------------------------------------------

template <class U>
__device__ __forceinline__ void load_x_unit(const float * x, int cu, float (&xr)[U::WEIGHTS], float (&sums)[U::XSUMS]) {
#pragma unroll
    for (int s = 0; s < U::XSUMS; ++s) sums[s] = 0.f;
#pragma unroll
    for (int g = 0; g < U::WEIGHTS / 4; ++g) {
        const float4 v = __ldcg(reinterpret_cast<const float4 *>(x + U::x_index(cu, 4 * g)));   // coherent load, see matvec_wide
        xr[4 * g + 0] = v.x; xr[4 * g + 1] = v.y; xr[4 * g + 2] = v.z; xr[4 * g + 3] = v.w;
        sums[U::sum_slot(4 * g)] += (v.x + v.y) + (v.z + v.w);
    }
}

// ---- kernel A: packed, M = 1, register-resident activations ---------------------------------------

template <class U>
__global__ void __launch_bounds__(U::MAX_THREADS) matvec_stream(const uint8_t * __restrict__ w, Planes P, const float * x,
                                                     float * y, int n_rows, int units_per_row, int rows_per_cta) {
    constexpr int STREAM_RIF = U::ROWS_IN_FLIGHT;
    extern __shared__ float red[];  // [STREAM_RIF][warps]
    const int tid = threadIdx.x;
    const int cu = tid % units_per_row;
    const int rl = tid / units_per_row;
    const int rp = blockDim.x / units_per_row;       // rows per pass
    const int warps = blockDim.x >> 5;
    const int warps_per_row = units_per_row >> 5;
    const int64_t bpr = units_per_row / U::UNITS_PER_BLOCK;
    const int row0 = blockIdx.x * rows_per_cta;
    const int row_end = min(n_rows, row0 + rows_per_cta);

    typename U::Data data[STREAM_RIF];
    // first batch of weights: independent of the predecessor kernel, so issue before the dependency wait
#pragma unroll
    for (int i = 0; i < STREAM_RIF; ++i) {
        const int r = row0 + rl + i * rp;
        if (r < row_end) U::load(w, P, r, bpr, cu, data[i]);
    }
    pdl_wait();
    float xr[U::WEIGHTS], sums[U::XSUMS];
    load_x_unit<U>(x, cu, xr, sums);
    pdl_launch_dependents();

    for (int base = row0; base < row_end; base += rp * STREAM_RIF) {
        float part[STREAM_RIF];
#pragma unroll
        for (int i = 0; i < STREAM_RIF; ++i) {
            const int r = base + rl + i * rp;
            part[i] = r < row_end ? U::dot(data[i], cu, xr, sums) : 0.f;
        }
        // prefetch the next batch while the reductions run
        const int next = base + rp * STREAM_RIF;
#pragma unroll
        for (int i = 0; i < STREAM_RIF; ++i) {
            const int r = next + rl + i * rp;
            if (r < row_end) U::load(w, P, r, bpr, cu, data[i]);
        }
#pragma unroll
        for (int i = 0; i < STREAM_RIF; ++i) {
            float v = part[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if ((tid & 31) == 0) red[i * warps + (tid >> 5)] = v;
        }
        __syncthreads();
        if (tid < rp * STREAM_RIF) {
            const int i = tid / rp, lr = tid % rp;
            const int r = base + lr + i * rp;
            if (r < row_end) {
                float v = 0.f;
                for (int k = 0; k < warps_per_row; ++k) v += red[i * warps + lr * warps_per_row + k];
                y[r] = v;
            }
        }
        __syncthreads();
    }
}

// ---- kernel A2: packed, M = 1, 32-byte wide units, conversion-free unpack, packed f32x2 FMAs ------------
//
// threads = units_per_row * rows_per_pass; a thread keeps the 32 or 64 activations of its column unit in
// registers and walks down the rows of its CTA with ROWS weight rows in flight.  Per batch of ROWS rows the
// per-thread partials are reduced with a transposing shuffle (6 shuffles for 4 rows instead of 20), then
// across the warps of a row through shared memory.

template <int ROWS>
__device__ __forceinline__ float transpose_reduce(const float (&v)[ROWS], int lane);

// 4 values per lane -> lane 8*r holds the warp-wide sum of value r
template <>
__device__ __forceinline__ float transpose_reduce<4>(const float (&v)[4], int lane) {
    const bool up16 = lane & 16, up8 = lane & 8;
    const float s0 = __shfl_xor_sync(0xffffffffu, up16 ? v[0] : v[2], 16);
    const float s1 = __shfl_xor_sync(0xffffffffu, up16 ? v[1] : v[3], 16);
    const float w0 = (up16 ? v[2] : v[0]) + s0;   // rows 0/2
    const float w1 = (up16 ? v[3] : v[1]) + s1;   // rows 1/3
    const float s2 = __shfl_xor_sync(0xffffffffu, up8 ? w0 : w1, 8);
    float u = (up8 ? w1 : w0) + s2;                // row = 2 * bit4 + bit3
    u += __shfl_xor_sync(0xffffffffu, u, 4);
    u += __shfl_xor_sync(0xffffffffu, u, 2);
    u += __shfl_xor_sync(0xffffffffu, u, 1);
    return u;
}

template <class W, int ROWS, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) matvec_wide(const uint8_t * __restrict__ w, Planes P, const float * x,
                                                          float * y, int n_rows, int units_per_row, int rows_per_cta) {
    static_assert(ROWS == 4, "the transposing reduction is written for 4 rows in flight");
    extern __shared__ float red[];  // [ROWS][warps]
    const int tid = threadIdx.x, lane = tid & 31;
    const int cu = tid % units_per_row;
    const int rl = tid / units_per_row;
    const int rp = blockDim.x / units_per_row;
    const int warps = blockDim.x >> 5;
    const int warps_per_row = units_per_row >> 5;
    const int64_t bpr = W::UNITS_PER_BLOCK > 0 ? units_per_row / W::UNITS_PER_BLOCK : (int64_t) units_per_row * -W::UNITS_PER_BLOCK;
    const int row0 = blockIdx.x * rows_per_cta;
    const int row_end = min(n_rows, row0 + rows_per_cta);

    typename W::Data data[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
        const int r = row0 + rl + i * rp;
        if (r < row_end) W::load(w, P, r, bpr, cu, data[i]);
    }
    pdl_wait();
    float2 xr[W::WEIGHTS / 2];
    float sums[W::XSUMS];
#pragma unroll
    for (int s = 0; s < W::XSUMS; ++s) sums[s] = 0.f;
#pragma unroll
    for (int g = 0; g < W::WEIGHTS / 4; ++g) {
        const float4 v = __ldcg(reinterpret_cast<const float4 *>(x + W::x_index(cu, g)));   // coherent: x may come from the kernel we overlap with
        xr[2 * g] = make_float2(v.x, v.y);
        xr[2 * g + 1] = make_float2(v.z, v.w);
        sums[W::sum_slot(g)] += (v.x + v.y) + (v.z + v.w);
    }
    pdl_launch_dependents();

    for (int base = row0; base < row_end; base += rp * ROWS) {
        float part[ROWS];
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            const int r = base + rl + i * rp;
            part[i] = r < row_end ? W::dot(data[i], cu, xr, sums) : 0.f;
        }
        const int next = base + rp * ROWS;
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            const int r = next + rl + i * rp;
            if (r < row_end) W::load(w, P, r, bpr, cu, data[i]);
        }
        const float u = transpose_reduce<ROWS>(part, lane);
        if ((lane & 7) == 0) red[(lane >> 3) * warps + (tid >> 5)] = u;
        __syncthreads();
        if (tid < rp * ROWS) {
            const int i = tid / rp, lr = tid % rp;
            const int r = base + lr + i * rp;
            if (r < row_end) {
                float v = 0.f;
                for (int k = 0; k < warps_per_row; ++k) v += red[i * warps + lr * warps_per_row + k];
                y[r] = v;
            }
        }
        __syncthreads();
    }
}

// ---- kernel B: one warp per row, any layout, M <= 8 -------------------------------------------------

template <class U, int M, bool PACKED>
__global__ void __launch_bounds__(256) matvec_rows(const uint8_t * __restrict__ w, Planes P, int64_t w_row_stride,
                                                   const float * x, int64_t ldx, float * y, int64_t ldy,
                                                   int row_begin, int n_rows, int units_per_row) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int warps = blockDim.x >> 5;
    const int64_t bpr = units_per_row / U::UNITS_PER_BLOCK;
    for (int r = row_begin + blockIdx.x * warps + (threadIdx.x >> 5); r < n_rows; r += gridDim.x * warps) {
        float acc[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = 0.f;
        for (int cu = lane; cu < units_per_row; cu += 32) {
            typename U::Data d;
            if (PACKED) {
                if constexpr (U::DTYPE >= 16) U::load(w, P, r, bpr, cu, d);
            } else {
                Natural<U>::load(w + (int64_t) r * w_row_stride, cu, d);
            }
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float xr[U::WEIGHTS], sums[U::XSUMS];
                load_x_unit<U>(x + (int64_t) m * ldx, cu, xr, sums);
                acc[m] += U::dot(d, cu, xr, sums);
            }
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float v = acc[m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) y[(int64_t) m * ldy + r] = v;
        }
    }
}

// scalar tail for rows whose K is not a whole number of units or whose x is not 16-byte aligned
// (F32 / F16 weights only; quantized rows are whole blocks by contract)
template <int DT>
__global__ void matvec_scalar(const uint8_t * __restrict__ w, int64_t w_row_stride, const float * x, int64_t ldx,
                              float * y, int64_t ldy, int n_rows, int k, int m_cols) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int warps = blockDim.x >> 5;
    for (int r = blockIdx.x * warps + (threadIdx.x >> 5); r < n_rows; r += gridDim.x * warps) {
        const uint8_t * row = w + (int64_t) r * w_row_stride;
        for (int m = 0; m < m_cols; ++m) {
            float acc = 0.f;
            for (int i = lane; i < k; i += 32) {
                float wv;
                if (DT == DT_F32) wv = __ldg((const float *) row + i);
                else wv = __half2float(__ldg((const __half *) row + i));
                acc = fmaf(wv, __ldcg(x + (int64_t) m * ldx + i), acc);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) y[(int64_t) m * ldy + r] = acc;
        }
    }
}

// ---- host dispatch ------------------------------------------------------------------------------------

// name of the kernel family the last matvec() call of this thread was served by (tests pin every dispatch branch by it)
static thread_local const char * t_last_kernel = "";
static int took(const char * name, int st) {
    t_last_kernel = name;
    return st;
}
const char * matvec_last_kernel() { return t_last_kernel; }
void matvec_note_kernel(const char * name) { t_last_kernel = name; }


template <class U>
static int launch_stream(cudaStream_t s, const void * w, int64_t k, int64_t n, const float * x, float * y) {
    const int upr = (int) (k / U::WEIGHTS);
    // threads: a whole number of rows per pass, 256..512 threads
    int rp = 1;
    while ((rp * 2) * upr <= U::MAX_THREADS) rp *= 2;
    const int threads = rp * upr;
    const Planes P = planes_for(U::DTYPE, n, k);
    // one wave: spread the rows over all SMs, rows per CTA a multiple of the rows per pass
    const int ctas_per_sm = threads <= 256 ? 2 : 1;
    const int64_t slots = (int64_t) sm_count() * ctas_per_sm;
    int64_t rows_per_cta = (n + slots - 1) / slots;
    rows_per_cta = (rows_per_cta + rp - 1) / rp * rp;
    const int64_t grid = (n + rows_per_cta - 1) / rows_per_cta;
    const size_t smem = (size_t) U::ROWS_IN_FLIGHT * (threads / 32) * sizeof(float);
    return launch(matvec_stream<U>, dim3((unsigned) grid), dim3(threads), smem, s, (const uint8_t *) w, P, x, y, (int) n, upr,
                  (int) rows_per_cta);
}

// tuning knobs of the wide kernel, overridable from the environment for experiments:
// SM100_MV_THREADS (target CTA size), SM100_MV_CTAS (CTAs per SM used to size the grid)
static int env_int(const char * name, int fallback) {
    const char * v = std::getenv(name);
    return v != nullptr && *v != '\0' ? std::atoi(v) : fallback;
}

template <class W>
static int launch_wide(cudaStream_t s, const void * w, int64_t k, int64_t n, const float * x, float * y) {
    static const int target_threads = env_int("SM100_MV_THREADS", 192);
    static const int ctas_per_sm = env_int("SM100_MV_CTAS", 2);
    const int upr = (int) (k / W::WEIGHTS);
    // a whole number of rows per pass; CTAs of at most 192 threads leave room for 168 registers per thread
    // at two CTAs per SM (64 activations + 4 rows of quants in flight do not fit in 128)
    const int rp = upr >= target_threads ? 1 : target_threads / upr;
    const int threads = rp * upr;
    const Planes P = planes_for(W::DTYPE, n, k);
    const int64_t slots = (int64_t) sm_count() * ctas_per_sm;
    int64_t rows_per_cta = (n + slots - 1) / slots;
    rows_per_cta = (rows_per_cta + rp - 1) / rp * rp;
    const int64_t grid = (n + rows_per_cta - 1) / rows_per_cta;
    const size_t smem = (size_t) 4 * (threads / 32) * sizeof(float);
    const uint8_t * wp = (const uint8_t *) w;
    if (threads <= 192) return launch(matvec_wide<W, 4, 192, 2>, dim3((unsigned) grid), dim3(threads), smem, s, wp, P, x, y, (int) n, upr, (int) rows_per_cta);
    if (threads <= 384) return launch(matvec_wide<W, 4, 384, 1>, dim3((unsigned) grid), dim3(threads), smem, s, wp, P, x, y, (int) n, upr, (int) rows_per_cta);
    return launch(matvec_wide<W, 4, 512, 1>, dim3((unsigned) grid), dim3(threads), smem, s, wp, P, x, y, (int) n, upr, (int) rows_per_cta);
}

template <class W>
static bool wide_ok(int64_t k, int64_t m) {
    const int64_t upr = k / W::WEIGHTS;
    return m == 1 && k % W::WEIGHTS == 0 && upr % 32 == 0 && upr <= 512;
}

template <class U, bool PACKED>
static int launch_rows(cudaStream_t s, const void * w, int64_t w_row_stride, int64_t k, int64_t n, const float * x, int64_t ldx,
                       int64_t m, float * y, int64_t ldy, int64_t row_begin = 0) {
    const int upr = (int) (k / U::WEIGHTS);
    Planes P = {};
    if (PACKED) P = planes_for(U::DTYPE, n, k);
    const int threads = 256, warps = threads / 32;
    int64_t grid = (n - row_begin + warps - 1) / warps;
    const int64_t cap = (int64_t) sm_count() * 8;
    if (grid > cap) grid = cap;
    const dim3 g((unsigned) grid), b(threads);
    const uint8_t * wp = (const uint8_t *) w;
#define SM100_ROWS_CASE(MM) \
    case MM: return launch(matvec_rows<U, MM, PACKED>, g, b, 0, s, wp, P, w_row_stride, x, ldx, y, ldy, (int) row_begin, (int) n, upr);
    switch (m) {
        SM100_ROWS_CASE(1) SM100_ROWS_CASE(2) SM100_ROWS_CASE(3) SM100_ROWS_CASE(4)
        SM100_ROWS_CASE(5) SM100_ROWS_CASE(6) SM100_ROWS_CASE(7) SM100_ROWS_CASE(8)
    }
#undef SM100_ROWS_CASE
    return fail(ST_INVALID, "matvec: M must be 1..8");
}

template <class U>
static int matvec_dispatch(cudaStream_t s, int layout, const void * w, int64_t w_row_stride, int64_t k, int64_t n, const float * x,
                           int64_t ldx, int64_t m, float * y, int64_t ldy) {
    const int upr = (int) (k / U::WEIGHTS);
    if (layout == LAYOUT_PACKED) {
        if (m == 1 && upr % 32 == 0 && upr <= U::MAX_THREADS) return took("matvec_stream", launch_stream<U>(s, w, k, n, x, y));
        return took("matvec_rows", launch_rows<U, true>(s, w, 0, k, n, x, ldx, m, y, ldy));
    }
    return took("matvec_rows_natural", launch_rows<U, false>(s, w, w_row_stride, k, n, x, ldx, m, y, ldy));
}

// Decode matvec entry used by sm100_mul_mat for m <= 8.  w_row_stride (bytes) only matters for the
// natural layout; 0 means dense rows.
int matvec(cudaStream_t s, int dtype, int layout, const void * w, int64_t w_row_stride, int64_t k, int64_t n, const float * x,
           int64_t ldx, int64_t m, float * y, int64_t ldy) {
    if (w == nullptr || x == nullptr || y == nullptr) return fail(ST_INVALID, "mul_mat: null tensor pointer");
    if (k <= 0 || n <= 0 || m <= 0) return fail(ST_INVALID, "mul_mat: K, N and M must be positive");
    if (n > INT32_MAX || k > INT32_MAX) return fail(ST_UNSUPPORTED, "mul_mat: dimension above 2^31");
    if (m > 8) return fail(ST_INVALID, "matvec: M must be 1..8");
    const int be = block_elems(dtype);
    if (be == 0) return fail(ST_UNSUPPORTED, "mul_mat: unsupported weight dtype %d", dtype);
    if (k % be != 0) return fail(ST_UNSUPPORTED, "mul_mat: quantized row length must be a multiple of the block size");
    if (w_row_stride == 0) w_row_stride = k / be * block_bytes(dtype);
    const bool x_aligned = ((uintptr_t) x & 15) == 0 && (m == 1 || (ldx % 4) == 0);
    if (layout == LAYOUT_PACKED && !is_quant(dtype)) return fail(ST_UNSUPPORTED, "mul_mat: only quantized weights have a packed layout");
    if (layout != LAYOUT_PACKED && layout != LAYOUT_NATURAL) return fail(ST_INVALID, "mul_mat: unknown layout %d", layout);
    if (is_quant(dtype) && !x_aligned) return fail(ST_UNSUPPORTED, "mul_mat: activations must be 16-byte aligned (columns too)");
    static const int use_imma = env_int("SM100_Q4K_IMMA", 1);
    if (use_imma && layout == LAYOUT_PACKED && dtype == DT_Q4_K && x_aligned && m == 1) {
        // the ring kernel (consecutive launches overlap; it declines unless the stream's last launch was such a matvec);
        // leftover rows take the row kernel
        bool handled = false;
        const int st = matvec_q4k_ring_multi(s, 1, &w, &n, k, x, &y, &handled, nullptr, nullptr);
        if (st != ST_OK) return st;
        if (handled) {
            const int64_t full = (n / 16) * 16;
            if (full < n) return took("matvec_q4k_ring+rows", launch_rows<UnitQ4K, true>(s, w, 0, k, n, x, ldx, m, y, ldy, full));
            return took("matvec_q4k_ring", ST_OK);
        }
    }
    if (use_imma && layout == LAYOUT_PACKED && dtype == DT_Q4_K && x_aligned && m <= 2) {
        // integer tensor-core kernel over the full 16-row tiles; leftover rows take the row kernel
        bool handled = false;
        const int st = matvec_q4k_imma_tiles(s, w, k, n, x, ldx, m, y, ldy, &handled);
        if (st != ST_OK) return st;
        if (handled) {
            const int64_t full = (n / 16) * 16;
            if (full < n) return took("matvec_q4k_imma+rows", launch_rows<UnitQ4K, true>(s, w, 0, k, n, x, ldx, m, y, ldy, full));
            if (m == 1) stream_tail_set(s, TAIL_Q4K_MATVEC);   // a second plain Q4_K matvec right behind this one starts a run of the ring kernel
            return took("matvec_q4k_imma", ST_OK);
        }
    }
    static const int use_b32 = env_int("SM100_B32_IMMA", 1);
    if (use_b32 && layout == LAYOUT_PACKED && (dtype == DT_Q4_0 || dtype == DT_Q8_0) && x_aligned && m == 1) {
        bool handled = false;
        const int st = matvec_b32_imma_tiles(s, dtype, w, k, n, x, y, &handled);
        if (st != ST_OK) return st;
        if (handled) {
            const int64_t full = (n / 16) * 16;
            if (full == n) return took("matvec_b32_imma", ST_OK);
            return took("matvec_b32_imma+rows", dtype == DT_Q4_0 ? launch_rows<UnitQ40, true>(s, w, 0, k, n, x, ldx, m, y, ldy, full)
                                                                 : launch_rows<UnitQ80, true>(s, w, 0, k, n, x, ldx, m, y, ldy, full));
        }
    }
    static const int use_q6k = env_int("SM100_Q6K_IMMA", 1);
    // measured: the tensor-core kernel wins on small tensors and on short rows (4096 x 4096: 1.9 vs 1.25 TB/s,
    // 4096 x 12288: 2.45 vs 2.29), the streaming kernel on long rows and large tensors (12288 x 4096: 2.98 vs 2.35,
    // vocabulary head: 4.1 vs 3.1 TB/s), where its lower instruction count per byte pays
    const int64_t q6k_limit = k <= 4096 ? (int64_t) 64 << 20 : (int64_t) 20 << 20;
    if (use_q6k && layout == LAYOUT_PACKED && dtype == DT_Q6_K && x_aligned && m == 1 && (use_q6k > 1 || n * k <= q6k_limit)) {
        bool handled = false;
        const int st = matvec_q6k_imma_tiles(s, w, k, n, x, y, &handled);
        if (st != ST_OK) return st;
        if (handled) {
            const int64_t full = (n / 16) * 16;
            return full == n ? took("matvec_q6k_imma", ST_OK) : took("matvec_q6k_imma+rows", launch_rows<UnitQ6K, true>(s, w, 0, k, n, x, ldx, m, y, ldy, full));
        }
    }
    if (use_imma && layout == LAYOUT_PACKED && dtype == DT_Q4_K && x_aligned && m >= 3) {
        // integer tensor-core kernel with the tokens in the B columns; when 8 columns do not fit shared memory, two passes of 4
        bool handled = false;
        int st = matvec_q4k_imma_cols_tiles(s, w, k, n, x, ldx, m, y, ldy, &handled);
        if (st != ST_OK) return st;
        if (!handled && m > 4) {
            st = matvec_q4k_imma_cols_tiles(s, w, k, n, x, ldx, 4, y, ldy, &handled);
            if (st != ST_OK) return st;
            if (handled) {
                bool second = false;
                const int64_t rest = m - 4;
                if (rest >= 3) st = matvec_q4k_imma_cols_tiles(s, w, k, n, x + 4 * ldx, ldx, rest, y + 4 * ldy, ldy, &second);
                else st = matvec_q4k_imma_tiles(s, w, k, n, x + 4 * ldx, ldx, rest, y + 4 * ldy, ldy, &second);
                if (st != ST_OK) return st;
                if (!second) return fail(ST_BACKEND, "mul_mat: the Q4_K column kernel accepted the first pass but not the second");
            }
        }
        if (handled) {
            const int64_t full = (n / 16) * 16;
            if (full < n) return took("matvec_q4k_imma_cols+rows", launch_rows<UnitQ4K, true>(s, w, 0, k, n, x, ldx, m, y, ldy, full));
            return took("matvec_q4k_imma_cols", ST_OK);
        }
    }
    static const int use_mma = env_int("SM100_Q4K_MMA", 1);
    if (use_mma && layout == LAYOUT_PACKED && dtype == DT_Q4_K && x_aligned) {
        // tensor-core tile kernel over the full 16-row tiles, up to 4 columns per pass; leftover rows take the row kernel
        bool all = true;
        int64_t width = k % 256 == 0 ? q4k_pass_width(k, m) : 0;
        if (width == 0) { all = false; width = 4; }
        for (int64_t c0 = 0; c0 < m && all; c0 += width) {
            const int64_t mm = m - c0 < width ? m - c0 : width;
            bool handled = false;
            const int st = matvec_q4k_tiles(s, w, k, n, x + c0 * ldx, ldx, mm, y + c0 * ldy, ldy, &handled);
            if (st != ST_OK) return st;
            if (!handled) {
                if (c0 != 0) return fail(ST_BACKEND, "mul_mat: the Q4_K tile kernel accepted the first column pass but not a later one");
                all = false;
            }
        }
        if (all) {
            const int64_t full = (n / 16) * 16;
            if (full < n) return took("matvec_q4k_mma+rows", launch_rows<UnitQ4K, true>(s, w, 0, k, n, x, ldx, m, y, ldy, full));
            return took("matvec_q4k_mma", ST_OK);
        }
    }
    // Q6_K with 2..8 columns: the tensor-core kernel assembles the 6-bit weights of a step once and multiplies them with every
    // column (measured on 4096 x 4096: 8 columns in 2.2 times the time of one, where eight single-column launches took 7.4 times)
    if (use_q6k && layout == LAYOUT_PACKED && dtype == DT_Q6_K && x_aligned && m >= 2 && m <= 8) {
        bool handled = false;
        const int st = matvec_q6k_imma_cols(s, w, k, n, x, ldx, (int) m, y, ldy, &handled);
        if (st != ST_OK) return st;
        if (handled) {
            const int64_t full = (n / 16) * 16;
            return full == n ? took("matvec_q6k_imma_cols", ST_OK) : took("matvec_q6k_imma_cols+rows", launch_rows<UnitQ6K, true>(s, w, 0, k, n, x, ldx, m, y, ldy, full));
        }
    }
    // Q6_K / Q4_0 / Q8_0 with 2..8 columns: the single-column tensor-core and wide kernels have no multi-column form yet,
    // and one launch of them per column (weights re-read per column, mostly from L2 for matrices below its size) is still
    // 2-3 times faster than the one-warp-per-row kernel that serves every column in one pass (measured on the sweep
    // shapes: Q6_K 4096 x 4096 at M = 2: 0.93 vs 0.35 TB/s of algorithmic bytes)
    if (layout == LAYOUT_PACKED && m > 1 && (dtype == DT_Q6_K || dtype == DT_Q4_0 || dtype == DT_Q8_0) && x_aligned && n >= 16 &&
        ((dtype == DT_Q6_K && k % 256 == 0) || (dtype != DT_Q6_K && k % 128 == 0))) {
        for (int64_t c = 0; c < m; ++c) {
            const int st = matvec(s, dtype, layout, w, w_row_stride, k, n, x + c * ldx, ldx, 1, y + c * ldy, ldy);
            if (st != ST_OK) return st;
        }
        return took("matvec_per_column", ST_OK);
    }
    static const int use_wide = env_int("SM100_MV_WIDE", 1);
    if (use_wide && layout == LAYOUT_PACKED) {
        switch (dtype) {
            case DT_Q6_K: if (wide_ok<WideQ6K>(k, m)) return took("matvec_wide", launch_wide<WideQ6K>(s, w, k, n, x, y)); break;
            case DT_Q4_0: if (wide_ok<WideQ40>(k, m)) return took("matvec_wide", launch_wide<WideQ40>(s, w, k, n, x, y)); break;
            case DT_Q8_0: if (wide_ok<WideQ80>(k, m)) return took("matvec_wide", launch_wide<WideQ80>(s, w, k, n, x, y)); break;
        }
    }
    switch (dtype) {
        case DT_Q4_K: return matvec_dispatch<UnitQ4K>(s, layout, w, w_row_stride, k, n, x, ldx, m, y, ldy);
        case DT_Q6_K: return matvec_dispatch<UnitQ6K>(s, layout, w, w_row_stride, k, n, x, ldx, m, y, ldy);
        case DT_Q4_0: return matvec_dispatch<UnitQ40>(s, layout, w, w_row_stride, k, n, x, ldx, m, y, ldy);
        case DT_Q8_0: return matvec_dispatch<UnitQ80>(s, layout, w, w_row_stride, k, n, x, ldx, m, y, ldy);
        case DT_F32:
        case DT_F16: {
            const int per = dtype == DT_F32 ? 4 : 8;
            const bool w_aligned = true;  // ld_u128_any handles any alignment
            if (x_aligned && w_aligned && k % per == 0) {
                if (dtype == DT_F32) return took("matvec_rows_f32", launch_rows<UnitF32, false>(s, w, w_row_stride, k, n, x, ldx, m, y, ldy));
                return took("matvec_rows_f16", launch_rows<UnitF16, false>(s, w, w_row_stride, k, n, x, ldx, m, y, ldy));
            }
            const int threads = 256, warps = 8;
            int64_t grid = (n + warps - 1) / warps;
            const int64_t cap = (int64_t) sm_count() * 8;
            if (grid > cap) grid = cap;
            t_last_kernel = "matvec_scalar";
            if (dtype == DT_F32)
                return launch(matvec_scalar<DT_F32>, dim3((unsigned) grid), dim3(threads), 0, s, (const uint8_t *) w, w_row_stride, x, ldx, y, ldy, (int) n, (int) k, (int) m);
            return launch(matvec_scalar<DT_F16>, dim3((unsigned) grid), dim3(threads), 0, s, (const uint8_t *) w, w_row_stride, x, ldx, y, ldy, (int) n, (int) k, (int) m);
        }
    }
    return fail(ST_UNSUPPORTED, "mul_mat: unsupported weight dtype %d", dtype);
}

}  // namespace sm100
