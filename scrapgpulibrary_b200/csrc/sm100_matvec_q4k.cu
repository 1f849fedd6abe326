// Q4_K decode MUL_MAT (1..4 activation columns per pass) on the warp-level tensor-core path of sm_100a.
//
// Why tensor cores for a matvec: on B200 the HBM stream delivers ~40 four-bit weights per SM per clock, and the
// integer/logic pipe that has to unpack them issues 64 lane-operations per clock.  A CUDA-core dot product needs
// more than one logic operation per weight (extract, convert), which caps it near half of the HBM roofline
// whatever the memory system does.  Here a nibble pair becomes a half2 with ONE logic operation
// ((w & 0x000F000F) | 0x64006400 is the half2 {1024 + n0, 1024 + n4}), the multiply-accumulate goes to
// mma.sync.m16n8k16 (f16 inputs, f32 accumulation), and the per-(row, sub-block) scale work is amortised over the
// 512 weights a warp-wide instruction covers.
//
// Values: the reference evaluates y[n] = sum_k (d*sc*q - dmin*m) * x[k] in f32 (src/core/ref/quant.cpp:55-82,
// src/core/ref/ops.cpp:891-984).  Here x[k] is split exactly into two f16 planes, x = hi + lo with
// hi = f16(x), lo = f16(x - hi) (22 significant bits), the integer quants are exact in f16, products are exact
// in f32, and every sum is an f32 accumulation: y = sum_sb d*sc * (q . hi + q . lo) - dmin*m * sum_sb(x).
// NMSE against the reference is ~1e-12.  Activations must be below 65504 in magnitude (f16 range).
//
// Work split: a CTA of 8 warps walks over 16-row tiles; for one row tile the warps split K in chunks of 512
// weights (8 tiles of 16 rows x 64 weights, two Q4_K blocks per row).  Weight tiles are 512 contiguous bytes in
// the packed layout (sm100_layout.h) and arrive with one 16-byte load per lane, prefetched one chunk ahead and
// issued before griddepcontrol.wait for the first chunk, so they overlap the predecessor kernel's tail.
#include "sm100_quant_units.cuh"

#include <cuda_fp16.h>

namespace sm100 {

constexpr int Q4K_WARPS = 8;                 // warps that share one row tile (they split K)
constexpr int Q4K_GROUPS = 2;                // row tiles a CTA works on at a time
constexpr int Q4K_THREADS = Q4K_WARPS * Q4K_GROUPS * 32;
constexpr int Q4K_TILES = 8;   // pair tiles (64 weights each) per chunk

struct Q4KArgs {
    const uint8_t * w;       // packed tensor base
    int64_t h_off;           // byte offset of the header plane
    const float * x;         // [K, M], column stride ldx floats
    float * y;               // [N, M], column stride ldy floats
    int64_t ldx, ldy;
    int n_tiles;             // full 16-row tiles
    int pairs;               // K / 64
    int blocks;              // K / 256
    int chunks;              // ceil(pairs / 8)
    int m;                   // activation columns, 1..4
};

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// first step of a sub-block: accumulator starts at zero (no register has to be cleared for it)
__device__ __forceinline__ void mma_16816_zero(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

// half2 of two nibbles as exact small integers: low-nibble positions (bits 0-3, 16-19) via the 1024 magic,
// high-nibble positions (bits 4-7, 20-23) via the 64 magic (one mantissa step of f16 at 64 is 1/16).  The magic
// constant is subtracted right away (exact in f16).  Leaving it in and removing C * sum(x) in the epilogue saves
// the subtraction but was measured to cost accuracy (NMSE 1e-7 instead of 1e-12: the tensor core's f32
// accumulation truncates the aligned products) and changed greedy tokens of the decode test, so it is not done.
__device__ __forceinline__ uint32_t nib_lo(uint32_t w) {
    const uint32_t h = (w & 0x000F000Fu) | 0x64006400u;
    const __half2 r = __hsub2(*reinterpret_cast<const __half2 *>(&h), __half2half2(__ushort_as_half(0x6400)));
    return *reinterpret_cast<const uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t nib_hi(uint32_t w) {
    const uint32_t h = (w & 0x00F000F0u) | 0x54005400u;
    const __half2 r = __hsub2(*reinterpret_cast<const __half2 *>(&h), __half2half2(__ushort_as_half(0x5400)));
    return *reinterpret_cast<const uint32_t *>(&r);
}

struct Q4KStage {
    uint4 a[Q4K_TILES];   // weight tiles of the chunk
    uint4 h;              // one block header per lane: row (lane & 15), block 2*chunk + (lane >> 4)
};

__device__ __forceinline__ void q4k_load_stage(const Q4KArgs & p, int rt, int chunk, int lane, Q4KStage & st) {
    const uint8_t * tiles = p.w + ((int64_t) rt * p.pairs + (int64_t) chunk * Q4K_TILES) * 512 + lane * 16;
#pragma unroll
    for (int j = 0; j < Q4K_TILES; ++j) {
        if (chunk * Q4K_TILES + j < p.pairs) st.a[j] = ldg_stream(tiles + j * 512);
        else st.a[j] = make_uint4(0, 0, 0, 0);
    }
    const int blk = 2 * chunk + (lane >> 4);
    if (blk < p.blocks) st.h = __ldg((const uint4 *) (p.w + p.h_off + (((int64_t) rt * 16 + (lane & 15)) * p.blocks + blk) * 16));
    else st.h = make_uint4(0, 0, 0, 0);
}

// f16 bit pattern -> f32 on the FMA pipe (exact for normal and subnormal halves)
__device__ __forceinline__ float h2f_fast(uint32_t h) {
    return __uint_as_float(((h & 0x8000u) << 16) | ((h & 0x7FFFu) << 13)) * 5.192296858534828e33f;
}

// Decodes one block header into (d*sc, dmin*m) for its 8 sub-blocks and stores them for the warp:
// sc_smem[(blk * 16 + row) * 4 + pair] = float4(d*sc_lo, dmin*m_lo, d*sc_hi, dmin*m_hi)
__device__ __forceinline__ void q4k_decode_header(const uint4 & h, float4 * dst) {
    const float d = h2f_fast(h.x & 0xFFFFu), dmin = h2f_fast(h.x >> 16);
    const uint32_t f[4] = {h.y, __funnelshift_r(h.y, h.z, 24), __funnelshift_r(h.z, h.w, 16), h.w >> 8};
#pragma unroll
    for (int pr = 0; pr < 4; ++pr) {
        // 6-bit fields to f32 without the conversion unit: or into the mantissa of 2^23, subtract 2^23
        const uint32_t lo = f[pr], up = f[pr] >> 12;
        const float s0 = __uint_as_float((lo & 63u) | 0x4B000000u) - 8388608.0f;
        const float m0 = (__uint_as_float((lo & 0xFC0u) | 0x4B000000u) - 8388608.0f) * 0.015625f;
        const float s1 = __uint_as_float((up & 63u) | 0x4B000000u) - 8388608.0f;
        const float m1 = (__uint_as_float((up & 0xFC0u) | 0x4B000000u) - 8388608.0f) * 0.015625f;
        dst[pr] = make_float4(d * s0, dmin * m0, d * s1, dmin * m1);
    }
}

// Shared memory of one CTA (byte offsets are 32-bit inside the hot loop):
//   xs    [pairs][2 sub-blocks][NCOL columns][4 lanes t] x 16 B   activations in B-fragment order; a zero block of
//                                                                the same per-pair size follows for the lanes whose
//                                                                fragment column holds no activation
//   sxs   [pairs][4] float2      sum of the 32 activations of the low / high sub-block, per activation column
//   scs   [warp][2 blocks][16 rows][4 pairs] float4   decoded (d*sc, dmin*m) of the warp's current chunk
//   red   [warp][16 rows][4 columns] float            partial outputs of the warps of one row tile
template <int M, bool FULL>
__global__ void __launch_bounds__(Q4K_THREADS, 1) matvec_q4k_mma(Q4KArgs p) {
    constexpr int NCOL = 2 * M;                 // B columns: (hi, lo) plane of each activation column
    constexpr uint32_t XS_PAIR = 2 * NCOL * 4;  // uint4 entries per pair tile
    extern __shared__ __align__(16) uint8_t smem[];
    uint4 * xs = reinterpret_cast<uint4 *>(smem);
    uint4 * xs_zero = xs + (uint32_t) p.pairs * XS_PAIR;
    float2 * sxs = reinterpret_cast<float2 *>(xs_zero + XS_PAIR);
    float4 * scs = reinterpret_cast<float4 *>(sxs + (uint32_t) p.pairs * 4);
    float * red = reinterpret_cast<float *>(scs + Q4K_WARPS * Q4K_GROUPS * 128);

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int group = wid / Q4K_WARPS, warp = wid % Q4K_WARPS;   // row-tile group of the CTA, K-split index inside it
    const int g = lane >> 2, t = lane & 3;

    // first chunk of weights: independent of the predecessor kernel
    Q4KStage cur, nxt;
    int rt = blockIdx.x * Q4K_GROUPS + group, chunk = warp;
    if (rt < p.n_tiles && chunk < p.chunks) q4k_load_stage(p, rt, chunk, lane, cur);

    pdl_wait();

    // activations -> f16 hi/lo planes in fragment order, plus per-sub-block sums.  One item = 4 consecutive
    // elements; the 8 items of a 32-element sub-block sit in 8 consecutive lanes.
    for (int i = tid; i < (int) XS_PAIR; i += Q4K_THREADS) xs_zero[i] = make_uint4(0, 0, 0, 0);
    for (int item = tid; item < p.pairs * 16; item += Q4K_THREADS) {
        const int c = item >> 4, sb = (item >> 3) & 1, q4 = item & 7, ks = q4 >> 2, tt = q4 & 3;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            if (m < M) {
                const float4 v = __ldcg(reinterpret_cast<const float4 *>(p.x + (int64_t) m * p.ldx + (int64_t) item * 4));   // coherent: the producer may still be running when this kernel starts
                // k-slots of the fragment: bytes (0, 2) -> b0b1, bytes (1, 3) -> b2b3
                const __half2 h02 = __floats2half2_rn(v.x, v.z), h13 = __floats2half2_rn(v.y, v.w);
                const float2 f02 = __half22float2(h02), f13 = __half22float2(h13);
                const __half2 l02 = __floats2half2_rn(v.x - f02.x, v.z - f02.y), l13 = __floats2half2_rn(v.y - f13.x, v.w - f13.y);
                uint2 * dh = reinterpret_cast<uint2 *>(xs + ((uint32_t) (c * 2 + sb) * NCOL + 2 * m) * 4 + tt) + ks;
                uint2 * dl = reinterpret_cast<uint2 *>(xs + ((uint32_t) (c * 2 + sb) * NCOL + 2 * m + 1) * 4 + tt) + ks;
                *dh = make_uint2(*reinterpret_cast<const uint32_t *>(&h02), *reinterpret_cast<const uint32_t *>(&h13));
                *dl = make_uint2(*reinterpret_cast<const uint32_t *>(&l02), *reinterpret_cast<const uint32_t *>(&l13));
                float s = (v.x + v.y) + (v.z + v.w);
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                s += __shfl_xor_sync(0xffffffffu, s, 4);
                if (q4 == 0) reinterpret_cast<float *>(sxs + (uint32_t) c * 4 + m)[sb] = s;
            } else if (q4 == 0) {
                reinterpret_cast<float *>(sxs + (uint32_t) c * 4 + m)[sb] = 0.f;
            }
        }
    }
    __syncthreads();
    pdl_launch_dependents();

    // per-lane views: lanes whose B-fragment column g carries no activation read the zero block (stride 0)
    const bool live = g < NCOL;
    const uint4 * xs_lane = live ? xs + g * 4 + t : xs_zero + t;
    const uint32_t xs_step = live ? XS_PAIR : 0u;
    const float2 * sx_lane = sxs + t;
    float4 * my_sc = scs + wid * 128;
    const float4 * sc_lane = my_sc + g * 4;
    float4 * sc_store = my_sc + ((lane >> 4) * 16 + (lane & 15)) * 4;
    const int rt_step = gridDim.x * Q4K_GROUPS;
    float * my_red = red + group * (Q4K_WARPS * 64);
    const int gtid = tid - group * (Q4K_WARPS * 32);

    // every group runs the same number of rounds so that the CTA-wide barriers match
    for (int round = blockIdx.x * Q4K_GROUPS; round < p.n_tiles; round += rt_step) {
        float acc0 = 0.f, acc1 = 0.f;   // rows g and g + 8 of the tile, activation column t
        for (; rt < p.n_tiles && chunk < p.chunks; chunk += Q4K_WARPS) {
            // prefetch the next work item of this warp
            int nrt = rt, nchunk = chunk + Q4K_WARPS;
            if (nchunk >= p.chunks) { nrt = rt + rt_step; nchunk = warp; }
            if (nrt < p.n_tiles && nchunk < p.chunks) q4k_load_stage(p, nrt, nchunk, lane, nxt);

            __syncwarp();
            q4k_decode_header(cur.h, sc_store);
            __syncwarp();

            const uint4 * xb = xs_lane + (uint32_t) (chunk * Q4K_TILES) * xs_step;
            const float2 * sxb = sx_lane + (uint32_t) (chunk * Q4K_TILES) * 4;
#pragma unroll
            for (int j = 0; j < Q4K_TILES; ++j) {
                if (FULL || chunk * Q4K_TILES + j < p.pairs) {
                    const uint32_t w0 = cur.a[j].x, w1 = cur.a[j].y, w2 = cur.a[j].z, w3 = cur.a[j].w;   // row g: k-step 0, 1; row g+8: k-step 0, 1
                    const uint32_t v0 = w0 >> 8, v1 = w1 >> 8, v2 = w2 >> 8, v3 = w3 >> 8;
                    const uint4 blo = xb[j * xs_step], bhi = xb[j * xs_step + NCOL * 4 * (live ? 1 : 0)];
                    float clo[4], chi[4];
                    {
                        const uint32_t a[4] = {nib_lo(w0), nib_lo(w2), nib_lo(v0), nib_lo(v2)};
                        mma_16816_zero(clo, a, blo.x, blo.y);
                        const uint32_t b[4] = {nib_hi(w0), nib_hi(w2), nib_hi(v0), nib_hi(v2)};
                        mma_16816_zero(chi, b, bhi.x, bhi.y);
                    }
                    {
                        const uint32_t a[4] = {nib_lo(w1), nib_lo(w3), nib_lo(v1), nib_lo(v3)};
                        mma_16816(clo, a, blo.z, blo.w);
                        const uint32_t b[4] = {nib_hi(w1), nib_hi(w3), nib_hi(v1), nib_hi(v3)};
                        mma_16816(chi, b, bhi.z, bhi.w);
                    }
                    // columns 2t, 2t+1 of the fragment are the hi and lo planes of activation column t
                    const float4 s0 = sc_lane[(j >> 2) * 64 + (j & 3)];
                    const float4 s1 = sc_lane[(j >> 2) * 64 + 32 + (j & 3)];
                    const float2 sx = sxb[j * 4];
                    acc0 += s0.x * (clo[0] + clo[1]) - s0.y * sx.x + s0.z * (chi[0] + chi[1]) - s0.w * sx.y;
                    acc1 += s1.x * (clo[2] + clo[3]) - s1.y * sx.x + s1.z * (chi[2] + chi[3]) - s1.w * sx.y;
                }
            }
            cur = nxt;
        }
        // partial sums of this warp's K chunks -> shared; 16 rows x 4 columns reduced over the warps
        my_red[(warp * 16 + g) * 4 + t] = acc0;
        my_red[(warp * 16 + g + 8) * 4 + t] = acc1;
        __syncthreads();
        if (gtid < 64 && rt < p.n_tiles) {
            const int row = gtid >> 2, col = gtid & 3;
            if (col < M) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < Q4K_WARPS; ++w) v += my_red[(w * 16 + row) * 4 + col];
                p.y[(int64_t) col * p.ldy + (int64_t) rt * 16 + row] = v;
            }
        }
        __syncthreads();
        rt += rt_step;
        chunk = warp;
    }
}

size_t q4k_smem_bytes(int pairs, int m) {
    return (size_t) (pairs + 1) * 2 * (2 * m) * 4 * 16 + (size_t) pairs * 4 * 8 + (size_t) Q4K_WARPS * Q4K_GROUPS * 128 * 16 +
           (size_t) Q4K_WARPS * Q4K_GROUPS * 16 * 4 * 4;
}

// widest column pass (4, 2 or 1 activation columns) whose activation planes fit in shared memory; 0 if none does
int q4k_pass_width(int64_t k, int64_t m) {
    for (int w = 4; w >= 1; --w) {
        const int cols = w < m ? w : (int) m;
        if (q4k_smem_bytes((int) (k / 64), cols) <= (size_t) 227 * 1024) return w;
    }
    return 0;
}

template <int M, bool FULL>
static int launch_q4k_one(cudaStream_t s, const Q4KArgs & a, size_t smem, int grid) {
    if (smem > 48 * 1024) {
        // raising the limit is idempotent and per device: repeat it rather than remember which devices saw it
        SM100_CUDA(cudaFuncSetAttribute(matvec_q4k_mma<M, FULL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    }
    return launch(matvec_q4k_mma<M, FULL>, dim3((unsigned) grid), dim3(Q4K_THREADS), smem, s, a);
}

template <int M>
static int launch_q4k(cudaStream_t s, const Q4KArgs & a, size_t smem, int grid) {
    return a.pairs % Q4K_TILES == 0 ? launch_q4k_one<M, true>(s, a, smem, grid) : launch_q4k_one<M, false>(s, a, smem, grid);
}

// Q4_K packed matvec over the full 16-row tiles of the tensor; returns ST_UNSUPPORTED (without an error message
// change) when the shape does not fit the kernel so that the caller can take the generic path.
int matvec_q4k_tiles(cudaStream_t s, const void * w, int64_t k, int64_t n, const float * x, int64_t ldx, int64_t m, float * y, int64_t ldy,
                     bool * handled) {
    *handled = false;
    const int64_t tiles = n / 16;
    if (tiles == 0 || m < 1 || m > 4 || k % 256 != 0 || k / 64 > 4096) return ST_OK;
    const int pairs = (int) (k / 64);
    const size_t smem = q4k_smem_bytes(pairs, (int) m);
    if (smem > 227 * 1024) return ST_OK;
    if (((uintptr_t) w & 15) != 0 || ((uintptr_t) x & 15) != 0 || (m > 1 && (ldx & 3) != 0)) return ST_OK;
    Q4KArgs a;
    a.w = (const uint8_t *) w;
    a.h_off = n * (k / 256) * 128;
    a.x = x;
    a.y = y;
    a.ldx = ldx;
    a.ldy = ldy;
    a.n_tiles = (int) tiles;
    a.pairs = pairs;
    a.blocks = (int) (k / 256);
    a.chunks = (pairs + Q4K_TILES - 1) / Q4K_TILES;
    a.m = (int) m;
    int64_t grid = sm_count();   // one CTA per SM: the activation planes are prepared once per SM
    const int64_t rounds = (tiles + Q4K_GROUPS - 1) / Q4K_GROUPS;
    if (grid > rounds) grid = rounds;
    int st;
    switch (m) {
        case 1: st = launch_q4k<1>(s, a, smem, (int) grid); break;
        case 2: st = launch_q4k<2>(s, a, smem, (int) grid); break;
        case 3: st = launch_q4k<3>(s, a, smem, (int) grid); break;
        default: st = launch_q4k<4>(s, a, smem, (int) grid); break;
    }
    *handled = st == ST_OK;
    return st;
}

}  // namespace sm100
