// Q4_0 / Q8_0 decode MUL_MAT (one activation column) on the integer tensor-core path, packed layout.
//
// Same idea as the Q4_K kernel (sm100_matvec_q4k_imma.cu): activations become 16-bit integers (two signed-byte
// planes h, l and one f32 scale per 32-element block), the weights' integers go straight into
// mma.sync.m16n8k32 (u8 x s8 for Q4_0 nibbles, s8 x s8 for Q8_0), and the per-block scale is applied to an exact
// integer dot product:   y[n] = sum_b d[n,b] s_b ((256 H + L) - 8 Sx_b)      (the -8 Sx_b term only for Q4_0;
// values as src/core/ref/quant.cpp:30-52 and src/core/ref/ops.cpp:891-984 of the reference, NMSE ~1e-9).
//
// The packed layout keeps a row's blocks contiguous (sm100_layout.h), which does not look like an A fragment, but
// the summation index of an MMA is free: a warp takes 16 rows x 4 blocks, lane (g, t) loads the whole block t of
// rows g and g + 8 (64 / 128 contiguous bytes per row across the four lanes), and in MMA j (j = 0..3) it feeds the
// j-th word of that block into "its" eight k-slots.  One MMA therefore mixes four blocks - they are kept apart by
// the B operand: column 2c (2c + 1) holds the h (l) plane of block c's activations in block c's k-slots and zeros
// elsewhere, so after the four MMAs lane (g, t) holds the integer dot products of block t for rows g and g + 8.
// Which lanes supply zeros is fixed per lane (t != g / 2), so there is no per-tile selection.
#include "sm100_quant_units.cuh"

#include <cstdlib>

namespace sm100 {

namespace {

constexpr int BQ_WARPS = 8;    // warps that share one row tile (they split K)
constexpr int BQ_GROUPS = 2;   // row tiles a CTA works on at a time
constexpr int BQ_THREADS = BQ_WARPS * BQ_GROUPS * 32;

struct BqArgs {
    const uint8_t * w;   // packed tensor base: quant plane, then the f16 scale plane
    int64_t d_off;       // byte offset of the scale plane
    const float * x;
    float * y;
    int n_tiles;         // full 16-row tiles
    int blocks;          // K / 32
    int quads;           // K / 128
};

__device__ __forceinline__ void bq_imma_u8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void bq_imma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// weights of one (row, block): Q4_0 4 words (16 bytes of nibble pairs), Q8_0 8 words
template <bool Q8>
struct BqBlock {
    uint32_t w[Q8 ? 8 : 4];
};

template <bool Q8>
__device__ __forceinline__ void bq_load(BqBlock<Q8> & b, const uint8_t * p) {
    if (Q8) {
        asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"   // 32-byte aligned: tensor base is
                     : "=r"(b.w[0]), "=r"(b.w[1]), "=r"(b.w[2]), "=r"(b.w[3]), "=r"(b.w[4]), "=r"(b.w[5]), "=r"(b.w[6]), "=r"(b.w[7])
                     : "l"(p));
    } else {
        const uint4 v = ldg_stream(p);
        b.w[0] = v.x; b.w[1] = v.y; b.w[2] = v.z; b.w[3] = v.w;
    }
}

// activations -> 16-bit integers per 32-element block (shared by the kernels below); the caller synchronises the CTA
__device__ __forceinline__ void bq_quantize_x(const BqArgs & p, uint32_t * xq, float2 * xs, int tid) {
    // activations -> 16-bit integers per 32-element block.  One item = 4 consecutive elements; the 8 items of a
    // block sit in 8 consecutive lanes.
    if (tid < 16) xq[p.blocks * 16 + tid] = 0u;
    // all loads of a batch are issued before the first one is used: one L2 latency per batch, not per trip
    constexpr int BATCH = 6;
    for (int base = 0; base < p.blocks * 8; base += BATCH * BQ_THREADS) {
        float4 xv[BATCH];
#pragma unroll
        for (int i = 0; i < BATCH; ++i) {
            const int it = base + i * BQ_THREADS + tid;
            if (it < p.blocks * 8) xv[i] = __ldcg(reinterpret_cast<const float4 *>(p.x) + it);   // coherent: the producer may still be running when this kernel starts
        }
#pragma unroll
        for (int i = 0; i < BATCH; ++i) {
            const int it = base + i * BQ_THREADS + tid;
            if (it >= p.blocks * 8) continue;   // warp-uniform: the item count is a multiple of 32
            const float4 v = xv[i];
            const int sb = it >> 3, q = it & 7;
            uint32_t amax_bits = act_abs_bits(v);
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, o));
            float inv, s;
            act_group_scale(amax_bits, inv, s);
            // round to nearest (even) without the conversion unit: 1.5 * 2^23 + x keeps the integer in the mantissa (|x| <= 32512)
        const int x0 = __float_as_int(fmaf(v.x, inv, 12582912.0f)) - 0x4B400000, x1 = __float_as_int(fmaf(v.y, inv, 12582912.0f)) - 0x4B400000,
                  x2 = __float_as_int(fmaf(v.z, inv, 12582912.0f)) - 0x4B400000, x3 = __float_as_int(fmaf(v.w, inv, 12582912.0f)) - 0x4B400000;
            int isum = (x0 + x1) + (x2 + x3);
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) isum += __shfl_xor_sync(0xffffffffu, isum, o);
            // 16-bit integer = 256 h + l with h, l signed bytes: h = (x + 128) >> 8, l = low byte of x
            const int h0 = (x0 + 128) >> 8, h1 = (x1 + 128) >> 8, h2 = (x2 + 128) >> 8, h3 = (x3 + 128) >> 8;
            xq[sb * 16 + q] = __byte_perm(__byte_perm((uint32_t) h0, (uint32_t) h1, 0x0040), __byte_perm((uint32_t) h2, (uint32_t) h3, 0x0040), 0x5410);
            xq[sb * 16 + 8 + q] = __byte_perm(__byte_perm((uint32_t) x0, (uint32_t) x1, 0x0040), __byte_perm((uint32_t) x2, (uint32_t) x3, 0x0040), 0x5410);
            if (q == 0) xs[sb] = make_float2(s, 8.0f * (float) isum);
        }
    }
}

// Shared memory of one CTA:
//   xq   [K/32][2 planes][32 B]   quantized activations, natural order inside a block; 64 zero bytes follow
//   xs   [K/32] float2            (s_b, 8 * sum of the block's integers as float - Q4_0's offset term)
//   red  [warp][16 rows] float    partial outputs of the warps of one row tile
template <bool Q8>
__global__ void __launch_bounds__(BQ_THREADS, 1) matvec_b32_imma(BqArgs p) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t * xq = reinterpret_cast<uint32_t *>(smem);
    float2 * xs = reinterpret_cast<float2 *>(smem + (size_t) p.blocks * 64 + 64);
    float * red = reinterpret_cast<float *>(xs + p.blocks);
    constexpr int BB = Q8 ? 32 : 16;   // quant bytes per block

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int group = wid / BQ_WARPS, warp = wid % BQ_WARPS;
    const int g = lane >> 2, t = lane & 3;
    const int rt_step = gridDim.x * BQ_GROUPS;
    const uint32_t row_bytes = (uint32_t) p.blocks * BB;

    // first quad of weights: independent of the predecessor kernel
    BqBlock<Q8> cur0, cur1, nxt0, nxt1;   // rows g and g + 8
    uint32_t cur_d = 0, nxt_d = 0;
    int rt = blockIdx.x * BQ_GROUPS + group, quad = warp;
    auto load = [&](int rt_, int quad_, BqBlock<Q8> & b0, BqBlock<Q8> & b1, uint32_t & dd) {
        const int blk = quad_ * 4 + t;
        const uint8_t * q0 = p.w + ((int64_t) rt_ * 16 + g) * row_bytes + (uint32_t) blk * BB;
        bq_load<Q8>(b0, q0);
        bq_load<Q8>(b1, q0 + 8 * (int64_t) row_bytes);
        const unsigned short * dp = reinterpret_cast<const unsigned short *>(p.w + p.d_off) + ((int64_t) rt_ * 16 + g) * p.blocks + blk;
        dd = (uint32_t) __ldg(dp) | (uint32_t) __ldg(dp + 8 * (int64_t) p.blocks) << 16;
    };
    if (rt < p.n_tiles && quad < p.quads) load(rt, quad, cur0, cur1, cur_d);

    pdl_wait();

    bq_quantize_x(p, xq, xs, tid);
    __syncthreads();
    pdl_launch_dependents();

    // B operand: lane (g, t) supplies column g; it is block t's plane (g & 1) when t == g / 2 and zero otherwise.
    // Dead lanes read the zero bytes and do not advance.
    const bool live = t == (g >> 1);
    const uint4 * xq_lane = reinterpret_cast<const uint4 *>(xq) + (live ? (t * 4 + (g & 1) * 2) : p.blocks * 4);
    const uint32_t xq_step = live ? 16u : 0u;   // uint4 units per quad (4 blocks x 64 B)
    float * my_red = red + group * (BQ_WARPS * 16);
    const int gtid = tid - group * (BQ_WARPS * 32);

    // every group runs the same number of rounds so that the CTA-wide barriers match
    for (int round = blockIdx.x * BQ_GROUPS; round < p.n_tiles; round += rt_step) {
        float acc0 = 0.f, acc1 = 0.f;   // rows g and g + 8, this lane's blocks
        for (; rt < p.n_tiles && quad < p.quads; quad += BQ_WARPS) {
            int nrt = rt, nquad = quad + BQ_WARPS;
            if (nquad >= p.quads) { nrt = rt + rt_step; nquad = warp; }
            if (nrt < p.n_tiles && nquad < p.quads) load(nrt, nquad, nxt0, nxt1, nxt_d);

            const uint4 bx0 = xq_lane[(uint32_t) quad * xq_step], bx1 = xq_lane[(uint32_t) quad * xq_step + 1];   // k 0..15 and 16..31 of the block
            const uint32_t blo[4] = {bx0.x, bx0.y, bx0.z, bx0.w}, bhi[4] = {bx1.x, bx1.y, bx1.z, bx1.w};
            int c[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (Q8) {
                    bq_imma_s8(c, cur0.w[j], cur1.w[j], cur0.w[4 + j], cur1.w[4 + j], blo[j], bhi[j]);
                } else {
                    // byte i of a block holds weight i (low nibble) and weight 16 + i (high nibble)
                    bq_imma_u8(c, cur0.w[j] & 0x0F0F0F0Fu, cur1.w[j] & 0x0F0F0F0Fu, (cur0.w[j] >> 4) & 0x0F0F0F0Fu, (cur1.w[j] >> 4) & 0x0F0F0F0Fu,
                               blo[j], bhi[j]);
                }
            }
            // columns 2t, 2t + 1 of this lane: (H, L) of block t
            const float2 sq = xs[quad * 4 + t];
            const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&cur_d));
            float v0 = (float) (c[0] * 256 + c[1]), v1 = (float) (c[2] * 256 + c[3]);
            if (!Q8) { v0 -= sq.y; v1 -= sq.y; }
            acc0 = fmaf(dd.x * sq.x, v0, acc0);
            acc1 = fmaf(dd.y * sq.x, v1, acc1);
            cur0 = nxt0; cur1 = nxt1; cur_d = nxt_d;
        }
        acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
        acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
        acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
        acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
        if (t == 0) {
            my_red[warp * 16 + g] = acc0;
            my_red[warp * 16 + g + 8] = acc1;
        }
        __syncthreads();
        if (gtid < 16 && rt < p.n_tiles) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < BQ_WARPS; ++w) v += my_red[w * 16 + gtid];
            p.y[(int64_t) rt * 16 + gtid] = v;
        }
        __syncthreads();
        rt += rt_step;
        quad = warp;
    }
}

// The same product with BQ_DEPTH steps (16 rows x 4 blocks each) of a warp in flight in registers instead of two: a
// slot is refilled as soon as its step has been multiplied, and the first BQ_DEPTH steps are requested before the
// dependency wait.  With two steps a CTA has 16 KB (Q4_0) on its way, which is half of what the HBM latency asks for.
// Needs a whole number of BQ_DEPTH-step batches per warp and row tile: K a multiple of 128 * BQ_WARPS * BQ_DEPTH.
constexpr int BQ_DEPTH = 4;

template <bool Q8>
__global__ void __launch_bounds__(BQ_THREADS, 1) matvec_b32_imma_deep(BqArgs p) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t * xq = reinterpret_cast<uint32_t *>(smem);
    float2 * xs = reinterpret_cast<float2 *>(smem + (size_t) p.blocks * 64 + 64);
    float * red = reinterpret_cast<float *>(xs + p.blocks);
    constexpr int BB = Q8 ? 32 : 16;   // quant bytes per block

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int group = wid / BQ_WARPS, warp = wid % BQ_WARPS;
    const int g = lane >> 2, t = lane & 3;
    const int rt_step = gridDim.x * BQ_GROUPS;
    const uint32_t row_bytes = (uint32_t) p.blocks * BB;

    BqBlock<Q8> s0[BQ_DEPTH], s1[BQ_DEPTH];   // rows g and g + 8 of the steps in flight
    uint32_t sd[BQ_DEPTH];
    auto load = [&](int rt_, int quad_, BqBlock<Q8> & b0, BqBlock<Q8> & b1, uint32_t & dd) {
        const int blk = quad_ * 4 + t;
        const uint8_t * q0 = p.w + ((int64_t) rt_ * 16 + g) * row_bytes + (uint32_t) blk * BB;
        bq_load<Q8>(b0, q0);
        bq_load<Q8>(b1, q0 + 8 * (int64_t) row_bytes);
        const unsigned short * dp = reinterpret_cast<const unsigned short *>(p.w + p.d_off) + ((int64_t) rt_ * 16 + g) * p.blocks + blk;
        dd = (uint32_t) __ldg(dp) | (uint32_t) __ldg(dp + 8 * (int64_t) p.blocks) << 16;
    };
    // load cursor: runs BQ_DEPTH steps ahead of the multiply over the same (row tile, quad) sequence
    int lrt = blockIdx.x * BQ_GROUPS + group, lquad = warp;
    auto advance = [&]() {
        lquad += BQ_WARPS;
        if (lquad >= p.quads) { lquad = warp; lrt += rt_step; }
    };
#pragma unroll
    for (int i = 0; i < BQ_DEPTH; ++i) {
        if (lrt < p.n_tiles) load(lrt, lquad, s0[i], s1[i], sd[i]);
        advance();
    }

    pdl_wait();
    bq_quantize_x(p, xq, xs, tid);
    __syncthreads();
    pdl_launch_dependents();

    const bool live = t == (g >> 1);
    const uint4 * xq_lane = reinterpret_cast<const uint4 *>(xq) + (live ? (t * 4 + (g & 1) * 2) : p.blocks * 4);
    const uint32_t xq_step = live ? 16u : 0u;
    float * my_red = red + group * (BQ_WARPS * 16);
    const int gtid = tid - group * (BQ_WARPS * 32);

    int rt = blockIdx.x * BQ_GROUPS + group;
    for (int round = blockIdx.x * BQ_GROUPS; round < p.n_tiles; round += rt_step) {
        float acc0 = 0.f, acc1 = 0.f;
        if (rt < p.n_tiles) {
            for (int quad = warp; quad < p.quads; quad += BQ_WARPS * BQ_DEPTH) {
#pragma unroll
                for (int i = 0; i < BQ_DEPTH; ++i) {
                    const int q = quad + i * BQ_WARPS;
                    const uint4 bx0 = xq_lane[(uint32_t) q * xq_step], bx1 = xq_lane[(uint32_t) q * xq_step + 1];
                    const uint32_t blo[4] = {bx0.x, bx0.y, bx0.z, bx0.w}, bhi[4] = {bx1.x, bx1.y, bx1.z, bx1.w};
                    int c[4] = {0, 0, 0, 0};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (Q8) {
                            bq_imma_s8(c, s0[i].w[j], s1[i].w[j], s0[i].w[4 + j], s1[i].w[4 + j], blo[j], bhi[j]);
                        } else {
                            bq_imma_u8(c, s0[i].w[j] & 0x0F0F0F0Fu, s1[i].w[j] & 0x0F0F0F0Fu, (s0[i].w[j] >> 4) & 0x0F0F0F0Fu,
                                       (s1[i].w[j] >> 4) & 0x0F0F0F0Fu, blo[j], bhi[j]);
                        }
                    }
                    const float2 sq = xs[q * 4 + t];
                    const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&sd[i]));
                    float v0 = (float) (c[0] * 256 + c[1]), v1 = (float) (c[2] * 256 + c[3]);
                    if (!Q8) { v0 -= sq.y; v1 -= sq.y; }
                    acc0 = fmaf(dd.x * sq.x, v0, acc0);
                    acc1 = fmaf(dd.y * sq.x, v1, acc1);
                    // the slot is free: its step BQ_DEPTH ahead goes in
                    if (lrt < p.n_tiles) load(lrt, lquad, s0[i], s1[i], sd[i]);
                    advance();
                }
            }
        }
        acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
        acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
        acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
        acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
        if (t == 0) {
            my_red[warp * 16 + g] = acc0;
            my_red[warp * 16 + g + 8] = acc1;
        }
        __syncthreads();
        if (gtid < 16 && rt < p.n_tiles) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < BQ_WARPS; ++w) v += my_red[w * 16 + gtid];
            p.y[(int64_t) rt * 16 + gtid] = v;
        }
        __syncthreads();
        rt += rt_step;
    }
}

size_t bq_smem_bytes(int blocks) { return (size_t) blocks * 64 + 64 + (size_t) blocks * 8 + (size_t) BQ_WARPS * BQ_GROUPS * 16 * 4; }

template <bool Q8>
int launch_bq(cudaStream_t s, const BqArgs & a, size_t smem, int grid) {
    static const int deep_ok = [] { const char * e = getenv("SM100_B32_DEEP"); return e != nullptr ? atoi(e) : 1; }();
    if (deep_ok && a.quads % (BQ_WARPS * BQ_DEPTH) == 0) {
        if (smem > 48 * 1024) SM100_CUDA(cudaFuncSetAttribute(matvec_b32_imma_deep<Q8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        return launch(matvec_b32_imma_deep<Q8>, dim3((unsigned) grid), dim3(BQ_THREADS), smem, s, a);
    }
    if (smem > 48 * 1024) SM100_CUDA(cudaFuncSetAttribute(matvec_b32_imma<Q8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    return launch(matvec_b32_imma<Q8>, dim3((unsigned) grid), dim3(BQ_THREADS), smem, s, a);
}

}  // namespace

// Q4_0 / Q8_0 packed matvec, one activation column, over the full 16-row tiles of the tensor; *handled = false
// when the shape is left to the caller's other kernels.
int matvec_b32_imma_tiles(cudaStream_t s, int dtype, const void * w, int64_t k, int64_t n, const float * x, float * y, bool * handled) {
    *handled = false;
    const int64_t tiles = n / 16;
    if (tiles == 0 || k % 128 != 0 || k > (int64_t) 1 << 20 || tiles > INT32_MAX / 2) return ST_OK;
    if (dtype != DT_Q4_0 && dtype != DT_Q8_0) return ST_OK;
    if (((uintptr_t) w & 31) != 0 || ((uintptr_t) x & 15) != 0) return ST_OK;
    const int blocks = (int) (k / 32);
    const size_t smem = bq_smem_bytes(blocks);
    if (smem > (size_t) 227 * 1024) return ST_OK;
    BqArgs a;
    a.w = (const uint8_t *) w;
    a.d_off = n * (int64_t) blocks * (dtype == DT_Q8_0 ? 32 : 16);
    a.x = x;
    a.y = y;
    a.n_tiles = (int) tiles;
    a.blocks = blocks;
    a.quads = blocks / 4;
    int64_t grid = sm_count();
    const int64_t rounds = (tiles + BQ_GROUPS - 1) / BQ_GROUPS;
    if (grid > rounds) grid = rounds;
    const int st = dtype == DT_Q8_0 ? launch_bq<true>(s, a, smem, (int) grid) : launch_bq<false>(s, a, smem, (int) grid);
    *handled = st == ST_OK;
    return st;
}

}  // namespace sm100
