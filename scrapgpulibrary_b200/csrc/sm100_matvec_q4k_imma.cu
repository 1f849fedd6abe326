// Q4_K decode MUL_MAT for 1 or 2 activation columns on the integer tensor-core path (mma.sync u8 x s8 -> s32).
//
// The decode matvec is bound by how many instructions it spends per weight, not by arithmetic: HBM delivers
// about 40 four-bit weights per SM per clock, so a kernel that wants the HBM roofline has roughly one warp
// instruction per 10 weights to spend.  This kernel needs about 32 warp instructions per 1024 weights:
//
//  * a 16-row x 64-weight tile of the packed layout (sm100_layout.h) is one 16-byte load per lane and already has
//    the register order of the A fragment of mma.m16n8k32: `w & 0x0F0F0F0F` IS the fragment of the low-nibble
//    sub-block, `w & 0xF0F0F0F0` the fragment of the high-nibble sub-block times 16 - two logic operations per
//    eight weights, no conversion;
//  * activations are quantized once per CTA to 16-bit integers with one f32 scale per 32 elements
//    (x ~ s_b (256 h + l), h and l signed bytes), which keeps 15 bits below each sub-block's largest element:
//    NMSE of the product is ~1e-9, far inside the 1e-6 the reference asks of a device
//    (tests/ops/ops_tests.cpp:725 of the reference);
//  * the h and l planes of the four pairs of one 256-weight block sit in different columns of the B fragment
//    (pair p in columns 2p, 2p+1), so that after the eight MMAs of a block every lane holds the exact integer
//    dot products of ITS sub-blocks (2t, 2t+1 of rows g and g+8) and the per-sub-block scale work
//    (d sc s_b (256 H + L) - dmin m sum(x), src/core/ref/quant.cpp:55-82) is spread over all 32 lanes instead of
//    being repeated by them.  Lane t of a row needs exactly the t-th 24-bit scale field of the packed header.
//
// Work split as in the f16 kernel: a CTA of 16 warps = 2 row-tile groups x 8 warps that split K in chunks of two
// blocks; weight tiles are prefetched one chunk ahead and the first chunk is issued before griddepcontrol.wait.
#include "sm100_quant_units.cuh"

namespace sm100 {

namespace {

constexpr int IQ_WARPS = 8;    // warps that share one row tile (they split K)
constexpr int IQ_GROUPS = 2;   // row tiles a CTA works on at a time
constexpr int IQ_THREADS = IQ_WARPS * IQ_GROUPS * 32;
constexpr int IQ_TILES = 8;    // pair tiles (64 weights each) per chunk = two 256-weight blocks

struct IqArgs {
    const uint8_t * w;   // packed tensor base
    int64_t h_off;       // byte offset of the header plane
    const float * x;     // [K, M], column stride ldx floats
    float * y;           // [N, M], column stride ldy floats
    int64_t ldx, ldy;
    int n_tiles;         // full 16-row tiles
    int pairs;           // K / 64
    int blocks;          // K / 256
    int chunks;          // ceil(blocks / 2)
};

__device__ __forceinline__ void imma_16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct IqStage {
    uint4 a[IQ_TILES];   // weight tiles of the chunk
    uint4 h;             // one block header per lane: row (lane & 15), block 2 * chunk + (lane >> 4)
};

__device__ __forceinline__ void iq_load_stage(const IqArgs & p, int rt, int chunk, int lane, IqStage & st) {
    const uint8_t * tiles = p.w + ((int64_t) rt * p.pairs + (int64_t) chunk * IQ_TILES) * 512 + lane * 16;
#pragma unroll
    for (int j = 0; j < IQ_TILES; ++j) {
        if (chunk * IQ_TILES + j < p.pairs) st.a[j] = ldg_stream(tiles + j * 512);
        else st.a[j] = make_uint4(0, 0, 0, 0);
    }
    const int blk = 2 * chunk + (lane >> 4);
    if (blk < p.blocks) st.h = __ldg((const uint4 *) (p.w + p.h_off + (((int64_t) rt * 16 + (lane & 15)) * p.blocks + blk) * 16));
    else st.h = make_uint4(0, 0, 0, 0);
}

// One row's share of a block for lane t: header words -> d, dmin and the scale field of sub-blocks 2t, 2t+1;
// clo / chi = (H, L) integer dot products of the low / high nibble sub-block (chi carries a factor 16).
// sq = (s_2t, sum_x_2t, s_2t+1, sum_x_2t+1).
__device__ __forceinline__ float iq_row_term(const uint4 & h, int t, int clo_h, int clo_l, int chi_h, int chi_l, const float4 & sq) {
    const __half2 dd = *reinterpret_cast<const __half2 *>(&h.x);
    const float2 df = __half22float2(dd);   // d, dmin
    // the 24-bit field t starts at bit 24 t of the 96-bit string (h.y, h.z, h.w)
    const uint32_t lo = t < 2 ? h.y : (t == 2 ? h.z : h.w);
    const uint32_t hi = t == 1 ? h.z : h.w;
    const uint32_t f = __funnelshift_r(lo, hi, (24 * t) & 31);
    const int sc0 = (int) (f & 63u), m0 = (int) ((f >> 6) & 63u), sc1 = (int) ((f >> 12) & 63u), m1 = (int) ((f >> 18) & 63u);
    const int v0 = clo_h * 256 + clo_l;          // exact: |v0| < 2^24
    const int v1 = (chi_h * 256 + chi_l) >> 4;   // exact: every term is a multiple of 16
    const float dot = fmaf((float) (v1 * sc1), sq.z, (float) (v0 * sc0) * sq.x);
    const float mins = fmaf((float) m1, sq.w, (float) m0 * sq.y);
    return fmaf(df.x, dot, -df.y * mins);
}

// Shared memory of one CTA:
//   xq   [M][K/32][64 B]      quantized activations in B-fragment order: per sub-block the h plane then the l plane,
//                             each as [t][b0 (k = 4t..4t+3), b1 (k = 16+4t..)] bytes
//   xs   [M][K/64] float4     (s, sum x) of the low and of the high sub-block of each pair
//   hdr  [warp][2 blocks][16 rows] uint4   raw headers of the warp's current chunk
//   red  [warp][16 rows][4] float          partial outputs of the warps of one row tile
template <int M>
__global__ void __launch_bounds__(IQ_THREADS, 1) matvec_q4k_imma(IqArgs p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int nsb = p.pairs * 2;
    uint32_t * xq = reinterpret_cast<uint32_t *>(smem);
    float2 * xs2 = reinterpret_cast<float2 *>(smem + (size_t) M * nsb * 64);
    uint4 * hdr = reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(xs2) + (size_t) M * nsb * 8);
    float * red = reinterpret_cast<float *>(hdr + IQ_WARPS * IQ_GROUPS * 32);

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int group = wid / IQ_WARPS, warp = wid % IQ_WARPS;
    const int g = lane >> 2, t = lane & 3;

    // first chunk of weights: independent of the predecessor kernel
    IqStage cur, nxt;
    int rt = blockIdx.x * IQ_GROUPS + group, chunk = warp;
    if (rt < p.n_tiles && chunk < p.chunks) iq_load_stage(p, rt, chunk, lane, cur);

    pdl_wait();

    // activations -> 16-bit integers per 32-element sub-block.  One item = 4 consecutive elements; the 8 items of
    // a sub-block sit in 8 consecutive lanes.
    const int items = p.pairs * 16;
    for (int it0 = tid; it0 < M * items; it0 += IQ_THREADS) {
        const int m = it0 / items, it = it0 - m * items;
        const int sb = it >> 3, q = it & 7;
        const float4 v = __ldcg(reinterpret_cast<const float4 *>(p.x + (int64_t) m * p.ldx + (int64_t) it * 4));   // coherent: the producer may still be running when this kernel starts
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
        float sum = (v.x + v.y) + (v.z + v.w);
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        const bool some = amax > 1e-30f;   // below that the block counts as zero
        const float inv = some ? 32512.0f / amax : 0.0f;
        const float s = some ? amax * (1.0f / 32512.0f) : 0.0f;
        const int xi[4] = {__float2int_rn(v.x * inv), __float2int_rn(v.y * inv), __float2int_rn(v.z * inv), __float2int_rn(v.w * inv)};
        uint32_t hp = 0, lp = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int lo = ((xi[e] + 128) & 255) - 128;
            const int hi = (xi[e] - lo) >> 8;
            hp |= ((uint32_t) hi & 255u) << (8 * e);
            lp |= ((uint32_t) lo & 255u) << (8 * e);
        }
        uint32_t * dst = xq + ((size_t) m * nsb + sb) * 16 + (q & 3) * 2 + (q >> 2);
        dst[0] = hp;
        dst[8] = lp;
        if (q == 0) xs2[(size_t) m * nsb + sb] = make_float2(s, sum);
    }
    __syncthreads();
    pdl_launch_dependents();

    // per-lane views.  Pair j of a block feeds B columns 2j (h plane) and 2j+1 (l plane): lane (g, t) supplies
    // column g, so it reads plane g & 1 of pair g >> 1 and zeros for the other pairs.
    const uint2 * xq_lane = reinterpret_cast<const uint2 *>(xq) + (g & 1) * 4 + t;   // uint2 units: 8 per sub-block
    const float4 * xs_lane = reinterpret_cast<const float4 *>(xs2) + t;
    uint4 * my_hdr = hdr + wid * 32;
    const int rt_step = gridDim.x * IQ_GROUPS;
    float * my_red = red + group * (IQ_WARPS * 64);
    const int gtid = tid - group * (IQ_WARPS * 32);

    // every group runs the same number of rounds so that the CTA-wide barriers match
    for (int round = blockIdx.x * IQ_GROUPS; round < p.n_tiles; round += rt_step) {
        float acc0[M], acc1[M];   // rows g and g + 8 of the tile
#pragma unroll
        for (int m = 0; m < M; ++m) acc0[m] = acc1[m] = 0.f;
        for (; rt < p.n_tiles && chunk < p.chunks; chunk += IQ_WARPS) {
            // prefetch the next work item of this warp
            int nrt = rt, nchunk = chunk + IQ_WARPS;
            if (nchunk >= p.chunks) { nrt = rt + rt_step; nchunk = warp; }
            if (nrt < p.n_tiles && nchunk < p.chunks) iq_load_stage(p, nrt, nchunk, lane, nxt);

            __syncwarp();
            my_hdr[lane] = cur.h;   // [block of the chunk][row]
            __syncwarp();

#pragma unroll
            for (int b2 = 0; b2 < 2; ++b2) {
                const int blk = chunk * 2 + b2;
                int clo[M][4], chi[M][4];
#pragma unroll
                for (int m = 0; m < M; ++m)
#pragma unroll
                    for (int i = 0; i < 4; ++i) clo[m][i] = chi[m][i] = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 wt = cur.a[b2 * 4 + j];   // x, y: row g k-halves 0, 1; z, w: row g + 8
                    const bool live = (g >> 1) == j;
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        uint2 blo = make_uint2(0u, 0u), bhi = make_uint2(0u, 0u);
                        if (live && blk < p.blocks) {
                            const uint2 * src = xq_lane + ((size_t) m * nsb + (size_t) (blk * 4 + j) * 2) * 8;
                            blo = src[0];
                            bhi = src[8];
                        }
                        imma_16832(clo[m], wt.x & 0x0F0F0F0Fu, wt.z & 0x0F0F0F0Fu, wt.y & 0x0F0F0F0Fu, wt.w & 0x0F0F0F0Fu, blo.x, blo.y);
                        imma_16832(chi[m], wt.x & 0xF0F0F0F0u, wt.z & 0xF0F0F0F0u, wt.y & 0xF0F0F0F0u, wt.w & 0xF0F0F0F0u, bhi.x, bhi.y);
                    }
                }
                if (blk < p.blocks) {
                    const uint4 h0 = my_hdr[b2 * 16 + g], h1 = my_hdr[b2 * 16 + g + 8];
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        const float4 sq = xs_lane[((size_t) m * nsb >> 1) + blk * 4];
                        acc0[m] += iq_row_term(h0, t, clo[m][0], clo[m][1], chi[m][0], chi[m][1], sq);
                        acc1[m] += iq_row_term(h1, t, clo[m][2], clo[m][3], chi[m][2], chi[m][3], sq);
                    }
                }
            }
            cur = nxt;
        }
        // sum over the four lanes of a row (each held other sub-blocks), then over the warps (each held other chunks)
#pragma unroll
        for (int m = 0; m < M; ++m) {
            acc0[m] += __shfl_xor_sync(0xffffffffu, acc0[m], 1);
            acc0[m] += __shfl_xor_sync(0xffffffffu, acc0[m], 2);
            acc1[m] += __shfl_xor_sync(0xffffffffu, acc1[m], 1);
            acc1[m] += __shfl_xor_sync(0xffffffffu, acc1[m], 2);
        }
        if (t < M) {
            float v0 = acc0[0], v1 = acc1[0];
#pragma unroll
            for (int m = 1; m < M; ++m)
                if (t == m) { v0 = acc0[m]; v1 = acc1[m]; }
            my_red[(warp * 16 + g) * 4 + t] = v0;
            my_red[(warp * 16 + g + 8) * 4 + t] = v1;
        }
        __syncthreads();
        if (gtid < 64 && rt < p.n_tiles) {
            const int row = gtid >> 2, col = gtid & 3;
            if (col < M) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < IQ_WARPS; ++w) v += my_red[(w * 16 + row) * 4 + col];
                p.y[(int64_t) col * p.ldy + (int64_t) rt * 16 + row] = v;
            }
        }
        __syncthreads();
        rt += rt_step;
        chunk = warp;
    }
}

size_t iq_smem_bytes(int pairs, int m) {
    return (size_t) m * pairs * 2 * (64 + 8) + (size_t) IQ_WARPS * IQ_GROUPS * 32 * 16 + (size_t) IQ_WARPS * IQ_GROUPS * 16 * 4 * 4;
}

template <int M>
int launch_iq(cudaStream_t s, const IqArgs & a, size_t smem, int grid) {
    if (smem > 48 * 1024) SM100_CUDA(cudaFuncSetAttribute(matvec_q4k_imma<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    return launch(matvec_q4k_imma<M>, dim3((unsigned) grid), dim3(IQ_THREADS), smem, s, a);
}

}  // namespace

// Q4_K packed matvec (1 or 2 activation columns) over the full 16-row tiles of the tensor; *handled = false when
// the shape is left to the caller's other kernels.
int matvec_q4k_imma_tiles(cudaStream_t s, const void * w, int64_t k, int64_t n, const float * x, int64_t ldx, int64_t m, float * y, int64_t ldy,
                          bool * handled) {
    *handled = false;
    const int64_t tiles = n / 16;
    if (tiles == 0 || m < 1 || m > 2 || k % 256 != 0 || k / 64 > 4096) return ST_OK;
    const int pairs = (int) (k / 64);
    const size_t smem = iq_smem_bytes(pairs, (int) m);
    if (smem > 227 * 1024) return ST_OK;
    if (((uintptr_t) w & 15) != 0 || ((uintptr_t) x & 15) != 0 || (m > 1 && (ldx & 3) != 0)) return ST_OK;
    IqArgs a;
    a.w = (const uint8_t *) w;
    a.h_off = n * (k / 256) * 128;
    a.x = x;
    a.y = y;
    a.ldx = ldx;
    a.ldy = ldy;
    a.n_tiles = (int) tiles;
    a.pairs = pairs;
    a.blocks = (int) (k / 256);
    a.chunks = (a.blocks + 1) / 2;
    int64_t grid = sm_count();   // one CTA per SM: the activations are quantized once per SM
    const int64_t rounds = (tiles + IQ_GROUPS - 1) / IQ_GROUPS;
    if (grid > rounds) grid = rounds;
    const int st = m == 1 ? launch_iq<1>(s, a, smem, (int) grid) : launch_iq<2>(s, a, smem, (int) grid);
    *handled = st == ST_OK;
    return st;
}

}  // namespace sm100
