// Q4_K decode MUL_MAT, one activation column, integer tensor cores, built so that CONSECUTIVE launches overlap.
//
// A decode matvec over a 9-28 MB matrix lasts 1.5-4 us at HBM speed; with one launch per op, what separates a kernel
// from the HBM roofline is not its streaming rate but what happens around it: the ramp of a fresh launch, the
// activation hand-over from the previous op, the tail.  This kernel is organised around that:
//
//  * it needs at most half of an SM (512 threads, <= 64 registers per thread, about 82 KB of shared memory), so the
//    CTAs of the NEXT launch on the stream become resident beside the running ones as soon as this launch has allowed
//    it - which it does in its first instructions (griddepcontrol.launch_dependents).  A resident successor copies
//    its first weights into its shared-memory ring (72 KB per SM: 10.9 MB over the GPU, more than a whole
//    4096 x 4096 matrix) and only then waits for its predecessor (griddepcontrol.wait): HBM streams the successor's
//    first weights while the predecessor computes and drains.  (Asking for the REST of the successor's weights to be
//    brought into L2 at the same moment was measured too - per-lane prefetch.global.L2 as well as
//    cp.async.bulk.prefetch.L2 - and made the sweep 4 % slower: the predecessor's loop already runs at the rate HBM
//    delivers, so the early requests only take bandwidth from it.);
//  * the ring is fed by per-lane 16-byte asynchronous copies (cp.async), not by bulk copies: a lane copies exactly
//    the 16 bytes of each tile that it will read back (the packed layout is in MMA-fragment order), so a slot needs no
//    barrier and no proxy fence - the lane waits for its own copy group - and issuing a refill costs four
//    instructions.  (Measured with a bulk copy per 2 KB unit: issuing one stalls the warp for about 0.4 us, which
//    made the loop latency-bound at 0.95 us per unit whatever the memory system delivered.);
//  * nothing in the main loop is CTA-wide.  A warp owns a fixed K range (whole 256-weight blocks), quantizes exactly
//    the activations of that range into REGISTERS in the B-fragment order of mma.m16n8k32 (no shared-memory image of
//    x, no barrier between quantization and the first MMA), and walks over the CTA's row tiles with its own ring
//    slots and mbarriers.  The warps of a row tile meet once, at the end, to add their partial sums;
//  * the arithmetic is that of matvec_q4k_imma (sm100_matvec_q4k_imma.cu): u8 nibbles x s16 activations (two s8 planes,
//    one f32 scale per 32) -> exact s32 dots per sub-block, then d * sc * s * dot - dmin * m * sum(x)
//    (src/core/ref/quant.cpp:55-82 of the reference folded into src/core/ref/ops.cpp:891-984).
//
// Replaces k_mvr_q4_k / k_mvm_q4_k of the OpenCL backend (src/backends/opencl11/kernels/mul_mv_k.cl:396-450,
// mul_mv_multi.cl:46-104) for packed tensors, M = 1, K up to 48 blocks per group of warps.
#include "sm100_quant_units.cuh"

#include <cstdlib>

namespace sm100 {

namespace {

constexpr int RG_WARPS = 16;
constexpr int RG_THREADS = RG_WARPS * 32;
constexpr int RG_MAX_SLOTS = 2;                   // ring slots per warp (a third one was measured: the 4 KB it takes from the partial-sum window cost more than it gave)
constexpr uint32_t RG_TILE_BYTES = 2048;          // 16 rows x 256 weights
constexpr uint32_t RG_HDR_BYTES = 256;            // their 16 block headers
constexpr int RG_WINDOW = 8;                      // rounds whose partial sums are kept before the CTA adds them up
constexpr int RG_MAX_TENSORS = 3;

struct RingArgs {
    const uint8_t * w[RG_MAX_TENSORS];   // packed tensor bases
    int64_t h_off[RG_MAX_TENSORS];       // byte offset of each header plane
    float * y[RG_MAX_TENSORS];
    int tile_end[RG_MAX_TENSORS];        // row tiles of tensors 0..i together (INT32_MAX for unused slots)
    const float * x;                     // [K] (prologue 0)
    const float * pa; const float * pb; const float * pw;   // prologue inputs (see Q4KPrologue)
    float * sum_out; float * x_out;
    float eps;
    int n_tiles;        // full 16-row tiles of all tensors
    int blocks;         // K / 256
    int wpt;            // warps that share one row tile (they split K); a power of two <= 16
    int groups;         // row tiles a CTA works on at a time = 16 / wpt
    int slots;          // ring slots per warp (2 or 3)
};

__device__ __forceinline__ uint32_t rg_smem(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }
// per-thread 16-byte asynchronous copy global -> shared (L2 only), and the grouping of such copies
__device__ __forceinline__ void rg_cp_async16(uint32_t dst, const void * src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void rg_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void rg_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// a value and its step tag as ONE 8-byte access (single-copy atomic: the reader sees both words of a store or neither)
__device__ __forceinline__ void rg_st_tagged(uint2 * p, float v, uint32_t tag) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 rg_ld_tagged(const uint2 * p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t rg_lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 rg_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void rg_imma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void rg_imma_zero(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// max(|a|, |b|) that keeps a NaN (fmaxf would drop it): the group scale must see it, see act_group_scale
__device__ __forceinline__ float rg_absmax_nan(float a, float b) {
    float r;
    asm("{\n\t.reg .f32 ta, tb;\n\tabs.f32 ta, %1;\n\tabs.f32 tb, %2;\n\tmax.NaN.f32 %0, ta, tb;\n\t}" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

__device__ __forceinline__ void rg_locate(const RingArgs & p, int tile, int & tensor, int & local) {
    tensor = (tile >= p.tile_end[0] ? 1 : 0) + (tile >= p.tile_end[1] ? 1 : 0);
    local = tile - (tensor == 0 ? 0 : p.tile_end[tensor - 1]);
}

// The activations of one 256-weight block as this lane's share of the MMA B operand.
// Lane (g, t) of the warp first quantizes 8 elements of sub-block g (k = 4t..4t+3 and 16+4t..19+4t of its 32: the
// k positions of its B-fragment registers), the 4 lanes of a sub-block agree on the scale, and lanes g and g ^ 1
// trade planes: pair j = g >> 1 feeds B column 2j with the high-byte plane and column 2j+1 with the low-byte plane
// of BOTH its sub-blocks, and lane (g, t) supplies column g.
struct RgBlockX {
    uint32_t lo0, lo1;   // B registers for the MMA over the pair's low-nibble sub-block (2j)
    uint32_t hi0, hi1;   // ... over the high-nibble sub-block (2j + 1)
    float s0, x0, s1, x1;   // (scale, sum of activations) of sub-blocks 2t and 2t+1: what this lane's C columns need
};

// Quantizes the NB blocks of a warp side by side, stage by stage, so that the shuffle and conversion latencies of the
// blocks overlap (one block after the other the chains are serial: 0.55 us per block was measured).
template <int NBW>
__device__ __forceinline__ void rg_quantize(const float4 (&va)[NBW], const float4 (&vb)[NBW], int nb, int lane, RgBlockX (&o)[NBW]) {
    const int g = lane >> 2, t = lane & 3;
    float amax[NBW], sum[NBW], inv[NBW], s[NBW];
#pragma unroll
    for (int i = 0; i < NBW; ++i) {
        if (i < nb) {
            amax[i] = rg_absmax_nan(rg_absmax_nan(rg_absmax_nan(va[i].x, va[i].y), rg_absmax_nan(va[i].z, va[i].w)),
                                    rg_absmax_nan(rg_absmax_nan(vb[i].x, vb[i].y), rg_absmax_nan(vb[i].z, vb[i].w)));
            sum[i] = ((va[i].x + va[i].y) + (va[i].z + va[i].w)) + ((vb[i].x + vb[i].y) + (vb[i].z + vb[i].w));
        }
    }
#pragma unroll
    for (int o2 = 1; o2 <= 2; o2 <<= 1) {
#pragma unroll
        for (int i = 0; i < NBW; ++i) {
            if (i < nb) {
                amax[i] = rg_absmax_nan(amax[i], __shfl_xor_sync(0xffffffffu, amax[i], o2));
                sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], o2);
            }
        }
    }
    // round to nearest even without the conversion unit: 1.5 * 2^23 + v keeps the integer in the mantissa (|v| <= 32512),
    // integer = bits - 0x4B400000.  16-bit integer = 256 h + l with h, l signed bytes: h = (integer + 128) >> 8, l = its
    // low byte, which is also the low byte of `bits`.
    constexpr int HB = 128 - 0x4B400000;
    const bool odd = (g & 1) != 0;   // an even g holds the pair's low sub-block and supplies the h plane; an odd g the high sub-block and the l plane
    uint32_t h0[NBW], h1[NBW], l0[NBW], l1[NBW];
#pragma unroll
    for (int i = 0; i < NBW; ++i) {
        if (i < nb) {
            act_group_scale(__float_as_uint(amax[i]), inv[i], s[i]);
            const int q0 = __float_as_int(fmaf(va[i].x, inv[i], 12582912.0f)), q1 = __float_as_int(fmaf(va[i].y, inv[i], 12582912.0f)),
                      q2 = __float_as_int(fmaf(va[i].z, inv[i], 12582912.0f)), q3 = __float_as_int(fmaf(va[i].w, inv[i], 12582912.0f)),
                      q4 = __float_as_int(fmaf(vb[i].x, inv[i], 12582912.0f)), q5 = __float_as_int(fmaf(vb[i].y, inv[i], 12582912.0f)),
                      q6 = __float_as_int(fmaf(vb[i].z, inv[i], 12582912.0f)), q7 = __float_as_int(fmaf(vb[i].w, inv[i], 12582912.0f));
            h0[i] = __byte_perm(__byte_perm((uint32_t) ((q0 + HB) >> 8), (uint32_t) ((q1 + HB) >> 8), 0x0040),
                                __byte_perm((uint32_t) ((q2 + HB) >> 8), (uint32_t) ((q3 + HB) >> 8), 0x0040), 0x5410);
            h1[i] = __byte_perm(__byte_perm((uint32_t) ((q4 + HB) >> 8), (uint32_t) ((q5 + HB) >> 8), 0x0040),
                                __byte_perm((uint32_t) ((q6 + HB) >> 8), (uint32_t) ((q7 + HB) >> 8), 0x0040), 0x5410);
            l0[i] = __byte_perm(__byte_perm((uint32_t) q0, (uint32_t) q1, 0x0040), __byte_perm((uint32_t) q2, (uint32_t) q3, 0x0040), 0x5410);
            l1[i] = __byte_perm(__byte_perm((uint32_t) q4, (uint32_t) q5, 0x0040), __byte_perm((uint32_t) q6, (uint32_t) q7, 0x0040), 0x5410);
        }
    }
#pragma unroll
    for (int i = 0; i < NBW; ++i) {
        if (i < nb) {
            const uint32_t r0 = __shfl_xor_sync(0xffffffffu, odd ? h0[i] : l0[i], 4);
            const uint32_t r1 = __shfl_xor_sync(0xffffffffu, odd ? h1[i] : l1[i], 4);
            o[i].lo0 = odd ? r0 : h0[i];
            o[i].lo1 = odd ? r1 : h1[i];
            o[i].hi0 = odd ? l0[i] : r0;
            o[i].hi1 = odd ? l1[i] : r1;
            // C column pair of lane t = sub-blocks 2t (low nibbles of pair t) and 2t + 1: their scales sit in quads 2t, 2t + 1
            o[i].s0 = __shfl_sync(0xffffffffu, s[i], 8 * t);
            o[i].x0 = __shfl_sync(0xffffffffu, sum[i], 8 * t);
            o[i].s1 = __shfl_sync(0xffffffffu, s[i], 8 * t + 4);
            o[i].x1 = __shfl_sync(0xffffffffu, sum[i], 8 * t + 4);
        }
    }
}

// one row's share of a block for lane t (see iq_row_term of sm100_matvec_q4k_imma.cu)
__device__ __forceinline__ float rg_row_term(uint32_t dd, uint32_t f0, uint32_t f1, uint32_t shift, int clo_h, int clo_l, int chi_h, int chi_l,
                                             const RgBlockX & b) {
    const float2 df = __half22float2(*reinterpret_cast<const __half2 *>(&dd));   // d, dmin
    const uint32_t f = __funnelshift_r(f0, f1, shift);
    const int sc0 = (int) (f & 63u), m0 = (int) ((f >> 6) & 63u), sc1 = (int) ((f >> 12) & 63u), m1 = (int) ((f >> 18) & 63u);
    const int v0 = clo_h * 256 + clo_l;          // exact: |v0| < 2^24
    const int v1 = (chi_h * 256 + chi_l) >> 4;   // exact: every term carries the factor 16 of the high nibble (kept out of v1 * sc1: |.| < 2^31)
    const float dot = fmaf((float) (v1 * sc1), b.s1, (float) (v0 * sc0) * b.s0);
    const float mins = fmaf((float) m1, b.x1, (float) m0 * b.x0);
    return fmaf(df.x, dot, -df.y * mins);
}

// Shared memory of one CTA:
//   red   [RG_WINDOW][warp][16 rows] float     partial sums of the warps, one window of rounds
//   hdr   [warp][slots][16 rows] uint4         block headers of the units in flight
//   ring  [warp][slots][4 tiles][512 B]        weight tiles of the units in flight (each lane's 16 bytes are its own)
//   row   [K] float                            PRO == 2 only: the residual row before normalisation
// NBW: 256-weight blocks of K per warp (compile time: their activations live in registers).
// PRO: 0 x is given; 1 x = swiglu(pa, pb); 2 s = pa (+ pb), x = rms_norm(s) * pw (s, x written out by CTA 0 when asked).
// AR: the launch is one rank's K shard of a product (single tensor): the row tiles' partial sums go through the all-reduce
//     exchange `f` (see ArFuse) instead of straight to y, and y receives the sum over the ranks.
template <int NBW, int PRO, bool AR>
__global__ void __launch_bounds__(RG_THREADS, 2) matvec_q4k_ring(RingArgs p, ArFuse f) {
    extern __shared__ __align__(128) uint8_t smem[];
    float * red = reinterpret_cast<float *>(smem);
    uint8_t * hdr = smem + RG_WINDOW * RG_WARPS * 16 * 4;
    uint8_t * ring = hdr + RG_WARPS * p.slots * RG_HDR_BYTES;
    float * row = reinterpret_cast<float *>(ring + RG_WARPS * p.slots * RG_TILE_BYTES);

    // the successor on the stream may become resident (and prefetch) from now on; it still waits for this grid's
    // completion before it reads anything this grid writes
    pdl_launch_dependents();

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int group = wid / p.wpt, kw = wid - group * p.wpt;
    const int tile_step = gridDim.x * p.groups;
    const int tile0 = blockIdx.x * p.groups + group;
    // blocks of K this warp owns: kw, kw + wpt, ... (nb of them, <= NBW)
    const int nb = kw < p.blocks ? (p.blocks - kw + p.wpt - 1) / p.wpt : 0;
    const int rounds = tile0 < p.n_tiles ? (p.n_tiles - tile0 + tile_step - 1) / tile_step : 0;   // row tiles of this warp's group
    const int units = rounds * nb;

    const uint32_t hdr0 = rg_smem(hdr) + (uint32_t) (wid * p.slots) * RG_HDR_BYTES;
    const uint32_t ring0 = rg_smem(ring) + (uint32_t) (wid * p.slots) * RG_TILE_BYTES + (uint32_t) lane * 16u;   // this lane's 16 bytes of tile 0, slot 0

    // Unit u of this warp = (round u / nb, block kw + wpt * (u % nb)), kept in slot u % slots.  The request cursor
    // walks the units in that order; the addresses of a round (tensor, row tile) are worked out once per round.
    const uint32_t tile_bytes_per_rt = (uint32_t) p.blocks * RG_TILE_BYTES;
    const uint32_t hdr_bytes_per_rt = (uint32_t) p.blocks * 256u;
    const uint32_t blk_tile_step = (uint32_t) p.wpt * RG_TILE_BYTES, blk_hdr_step = (uint32_t) p.wpt * 16u;
    int issued = 0, rq_r = 0, rq_i = 0;
    uint32_t rq_slot = 0;
    const uint8_t * rq_tiles = nullptr;   // tiles of (round rq_r, this warp's first block)
    const uint8_t * rq_hdrs = nullptr;    // header of (round rq_r, row lane & 15, this warp's first block)
    auto rq_round = [&]() {
        int ti, rt;
        rg_locate(p, tile0 + rq_r * tile_step, ti, rt);
        const uint8_t * wbase = p.w[ti];
        rq_tiles = wbase + (uint64_t) rt * tile_bytes_per_rt + (uint32_t) kw * RG_TILE_BYTES;
        rq_hdrs = wbase + p.h_off[ti] + (uint64_t) rt * hdr_bytes_per_rt + (uint32_t) ((lane & 15) * p.blocks + kw) * 16u;
    };
    auto request = [&]() {   // copies the unit under the cursor into the next slot (one copy group per unit) and advances the cursor
        const uint32_t s = rq_slot;
        rq_slot = rq_slot + 1 == (uint32_t) p.slots ? 0u : rq_slot + 1;
        const uint8_t * src = rq_tiles + (uint32_t) rq_i * blk_tile_step + (uint32_t) lane * 16u;
#pragma unroll
        for (int j = 0; j < 4; ++j) rg_cp_async16(ring0 + s * RG_TILE_BYTES + j * 512, src + j * 512);
        if (lane < 16) rg_cp_async16(hdr0 + s * RG_HDR_BYTES + lane * 16, rq_hdrs + (uint32_t) rq_i * blk_hdr_step);
        rg_cp_async_commit();
        ++issued;
        if (++rq_i == nb) {
            rq_i = 0;
            if (++rq_r < rounds) rq_round();
        }
    };
    if (units > 0) rq_round();
    while (issued < p.slots && issued < units) request();

    pdl_wait();   // everything below may depend on the predecessor's output

    // fused all-reduce: the number of this fused launch (every rank counts alike) tags its values and picks one of the
    // two receive buffers; the last CTA to finish advances the counter, which the next fused launch reads after its own
    // dependency wait, i.e. after this grid has completed
    uint32_t ar_step = 0;
    if constexpr (AR) ar_step = __ldcg(f.step) + 1u;

    // ---- activations of this warp's K range -> registers ----
    RgBlockX bx[NBW];
    if (PRO == 2) {
        // (ADD_)RMS_NORM_MUL (src/core/ref/ops.cpp:466-519): the CTA adds and squares the row once (kept in shared
        // memory), then every warp normalises and quantizes its own range
        const int items = p.blocks * 64;   // float4 items
        double sq = 0.0;
        for (int it = tid; it < items; it += RG_THREADS) {
            float4 v = __ldcg(reinterpret_cast<const float4 *>(p.pa) + it);
            if (p.pb != nullptr) {
                const float4 b = __ldcg(reinterpret_cast<const float4 *>(p.pb) + it);
                v = make_float4(__fadd_rn(v.x, b.x), __fadd_rn(v.y, b.y), __fadd_rn(v.z, b.z), __fadd_rn(v.w, b.w));
            }
            reinterpret_cast<float4 *>(row)[it] = v;
            if (p.sum_out != nullptr && blockIdx.x == 0) reinterpret_cast<float4 *>(p.sum_out)[it] = v;
            sq += ((double) v.x * (double) v.x + (double) v.y * (double) v.y) + ((double) v.z * (double) v.z + (double) v.w * (double) v.w);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        double * dred = reinterpret_cast<double *>(red);   // free until the first round's partial sums
        if (lane == 0) dred[wid] = sq;
        __syncthreads();
        double tot = 0.0;
#pragma unroll
        for (int w = 0; w < RG_WARPS; ++w) tot += dred[w];
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float) (tot / (double) (items * 4)), p.eps)));
        __syncthreads();   // dred is part of `red`
        float4 va[NBW], vb[NBW];
#pragma unroll
        for (int i = 0; i < NBW; ++i) {
            if (i < nb) {
                const int e0 = (kw + p.wpt * i) * 256 + g * 32 + 4 * t;   // element index of the lane's first float4
                va[i] = *reinterpret_cast<const float4 *>(row + e0);
                vb[i] = *reinterpret_cast<const float4 *>(row + e0 + 16);
                const float4 wa = __ldg(reinterpret_cast<const float4 *>(p.pw + e0)), wb = __ldg(reinterpret_cast<const float4 *>(p.pw + e0 + 16));
                va[i] = make_float4(__fmul_rn(__fmul_rn(va[i].x, scale), wa.x), __fmul_rn(__fmul_rn(va[i].y, scale), wa.y),
                                    __fmul_rn(__fmul_rn(va[i].z, scale), wa.z), __fmul_rn(__fmul_rn(va[i].w, scale), wa.w));
                vb[i] = make_float4(__fmul_rn(__fmul_rn(vb[i].x, scale), wb.x), __fmul_rn(__fmul_rn(vb[i].y, scale), wb.y),
                                    __fmul_rn(__fmul_rn(vb[i].z, scale), wb.z), __fmul_rn(__fmul_rn(vb[i].w, scale), wb.w));
                if (p.x_out != nullptr && blockIdx.x == 0 && group == 0) {
                    *reinterpret_cast<float4 *>(p.x_out + e0) = va[i];
                    *reinterpret_cast<float4 *>(p.x_out + e0 + 16) = vb[i];
                }
            }
        }
        rg_quantize<NBW>(va, vb, nb, lane, bx);
    } else {
        float4 va[NBW], vb[NBW], ga[NBW], gb[NBW];
#pragma unroll
        for (int i = 0; i < NBW; ++i) {
            if (i < nb) {
                const int e0 = (kw + p.wpt * i) * 256 + g * 32 + 4 * t;
                // coherent loads: the producer may have been running when this kernel started
                if (PRO == 0) {
                    va[i] = __ldcg(reinterpret_cast<const float4 *>(p.x + e0));
                    vb[i] = __ldcg(reinterpret_cast<const float4 *>(p.x + e0 + 16));
                } else {
                    va[i] = __ldcg(reinterpret_cast<const float4 *>(p.pa + e0));
                    vb[i] = __ldcg(reinterpret_cast<const float4 *>(p.pa + e0 + 16));
                    ga[i] = __ldcg(reinterpret_cast<const float4 *>(p.pb + e0));
                    gb[i] = __ldcg(reinterpret_cast<const float4 *>(p.pb + e0 + 16));
                }
            }
        }
#pragma unroll
        for (int i = 0; i < NBW; ++i) {
            if (i < nb) {
                if (PRO == 1) {
                    // SwiGLU (src/core/ref/ops.cpp:383-425): (a / (1 + expf(-a))) * b, the arithmetic of swiglu_kernel
                    va[i] = make_float4(__fmul_rn(__fdiv_rn(va[i].x, __fadd_rn(1.0f, expf(-va[i].x))), ga[i].x),
                                        __fmul_rn(__fdiv_rn(va[i].y, __fadd_rn(1.0f, expf(-va[i].y))), ga[i].y),
                                        __fmul_rn(__fdiv_rn(va[i].z, __fadd_rn(1.0f, expf(-va[i].z))), ga[i].z),
                                        __fmul_rn(__fdiv_rn(va[i].w, __fadd_rn(1.0f, expf(-va[i].w))), ga[i].w));
                    vb[i] = make_float4(__fmul_rn(__fdiv_rn(vb[i].x, __fadd_rn(1.0f, expf(-vb[i].x))), gb[i].x),
                                        __fmul_rn(__fdiv_rn(vb[i].y, __fadd_rn(1.0f, expf(-vb[i].y))), gb[i].y),
                                        __fmul_rn(__fdiv_rn(vb[i].z, __fadd_rn(1.0f, expf(-vb[i].z))), gb[i].z),
                                        __fmul_rn(__fdiv_rn(vb[i].w, __fadd_rn(1.0f, expf(-vb[i].w))), gb[i].w));
                }
            }
        }
        rg_quantize<NBW>(va, vb, nb, lane, bx);
    }

    // ---- main loop: this warp's units, round by round ----
    const int live_pair = g >> 1;
    // the 24-bit scale field of lane t starts at byte 4 + 3 t of a 16-byte header
    const uint32_t fld_off = (uint32_t) (4 + 3 * t) & ~3u, fld_shift = ((uint32_t) (4 + 3 * t) & 3u) * 8u;
    int u = 0;
    uint32_t cs = 0;   // slot of unit u
    // rounds of group 0, the most any group of this CTA has: the window loop and its barriers are CTA-uniform
    const int cta_rounds = (p.n_tiles - (int) blockIdx.x * p.groups + tile_step - 1) / tile_step;
    for (int base = 0; base < cta_rounds; base += RG_WINDOW) {
        const int wend = base + RG_WINDOW < rounds ? base + RG_WINDOW : rounds;
        for (int r = base; r < wend; ++r) {
            float acc0 = 0.f, acc1 = 0.f;   // rows g and g + 8 of the tile
#pragma unroll
            for (int i = 0; i < NBW; ++i) {
                if (i < nb) {
                    const uint32_t s = cs;
                    cs = cs + 1 == (uint32_t) p.slots ? 0u : cs + 1;
                    // unit u's copy group is the oldest one outstanding; those of the units requested after it may still be in flight
                    const int younger = issued - u - 1;
                    if (younger >= 2) rg_cp_async_wait<2>();
                    else if (younger == 1) rg_cp_async_wait<1>();
                    else rg_cp_async_wait<0>();
                    __syncwarp();   // the headers were copied by lanes 0..15 for the whole warp
                    {
                        const uint32_t tiles_lane = ring0 + s * RG_TILE_BYTES;
                        int clo[4], chi[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint4 wt = rg_lds128(tiles_lane + j * 512);   // x, y: row g k-halves 0, 1; z, w: row g + 8
                            const bool live = j == live_pair;
                            const uint32_t b0 = live ? bx[i].lo0 : 0u, b1 = live ? bx[i].lo1 : 0u, b2 = live ? bx[i].hi0 : 0u, b3 = live ? bx[i].hi1 : 0u;
                            if (j == 0) {
                                rg_imma_zero(clo, wt.x & 0x0F0F0F0Fu, wt.z & 0x0F0F0F0Fu, wt.y & 0x0F0F0F0Fu, wt.w & 0x0F0F0F0Fu, b0, b1);
                                rg_imma_zero(chi, wt.x & 0xF0F0F0F0u, wt.z & 0xF0F0F0F0u, wt.y & 0xF0F0F0F0u, wt.w & 0xF0F0F0F0u, b2, b3);
                            } else {
                                rg_imma(clo, wt.x & 0x0F0F0F0Fu, wt.z & 0x0F0F0F0Fu, wt.y & 0x0F0F0F0Fu, wt.w & 0x0F0F0F0Fu, b0, b1);
                                rg_imma(chi, wt.x & 0xF0F0F0F0u, wt.z & 0xF0F0F0F0u, wt.y & 0xF0F0F0F0u, wt.w & 0xF0F0F0F0u, b2, b3);
                            }
                        }
                        const uint32_t ha = hdr0 + s * RG_HDR_BYTES + g * 16, hb = ha + 128;   // headers of rows g and g + 8
                        const uint32_t da = rg_lds32(ha), fa0 = rg_lds32(ha + fld_off), fa1 = rg_lds32(ha + fld_off + 4);
                        const uint32_t db = rg_lds32(hb), fb0 = rg_lds32(hb + fld_off), fb1 = rg_lds32(hb + fld_off + 4);
                        acc0 += rg_row_term(da, fa0, fa1, fld_shift, clo[0], clo[1], chi[0], chi[1], bx[i]);
                        acc1 += rg_row_term(db, fb0, fb1, fld_shift, clo[2], clo[3], chi[2], chi[3], bx[i]);
                        // the slot's contents sit in registers that the MMAs have read: refill it
                        __syncwarp();
                        if (issued < units) request();
                        ++u;
                    }
                }
            }
            // the four lanes of a row held different sub-blocks
            acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
            acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
            if (t == 0) {
                float * dst = red + ((r - base) * RG_WARPS + wid) * 16;
                dst[g] = acc0;
                dst[g + 8] = acc1;
            }
        }
        __syncthreads();
        // add the partial sums of the warps of each (round, group) and store the tile's 16 outputs
        const int wr = (base + RG_WINDOW < cta_rounds ? base + RG_WINDOW : cta_rounds) - base;
        for (int idx = tid; idx < wr * p.groups * 16; idx += RG_THREADS) {
            const int r = idx / (p.groups * 16), rem = idx - r * (p.groups * 16);
            const int gq = rem >> 4, rw = rem & 15;
            const int tile = blockIdx.x * p.groups + gq + (base + r) * tile_step;
            if (tile < p.n_tiles) {
                const float * src = red + (r * RG_WARPS + gq * p.wpt) * 16 + rw;
                float v = 0.f;
                for (int w = 0; w < p.wpt; ++w) v += src[w * 16];
                if constexpr (AR) {
                    // my partial, tagged with the step, into my slot on every rank: one 8-byte store each (plain stores over
                    // NVLink, the local slot included); the tag travels with the value, so no fence and no separate flag
                    const size_t at = ((size_t) (ar_step & 1u) * f.world + f.rank) * f.capacity + (size_t) tile * 16 + rw;
                    for (int r = 0; r < f.world; ++r) rg_st_tagged(f.recv[r] + at, v, ar_step);
                } else {
                    int ti, lrt;
                    rg_locate(p, tile, ti, lrt);
                    p.y[ti][(int64_t) lrt * 16 + rw] = v;
                }
            }
        }
        if (base + RG_WINDOW < cta_rounds) __syncthreads();   // the next window reuses `red`
    }
    if constexpr (AR) {
        // the sum of the ranks' partials for this CTA's row tiles, in rank order (the same bits on every rank).  A value
        // is there when its tag equals this step; the wait for it is bounded (about a second), a give-up raises the fault
        // word and the sum goes on with what is there
        const uint2 * mine = f.recv[f.rank] + (size_t) (ar_step & 1u) * f.world * f.capacity;
        uint32_t limit = f.wait_limit;   // a thread waits out the bound once at most: after a give-up it only looks
        for (int idx = tid; idx < cta_rounds * p.groups * 16; idx += RG_THREADS) {
            const int r = idx / (p.groups * 16), rem = idx - r * (p.groups * 16);
            const int tile = blockIdx.x * p.groups + (rem >> 4) + r * tile_step;
            if (tile < p.n_tiles) {
                const int64_t at = (int64_t) tile * 16 + (rem & 15);
                float acc = 0.f;
                for (int q = 0; q < f.world; ++q) {
                    const uint2 * src = mine + (size_t) q * f.capacity + at;
                    uint2 got = rg_ld_tagged(src);
                    for (uint32_t spins = 0; got.y != ar_step && spins < limit; ++spins) {
                        if (spins > 32) __nanosleep(50);
                        got = rg_ld_tagged(src);
                    }
                    if (got.y != ar_step) {
                        atomicExch(f.fault, 100 + q);
                        limit = 0;
                    }
                    acc = q == 0 ? __uint_as_float(got.x) : __fadd_rn(acc, __uint_as_float(got.x));
                }
                p.y[0][at] = acc;
            }
        }
        __syncthreads();
        if (tid == 0 && atomicAdd(f.done, 1u) == gridDim.x - 1) {
            *f.done = 0u;
            *f.step = ar_step;
        }
    }
}

size_t ring_smem_bytes(int64_t k, int pro, int slots) {
    return (size_t) RG_WINDOW * RG_WARPS * 16 * 4 + (size_t) RG_WARPS * slots * (RG_HDR_BYTES + RG_TILE_BYTES) + (pro == 2 ? (size_t) k * 4 : 0);
}

template <int NBW>
int launch_ring(cudaStream_t s, const RingArgs & a, int pro, size_t smem, int grid, const ArFuse * fuse) {
    const ArFuse f = fuse != nullptr ? *fuse : ArFuse{};
#define SM100_RING_CASE(P, A)                                                                                                          \
    if (pro == P && (fuse != nullptr) == A) {                                                                                          \
        SM100_CUDA(cudaFuncSetAttribute(matvec_q4k_ring<NBW, P, A>, cudaFuncAttributeMaxDynamicSharedMemorySize, 113 * 1024));       \
        return launch(matvec_q4k_ring<NBW, P, A>, dim3((unsigned) grid), dim3(RG_THREADS), smem, s, a, f);                           \
    }
    SM100_RING_CASE(0, false)
    SM100_RING_CASE(1, false)
    SM100_RING_CASE(2, false)
    SM100_RING_CASE(0, true)
    SM100_RING_CASE(1, true)
#undef SM100_RING_CASE
    return fail(ST_INVALID, "matvec (Q4_K ring): unknown prologue");
}

}  // namespace

// Q4_K packed matvec, one activation column, over the full 16-row tiles of up to three tensors that share the
// activations; *handled = false when the shapes are left to the caller's other kernels.
// fuse (optional): the launch is this rank's K shard, y receives the sum over the ranks (single tensor, whole row tiles).
int matvec_q4k_ring_multi(cudaStream_t s, int count, const void * const * ws, const int64_t * ns, int64_t k, const float * x,
                          float * const * ys, bool * handled, const Q4KPrologue * pro, const ArFuse * fuse) {
    *handled = false;
    // SM100_Q4K_RING: 0 never; 1 (default) in runs of plain matvecs: a single tensor without prologue whose predecessor
    // on the stream is a matvec of the same kind; 2 wherever the shapes allow (tests).  The kernel pays off when launch
    // N + 1 finds ONE free CTA slot on every SM beside launch N (back to back 4.0 / 7.0 / 8.2 us per launch on the three
    // projection shapes against 4.4 / 7.9 / 8.6 of matvec_q4k_imma).  Behind a kernel of another kind its CTAs are placed
    // as SMs drain, two on the first SMs that become free and none on others, and the skew is inherited by every later
    // launch of the run (measured: 5.4 / 10.3 / 12.9 us per launch in a run started behind matvec_q4k_imma; a decode step
    // that used this kernel for its fused projections lost a fifth of its speed).  So the first ring launch of a run is
    // launched fully serialized - on an empty GPU the CTAs are dealt one per SM - and the later ones with programmatic
    // dependent launch.
    static const int enabled = [] { const char * e = getenv("SM100_Q4K_RING"); return e != nullptr ? atoi(e) : 1; }();
    if (!enabled) return ST_OK;
    const int tail = stream_tail(s);
    if (fuse != nullptr) {
        // only this kernel has the fused exchange: taken whenever the shapes allow, with the same care at the start of a run
        if (count != 1 || (pro != nullptr && pro->mode == 2) || ns[0] % 16 != 0 || ns[0] > fuse->capacity || fuse->world < 2 || fuse->world > AR_MAX_RANKS) return ST_OK;
    } else if (enabled == 1 && (count != 1 || (pro != nullptr && pro->mode != 0) || tail == TAIL_OTHER)) {
        return ST_OK;
    }
    const bool run_start = (enabled == 1 || fuse != nullptr) && tail != TAIL_Q4K_RING;
    int mode = 0;
    if (pro != nullptr && pro->mode != 0) {
        mode = pro->mode;
        if (pro->a == nullptr) return ST_OK;
        const uintptr_t al = (uintptr_t) pro->a | (uintptr_t) pro->b | (uintptr_t) pro->norm_w | (uintptr_t) pro->sum_out | (uintptr_t) pro->x_out;
        if ((al & 15) != 0) return ST_OK;
        if (mode == 1 && pro->b == nullptr) return ST_OK;
        if (mode == 2 && (pro->norm_w == nullptr || k > 4096)) return ST_OK;   // the row is staged in shared memory beside the ring
    } else if (x == nullptr || ((uintptr_t) x & 15) != 0) {
        return ST_OK;
    }
    if (count < 1 || count > RG_MAX_TENSORS || k <= 0 || k % 256 != 0) return ST_OK;
    const int blocks = (int) (k / 256);
    int wpt = 1;
    while (wpt < RG_WARPS && wpt < blocks) wpt *= 2;
    const int nbw = (blocks + wpt - 1) / wpt;
    if (nbw > 3) return ST_OK;   // activations of a warp's K range live in registers
    int64_t tiles = 0;
    for (int i = 0; i < count; ++i) {
        if (ns[i] / 16 == 0 || ((uintptr_t) ws[i] & 15) != 0) return ST_OK;
        if (count > 1 && ns[i] % 16 != 0) return ST_OK;   // leftover rows are the single-tensor caller's business
        tiles += ns[i] / 16;
    }
    if (tiles > INT32_MAX / 2) return ST_OK;
    RingArgs a = {};
    int end = 0;
    for (int i = 0; i < RG_MAX_TENSORS; ++i) {
        if (i < count) {
            a.w[i] = (const uint8_t *) ws[i];
            a.h_off[i] = ns[i] * (k / 256) * 128;
            a.y[i] = ys[i];
            end += (int) (ns[i] / 16);
            a.tile_end[i] = end;
        } else {
            a.tile_end[i] = INT32_MAX;
        }
    }
    a.x = x;
    if (mode != 0) {
        a.pa = pro->a; a.pb = pro->b; a.pw = pro->norm_w; a.sum_out = pro->sum_out; a.x_out = pro->x_out; a.eps = pro->eps;
    }
    a.n_tiles = (int) tiles;
    a.blocks = blocks;
    a.wpt = wpt;
    a.groups = RG_WARPS / wpt;
    int64_t grid = sm_count();
    const int64_t rounds = (tiles + a.groups - 1) / a.groups;
    if (grid > rounds) grid = rounds;
    // two CTAs (this launch's and its successor's) have to fit one SM: 228 KB less 1 KB per CTA
    a.slots = ring_smem_bytes(k, mode, RG_MAX_SLOTS) <= (size_t) 113 * 1024 ? RG_MAX_SLOTS : 2;
    const size_t smem = ring_smem_bytes(k, mode, a.slots);
    int st;
    if (run_start) thread_serialized(true);
    if (nbw == 1) st = launch_ring<1>(s, a, mode, smem, (int) grid, fuse);
    else if (nbw == 2) st = launch_ring<2>(s, a, mode, smem, (int) grid, fuse);
    else st = launch_ring<3>(s, a, mode, smem, (int) grid, fuse);
    if (run_start) thread_serialized(false);
    *handled = st == ST_OK;
    if (st == ST_OK && count == 1 && (mode == 0 || fuse != nullptr)) stream_tail_set(s, TAIL_Q4K_RING);
    return st;
}

}  // namespace sm100
