// Q4_K decode MUL_MAT, one activation column, integer tensor cores, built so that CONSECUTIVE launches overlap.
//
// A decode matvec over a 9-28 MB matrix lasts 1.5-4 us at HBM speed; with one launch per op, what separates a kernel
// from the HBM roofline is not its streaming rate but what happens around it: the ramp of a fresh launch, the
// activation hand-over from the previous op, the tail.  This kernel is organised around that:
//
//  * it needs at most half of an SM (512 threads, <= 64 registers per thread, about 100 KB of shared memory), so the
//    CTAs of the NEXT launch on the stream become resident beside the running ones as soon as this launch has allowed
//    it - which it does in its first instructions (griddepcontrol.launch_dependents).  A resident successor requests
//    its first weights (up to 72 KB per SM: 10.9 MB over the GPU, more than a whole 4096 x 4096 matrix) with bulk
//    copies into its shared-memory ring and only then waits for its predecessor (griddepcontrol.wait): HBM streams the
//    successor's weights while the predecessor computes and drains;
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

#include <atomic>
#include <cstdlib>

namespace sm100 {

namespace {

constexpr int RG_WARPS = 16;
constexpr int RG_THREADS = RG_WARPS * 32;
constexpr int RG_SLOTS = 2;                       // ring slots per warp
constexpr uint32_t RG_TILE_BYTES = 2048;          // 16 rows x 256 weights
constexpr uint32_t RG_HDR_BYTES = 256;            // their 16 block headers
constexpr int RG_WINDOW = 8;                      // rounds whose partial sums are kept before the CTA adds them up
constexpr int RG_MAX_TENSORS = 3;
constexpr uint32_t RG_WAIT_LIMIT = 1u << 22;      // polls of one barrier before the warp gives up

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
};

__device__ int g_ring_fault;

__device__ __forceinline__ uint32_t rg_smem(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }
__device__ __forceinline__ void rg_bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void rg_bar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool rg_bar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// global -> shared bulk copy (the TMA unit, untiled form); addresses and size are multiples of 16
__device__ __forceinline__ void rg_bulk_g2s(uint32_t dst, const void * src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void rg_cp_async16(uint32_t dst, const void * src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void rg_cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
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

__device__ __forceinline__ void rg_quantize(const float4 va, const float4 vb, int lane, RgBlockX & o) {
    const int g = lane >> 2, t = lane & 3;
    float amax = rg_absmax_nan(rg_absmax_nan(rg_absmax_nan(va.x, va.y), rg_absmax_nan(va.z, va.w)),
                               rg_absmax_nan(rg_absmax_nan(vb.x, vb.y), rg_absmax_nan(vb.z, vb.w)));
    float sum = ((va.x + va.y) + (va.z + va.w)) + ((vb.x + vb.y) + (vb.z + vb.w));
    amax = rg_absmax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    amax = rg_absmax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    float inv, s;
    act_group_scale(__float_as_uint(amax), inv, s);
    // round to nearest even without the conversion unit: 1.5 * 2^23 + v keeps the integer in the mantissa (|v| <= 32512),
    // integer = bits - 0x4B400000.  16-bit integer = 256 h + l with h, l signed bytes: h = (integer + 128) >> 8, l = its
    // low byte, which is also the low byte of `bits`.
    const int q0 = __float_as_int(fmaf(va.x, inv, 12582912.0f)), q1 = __float_as_int(fmaf(va.y, inv, 12582912.0f)),
              q2 = __float_as_int(fmaf(va.z, inv, 12582912.0f)), q3 = __float_as_int(fmaf(va.w, inv, 12582912.0f)),
              q4 = __float_as_int(fmaf(vb.x, inv, 12582912.0f)), q5 = __float_as_int(fmaf(vb.y, inv, 12582912.0f)),
              q6 = __float_as_int(fmaf(vb.z, inv, 12582912.0f)), q7 = __float_as_int(fmaf(vb.w, inv, 12582912.0f));
    constexpr int HB = 128 - 0x4B400000;
    const uint32_t h0 = __byte_perm(__byte_perm((uint32_t) ((q0 + HB) >> 8), (uint32_t) ((q1 + HB) >> 8), 0x0040),
                                    __byte_perm((uint32_t) ((q2 + HB) >> 8), (uint32_t) ((q3 + HB) >> 8), 0x0040), 0x5410);
    const uint32_t h1 = __byte_perm(__byte_perm((uint32_t) ((q4 + HB) >> 8), (uint32_t) ((q5 + HB) >> 8), 0x0040),
                                    __byte_perm((uint32_t) ((q6 + HB) >> 8), (uint32_t) ((q7 + HB) >> 8), 0x0040), 0x5410);
    const uint32_t l0 = __byte_perm(__byte_perm((uint32_t) q0, (uint32_t) q1, 0x0040), __byte_perm((uint32_t) q2, (uint32_t) q3, 0x0040), 0x5410);
    const uint32_t l1 = __byte_perm(__byte_perm((uint32_t) q4, (uint32_t) q5, 0x0040), __byte_perm((uint32_t) q6, (uint32_t) q7, 0x0040), 0x5410);
    // an even g holds the pair's low sub-block and supplies the h plane; an odd g the high sub-block and the l plane
    const bool odd = (g & 1) != 0;
    const uint32_t r0 = __shfl_xor_sync(0xffffffffu, odd ? h0 : l0, 4);
    const uint32_t r1 = __shfl_xor_sync(0xffffffffu, odd ? h1 : l1, 4);
    o.lo0 = odd ? r0 : h0;
    o.lo1 = odd ? r1 : h1;
    o.hi0 = odd ? l0 : r0;
    o.hi1 = odd ? l1 : r1;
    // C column pair of lane t = sub-blocks 2t (low nibbles of pair t) and 2t + 1: their scales sit in quads 2t, 2t + 1
    o.s0 = __shfl_sync(0xffffffffu, s, 8 * t);
    o.x0 = __shfl_sync(0xffffffffu, sum, 8 * t);
    o.s1 = __shfl_sync(0xffffffffu, s, 8 * t + 4);
    o.x1 = __shfl_sync(0xffffffffu, sum, 8 * t + 4);
}

// one row's share of a block for lane t (see iq_row_term of sm100_matvec_q4k_imma.cu)
__device__ __forceinline__ float rg_row_term(uint32_t dd, uint32_t f0, uint32_t f1, uint32_t shift, int clo_h, int clo_l, int chi_h, int chi_l,
                                             const RgBlockX & b) {
    const float2 df = __half22float2(*reinterpret_cast<const __half2 *>(&dd));   // d, dmin
    const uint32_t f = __funnelshift_r(f0, f1, shift);
    const int sc0 = (int) (f & 63u), m0 = (int) ((f >> 6) & 63u), sc1 = (int) ((f >> 12) & 63u), m1 = (int) ((f >> 18) & 63u);
    const int v0 = clo_h * 256 + clo_l;          // exact: |v0| < 2^24
    const int v1 = (chi_h * 256 + chi_l) >> 4;   // exact: every term carries the factor 16 of the high nibble
    const float dot = fmaf((float) (v1 * sc1), b.s1, (float) (v0 * sc0) * b.s0);
    const float mins = fmaf((float) m1, b.x1, (float) m0 * b.x0);
    return fmaf(df.x, dot, -df.y * mins);
}

// Shared memory of one CTA:
//   bars  [warp][RG_SLOTS] mbarrier
//   red   [RG_WINDOW][warp][16 rows] float     partial sums of the warps, one window of rounds
//   hdr   [warp][RG_SLOTS][16 rows] uint4      block headers of the units in flight (128-byte aligned)
//   ring  [warp][RG_SLOTS][4 tiles][512 B]     weight tiles of the units in flight
//   row   [K] float                            PRO == 2 only: the residual row before normalisation
// NBW: 256-weight blocks of K per warp (compile time: their activations live in registers).
// PRO: 0 x is given; 1 x = swiglu(pa, pb); 2 s = pa (+ pb), x = rms_norm(s) * pw (s, x written out by CTA 0 when asked).
template <int NBW, int PRO>
__global__ void __launch_bounds__(RG_THREADS, 2) matvec_q4k_ring(RingArgs p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t * bars = reinterpret_cast<uint64_t *>(smem);
    float * red = reinterpret_cast<float *>(smem + RG_WARPS * RG_SLOTS * 8);
    uint8_t * hdr = smem + RG_WARPS * RG_SLOTS * 8 + RG_WINDOW * RG_WARPS * 16 * 4;
    uint8_t * ring = hdr + RG_WARPS * RG_SLOTS * RG_HDR_BYTES;
    float * row = reinterpret_cast<float *>(ring + RG_WARPS * RG_SLOTS * RG_TILE_BYTES);

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

    const uint32_t bar0 = rg_smem(bars + wid * RG_SLOTS);
    const uint32_t hdr0 = rg_smem(hdr) + (uint32_t) wid * RG_SLOTS * RG_HDR_BYTES;
    const uint32_t ring0 = rg_smem(ring) + (uint32_t) wid * RG_SLOTS * RG_TILE_BYTES;
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < RG_SLOTS; ++s) rg_bar_init(bar0 + 8 * s, 33);   // lane 0's expect_tx + 32 header-copy arrivals
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // unit u of this warp = (round u / nb, block kw + wpt * (u % nb)); requests it into slot u % RG_SLOTS
    const uint32_t tile_bytes_per_rt = (uint32_t) p.blocks * RG_TILE_BYTES;
    const uint32_t hdr_bytes_per_rt = (uint32_t) p.blocks * 256u;
    auto request = [&](int u) {
        const int r = u / nb, i = u - r * nb;
        const int blk = kw + p.wpt * i;
        int ti, rt;
        rg_locate(p, tile0 + r * tile_step, ti, rt);
        const uint8_t * wbase = p.w[ti];
        const int s = u % RG_SLOTS;
        const uint32_t bar = bar0 + 8 * s;
        if (lane == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // earlier reads of the slot precede the copy's writes
            rg_bar_expect_tx(bar, RG_TILE_BYTES);
            rg_bulk_g2s(ring0 + s * RG_TILE_BYTES, wbase + (uint64_t) rt * tile_bytes_per_rt + (uint32_t) blk * RG_TILE_BYTES, RG_TILE_BYTES, bar);
        }
        if (lane < 16)
            rg_cp_async16(hdr0 + s * RG_HDR_BYTES + lane * 16,
                          wbase + p.h_off[ti] + (uint64_t) rt * hdr_bytes_per_rt + (uint32_t) (lane * p.blocks + blk) * 16u);
        rg_cp_async_arrive(bar);
    };
    int issued = 0;
    for (; issued < RG_SLOTS && issued < units; ++issued) request(issued);

    pdl_wait();   // everything below may depend on the predecessor's output

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
#pragma unroll
        for (int i = 0; i < NBW; ++i) {
            if (i < nb) {
                const int e0 = (kw + p.wpt * i) * 256 + g * 32 + 4 * t;   // element index of the lane's first float4
                float4 va = *reinterpret_cast<const float4 *>(row + e0), vb = *reinterpret_cast<const float4 *>(row + e0 + 16);
                const float4 wa = __ldg(reinterpret_cast<const float4 *>(p.pw + e0)), wb = __ldg(reinterpret_cast<const float4 *>(p.pw + e0 + 16));
                va = make_float4(__fmul_rn(__fmul_rn(va.x, scale), wa.x), __fmul_rn(__fmul_rn(va.y, scale), wa.y),
                                 __fmul_rn(__fmul_rn(va.z, scale), wa.z), __fmul_rn(__fmul_rn(va.w, scale), wa.w));
                vb = make_float4(__fmul_rn(__fmul_rn(vb.x, scale), wb.x), __fmul_rn(__fmul_rn(vb.y, scale), wb.y),
                                 __fmul_rn(__fmul_rn(vb.z, scale), wb.z), __fmul_rn(__fmul_rn(vb.w, scale), wb.w));
                if (p.x_out != nullptr && blockIdx.x == 0 && group == 0) {
                    *reinterpret_cast<float4 *>(p.x_out + e0) = va;
                    *reinterpret_cast<float4 *>(p.x_out + e0 + 16) = vb;
                }
                rg_quantize(va, vb, lane, bx[i]);
            }
        }
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
                rg_quantize(va[i], vb[i], lane, bx[i]);
            }
        }
    }

    // ---- main loop: this warp's units, round by round ----
    const int live_pair = g >> 1;
    // the 24-bit scale field of lane t starts at byte 4 + 3 t of a 16-byte header
    const uint32_t fld_off = (uint32_t) (4 + 3 * t) & ~3u, fld_shift = ((uint32_t) (4 + 3 * t) & 3u) * 8u;
    bool alive = true;
    int u = 0;
    // rounds of group 0, the most any group of this CTA has: the window loop and its barriers are CTA-uniform
    const int cta_rounds = (p.n_tiles - (int) blockIdx.x * p.groups + tile_step - 1) / tile_step;
    for (int base = 0; base < cta_rounds; base += RG_WINDOW) {
        const int wend = base + RG_WINDOW < rounds ? base + RG_WINDOW : rounds;
        for (int r = base; r < wend && alive; ++r) {
            float acc0 = 0.f, acc1 = 0.f;   // rows g and g + 8 of the tile
#pragma unroll
            for (int i = 0; i < NBW; ++i) {
                if (i < nb && alive) {
                    const int s = u % RG_SLOTS;
                    const uint32_t bar = bar0 + 8 * s, parity = (uint32_t) (u / RG_SLOTS) & 1u;
                    bool ok = rg_bar_try_wait(bar, parity);
                    for (uint32_t n = 0; !ok && n < RG_WAIT_LIMIT; ++n) ok = rg_bar_try_wait(bar, parity);
                    if (!__all_sync(0xffffffffu, ok)) {   // a copy that never lands must not hang the GPU
                        if (lane == 0) atomicExch(&g_ring_fault, 1);
                        alive = false;
                    } else {
                        const uint32_t tiles_lane = ring0 + s * RG_TILE_BYTES + lane * 16;
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
                        if (issued < units) { request(issued); ++issued; }
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
                int ti, lrt;
                rg_locate(p, tile, ti, lrt);
                p.y[ti][(int64_t) lrt * 16 + rw] = v;
            }
        }
        __syncthreads();
    }

    // copies that were requested but never consumed (only after a fault) must land before the CTA's memory goes away
    if (!alive) {
        for (int q = u; q < issued; ++q) {
            const uint32_t bar = bar0 + 8 * (q % RG_SLOTS), parity = (uint32_t) (q / RG_SLOTS) & 1u;
            for (uint32_t n = 0; n < RG_WAIT_LIMIT && !rg_bar_try_wait(bar, parity); ++n) {}
        }
    }
}

size_t ring_smem_bytes(int64_t k, int pro) {
    return (size_t) RG_WARPS * RG_SLOTS * 8 + (size_t) RG_WINDOW * RG_WARPS * 16 * 4 + (size_t) RG_WARPS * RG_SLOTS * (RG_HDR_BYTES + RG_TILE_BYTES) +
           (pro == 2 ? (size_t) k * 4 : 0);
}

std::atomic<bool> g_ring_launched[MAX_DEVICES];

template <int NBW>
int launch_ring(cudaStream_t s, const RingArgs & a, int pro, size_t smem, int grid) {
#define SM100_RING_CASE(P)                                                                                                             \
    case P:                                                                                                                            \
        SM100_CUDA(cudaFuncSetAttribute(matvec_q4k_ring<NBW, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024));          \
        return launch(matvec_q4k_ring<NBW, P>, dim3((unsigned) grid), dim3(RG_THREADS), smem, s, a);
    switch (pro) {
        SM100_RING_CASE(0)
        SM100_RING_CASE(1)
        SM100_RING_CASE(2)
    }
#undef SM100_RING_CASE
    return fail(ST_INVALID, "matvec (Q4_K ring): unknown prologue");
}

}  // namespace

int ring_poll_fault() {
    if (!g_ring_launched[current_device()].exchange(false, std::memory_order_relaxed)) return ST_OK;
    int v = 0;
    SM100_CUDA(cudaMemcpyFromSymbol(&v, g_ring_fault, sizeof(v)));
    if (v == 0) return ST_OK;
    const int zero = 0;
    SM100_CUDA(cudaMemcpyToSymbol(g_ring_fault, &zero, sizeof(zero)));
    return fail(ST_BACKEND, "mul_mat: the Q4_K ring matvec gave up waiting for a weight copy; its output is incomplete");
}

// Q4_K packed matvec, one activation column, over the full 16-row tiles of up to three tensors that share the
// activations; *handled = false when the shapes are left to the caller's other kernels.
int matvec_q4k_ring_multi(cudaStream_t s, int count, const void * const * ws, const int64_t * ns, int64_t k, const float * x,
                          float * const * ys, bool * handled, const Q4KPrologue * pro) {
    *handled = false;
    static const int enabled = [] { const char * e = getenv("SM100_Q4K_RING"); return e != nullptr ? atoi(e) : 1; }();
    if (!enabled) return ST_OK;
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
    const size_t smem = ring_smem_bytes(k, mode);
    g_ring_launched[current_device()].store(true, std::memory_order_relaxed);
    int st;
    if (nbw == 1) st = launch_ring<1>(s, a, mode, smem, (int) grid);
    else if (nbw == 2) st = launch_ring<2>(s, a, mode, smem, (int) grid);
    else st = launch_ring<3>(s, a, mode, smem, (int) grid);
    *handled = st == ST_OK;
    return st;
}

}  // namespace sm100
