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

#include <atomic>
#include <cstdlib>

namespace sm100 {

int device_scratch(int slot, size_t bytes, void ** out);

namespace {

constexpr int IQ_WARPS = 8;    // warps that share one row tile (they split K)
constexpr int IQ_GROUPS = 2;   // row tiles a CTA works on at a time
constexpr int IQ_THREADS = IQ_WARPS * IQ_GROUPS * 32;

// Up to three weight tensors that share the activations (MUL_MAT_MULTI: Q/K/V, gate/up) are handled as one
// concatenation of row tiles, so one launch quantizes x once and fills the machine even when a tensor is small.
constexpr int IQ_MAX_TENSORS = 3;

struct IqArgs {
    const uint8_t * w[IQ_MAX_TENSORS];   // packed tensor bases
    int64_t h_off[IQ_MAX_TENSORS];       // byte offset of each header plane
    float * y[IQ_MAX_TENSORS];           // [N_i, M], column stride ldy[i] floats
    int64_t ldy[IQ_MAX_TENSORS];
    int tile_end[IQ_MAX_TENSORS];        // row tiles of tensors 0..i together (INT32_MAX for unused slots)
    const float * x;     // [K, M], column stride ldx floats
    int64_t ldx;
    // producer of the activation column folded in (M = 1): 0 none; 1 x = swiglu(pa, pb); 2 s = pa (+ pb),
    // x = rms_norm(s) * pw, with s and x also written out (by CTA 0) when the pointers are set
    int prologue;
    const float * pa; const float * pb; const float * pw;
    float * sum_out; float * x_out;
    float eps;
    int n_tiles;         // full 16-row tiles of all tensors
    int pairs;           // K / 64
    int blocks;          // K / 256
    int chunks;          // ceil(blocks / blocks per chunk)
    int ring;            // slots per warp of the shared-memory ring
    // gate / up mode (M = 1, two tensors of equal row counts): the row tiles of the two tensors alternate (even tiles gate, odd
    // tiles up), so the two row groups of a CTA hold tile T of both at the same time and the epilogue writes
    // act = swiglu(gate, up) (src/core/ref/ops.cpp:383-425, the arithmetic of swiglu_kernel); y[0], y[1] are written too when set
    float * act;
};

__device__ __forceinline__ int nsb_of(const IqArgs & p) { return p.pairs * 2; }

// tensor of a global row tile and the tile's index inside it
__device__ __forceinline__ void iq_locate(const IqArgs & p, int rt, int & tensor, int & local) {
    if (p.act != nullptr) {   // gate / up mode: the tensors' tiles alternate
        tensor = rt & 1;
        local = rt >> 1;
        return;
    }
    tensor = (rt >= p.tile_end[0] ? 1 : 0) + (rt >= p.tile_end[1] ? 1 : 0);
    local = rt - (tensor == 0 ? 0 : p.tile_end[tensor - 1]);
}

__device__ __forceinline__ void imma_16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One row's share of a block for lane t: header words -> d, dmin and the scale field of sub-blocks 2t, 2t+1;
// clo / chi = (H, L) integer dot products of the low / high nibble sub-block (chi carries a factor 16).
// sq = (s_2t, sum_x_2t, s_2t+1, sum_x_2t+1).
struct IqHdr { uint32_t dd, f0, f1; };   // (d, dmin) halves; the two words around the lane's scale field

__device__ __forceinline__ float iq_row_term(const IqHdr & h, uint32_t shift, int clo_h, int clo_l, int chi_h, int chi_l, const float4 & sq) {
    const float2 df = __half22float2(*reinterpret_cast<const __half2 *>(&h.dd));   // d, dmin
    const uint32_t f = __funnelshift_r(h.f0, h.f1, shift);
    const int sc0 = (int) (f & 63u), m0 = (int) ((f >> 6) & 63u), sc1 = (int) ((f >> 12) & 63u), m1 = (int) ((f >> 18) & 63u);
    const int v0 = clo_h * 256 + clo_l;          // exact: |v0| < 2^24
    const int v1 = (chi_h * 256 + chi_l) >> 4;   // exact: every term is a multiple of 16
    const float dot = fmaf((float) (v1 * sc1), sq.z, (float) (v0 * sc0) * sq.x);
    const float mins = fmaf((float) m1, sq.w, (float) m0 * sq.y);
    return fmaf(df.x, dot, -df.y * mins);
}

// ---- shared-memory ring fed by the copy engine ----
__device__ __forceinline__ uint32_t iq_smem_addr(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }
__device__ __forceinline__ void iq_bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void iq_bar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool iq_bar_try_wait(uint32_t bar, uint32_t parity) {
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
// global -> shared bulk copy (TMA unit); addresses and size are multiples of 16
__device__ __forceinline__ void iq_bulk_g2s(uint32_t dst, const void * src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
// per-thread 16-byte asynchronous copy and its arrival on the slot's barrier
__device__ __forceinline__ void iq_cp_async16(uint32_t dst, const void * src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void iq_cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t iq_lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 iq_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
// first MMA of a block: the accumulator starts at zero
__device__ __forceinline__ void imma_16832_zero(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

constexpr uint32_t IQ_WAIT_LIMIT = 1u << 22;         // polls of one barrier before the warp gives up

__device__ int g_iq_fault;

// Shared memory of one CTA:
//   xq    [M][K/64][128 B]    quantized activations in B-fragment order: per pair [plane h, l][t][low sub-block b0, b1,
//                             high sub-block b0, b1], b0 = bytes of k = 4t..4t+3, b1 of k = 16+4t..; 16 zero bytes follow
//                             for the lanes whose fragment column holds no activation
//   xs    [M][K/64] float4    (s, sum x) of the low and of the high sub-block of each pair
//   red   [warp][16 rows][4] float   partial outputs of the warps of one row tile
//   bars  [warp][R] mbarrier
//   hdr   [warp][R][2 blocks][16 rows] uint4   block headers of the chunks in flight
//   ring  [warp][R][8 tiles][512 B]            weight tiles of the chunks in flight
// A warp owns R slots.  Lane 0 fills a slot with one bulk copy (the chunk's tiles are contiguous in the packed
// layout), all lanes add one 16-byte asynchronous copy of a block header, and both complete on the slot's barrier.
// The first R chunks are requested before griddepcontrol.wait: weights do not depend on the predecessor kernel.
// NB = 256-weight blocks per chunk: 2 with one CTA per SM, or 1 with two CTAs per SM (more warps to hide latencies,
// and one CTA's barriers overlap the other's arithmetic).
// FULL: K is a whole number of chunks (no block-range checks in the loops).
// CL = 2: the kernel runs in clusters of two CTAs (the two SMs of a TPC) that quantize half of the activation column
// each and store the result into both CTAs' shared memory (distributed shared memory), which halves the fixed
// cost every CTA pays before its first MMA.
template <int M, int NB, bool FULL, int CL>
__global__ void __launch_bounds__(IQ_THREADS, NB == 1 ? 2 : 1) matvec_q4k_imma(IqArgs p) {
    constexpr int IQ_TILES = 4 * NB;                    // pair tiles (64 weights each) per chunk
    constexpr uint32_t IQ_SLOT_BYTES = IQ_TILES * 512;  // weight tiles of one chunk
    constexpr uint32_t IQ_HDR_BYTES = 256 * NB;         // its NB x 16 block headers
    extern __shared__ __align__(128) uint8_t smem[];
    const int R = p.ring;
    const uint32_t xq_bytes = (uint32_t) M * p.pairs * 128;
    uint32_t * xq = reinterpret_cast<uint32_t *>(smem);
    float2 * xs2 = reinterpret_cast<float2 *>(smem + xq_bytes + 16);
    float * red = reinterpret_cast<float *>(smem + xq_bytes + 16 + (uint32_t) M * p.pairs * 16);
    uint64_t * bars = reinterpret_cast<uint64_t *>(red + IQ_WARPS * IQ_GROUPS * 64);
    uint8_t * hdr = reinterpret_cast<uint8_t *>(bars + IQ_WARPS * IQ_GROUPS * R);
    hdr += (128 - (iq_smem_addr(hdr) & 127)) & 127;
    uint8_t * ring = hdr + (uint32_t) IQ_WARPS * IQ_GROUPS * R * IQ_HDR_BYTES;

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int group = wid / IQ_WARPS, warp = wid % IQ_WARPS;
    const int g = lane >> 2, t = lane & 3;
    const int rt_step = gridDim.x * IQ_GROUPS;
    const uint32_t bar0 = iq_smem_addr(bars + wid * R);
    const uint32_t hdr0 = iq_smem_addr(hdr) + (uint32_t) wid * R * IQ_HDR_BYTES;
    const uint32_t ring0 = iq_smem_addr(ring) + (uint32_t) wid * R * IQ_SLOT_BYTES;

    if (lane == 0) {
        for (int s = 0; s < R; ++s) iq_bar_init(bar0 + 8 * s, 33);   // lane 0's expect_tx + 32 header copies
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // requests the chunk (rt, chunk) into slot s.  Per-lane constants keep the address work to a few operations.
    const uint32_t rt_tile_bytes = (uint32_t) p.pairs * 512u;         // tiles of one row tile
    const uint32_t rt_hdr_bytes = (uint32_t) p.blocks * 256u;         // headers of one row tile (16 rows)
    const uint32_t lane_hdr_off = (uint32_t) (lane & 15) * (uint32_t) p.blocks * 16u + (uint32_t) (lane >> 4) * 16u;
    auto request = [&](int rt_global, int chunk, int s) {
        int ti, rt;
        iq_locate(p, rt_global, ti, rt);
        const uint8_t * wbase = p.w[ti];
        const uint32_t bar = bar0 + 8 * s;
        if (lane == 0) {
            const int tiles = FULL ? IQ_TILES : (p.pairs - chunk * IQ_TILES < IQ_TILES ? p.pairs - chunk * IQ_TILES : IQ_TILES);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // earlier reads of the slot precede the copy's writes
            iq_bar_expect_tx(bar, (uint32_t) tiles * 512);
            iq_bulk_g2s(ring0 + s * IQ_SLOT_BYTES, wbase + (uint64_t) rt * rt_tile_bytes + (uint32_t) chunk * IQ_SLOT_BYTES, (uint32_t) tiles * 512, bar);
        }
        if (lane < 16 * NB && (FULL || NB * chunk + (lane >> 4) < p.blocks))
            iq_cp_async16(hdr0 + s * IQ_HDR_BYTES + lane * 16,
                          wbase + p.h_off[ti] + (uint64_t) rt * rt_hdr_bytes + lane_hdr_off + (uint32_t) chunk * (NB * 16u));
        iq_cp_async_arrive(bar);
    };

    // issue cursor: runs R chunks ahead of the consume cursor over the same sequence
    int irt = blockIdx.x * IQ_GROUPS + group, ichunk = warp, islot = 0;
    for (int i = 0; i < R; ++i) {
        if (irt < p.n_tiles && ichunk < p.chunks) {
            request(irt, ichunk, islot);
            if (++islot == R) islot = 0;
            ichunk += IQ_WARPS;
            if (ichunk >= p.chunks) { ichunk = warp; irt += rt_step; }
        }
    }

    pdl_wait();

    // activations -> 16-bit integers per 32-element sub-block.  One item = 4 consecutive elements; the 8 items of
    // a sub-block sit in 8 consecutive lanes.
    const int items = p.pairs * 16;
    if (tid < 4) xq[xq_bytes / 4 + tid] = 0u;
    // cluster peer's view of this CTA's shared-memory offsets (CL = 2 and a prologue that can be split)
    uint32_t cta_rank = 0;
    bool share = false;
    uint32_t peer_xq = 0, peer_xs = 0;
    if (CL == 2) {
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cta_rank));
        share = M == 1;
        const uint32_t peer = cta_rank ^ 1u;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer_xq) : "r"(iq_smem_addr(xq)), "r"(peer));
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer_xs) : "r"(iq_smem_addr(xs2)), "r"(peer));
    }
    // with sharing, this CTA takes every other group of 32 items (4 sub-blocks): local item li -> item it
    const int my_items = share ? items / 2 : items;
    auto item_of = [&](int li) { return share ? (((li >> 5) * 2 + (int) cta_rank) << 5) + (li & 31) : li; };
    auto quantize_item = [&](const float4 v, int m, int it) {
        const int sb = it >> 3, q = it & 7;
        uint32_t amax_bits = act_abs_bits(v);
        float sum = (v.x + v.y) + (v.z + v.w);
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, o));
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        float inv, s;
        act_group_scale(amax_bits, inv, s);
        // 16-bit integer = 256 h + l with h, l signed bytes: h = (x + 128) >> 8, l = x - 256 h
        // round to nearest (even) without the conversion unit: 1.5 * 2^23 + x keeps the integer in the mantissa (|x| <= 32512)
        const int x0 = __float_as_int(fmaf(v.x, inv, 12582912.0f)) - 0x4B400000, x1 = __float_as_int(fmaf(v.y, inv, 12582912.0f)) - 0x4B400000,
                  x2 = __float_as_int(fmaf(v.z, inv, 12582912.0f)) - 0x4B400000, x3 = __float_as_int(fmaf(v.w, inv, 12582912.0f)) - 0x4B400000;
        const int h0 = (x0 + 128) >> 8, h1 = (x1 + 128) >> 8, h2 = (x2 + 128) >> 8, h3 = (x3 + 128) >> 8;
        const uint32_t hp = __byte_perm(__byte_perm((uint32_t) h0, (uint32_t) h1, 0x0040), __byte_perm((uint32_t) h2, (uint32_t) h3, 0x0040), 0x5410);
        // the low bytes of x are the bytes of l (x - 256 h keeps the low byte)
        const uint32_t lp = __byte_perm(__byte_perm((uint32_t) x0, (uint32_t) x1, 0x0040), __byte_perm((uint32_t) x2, (uint32_t) x3, 0x0040), 0x5410);
        // word of the pair: plane * 16 + t * 4 + (high sub-block ? 2 : 0) + (k >= 16 ? 1 : 0)
        const uint32_t word = (uint32_t) (((size_t) m * p.pairs + (sb >> 1)) * 32 + (q & 3) * 4 + (sb & 1) * 2 + (q >> 2));
        xq[word] = hp;
        xq[word + 16] = lp;
        if (q == 0) xs2[(size_t) m * nsb_of(p) + sb] = make_float2(s, sum);
        if (CL == 2 && share) {
            asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer_xq + word * 4u), "r"(hp) : "memory");
            asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer_xq + (word + 16u) * 4u), "r"(lp) : "memory");
            if (q == 0)
                asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(peer_xs + (uint32_t) ((size_t) m * nsb_of(p) + sb) * 8u), "f"(s), "f"(sum)
                             : "memory");
        }
    };
    if (M > 1 || p.prologue == 0) {
        // all loads of a batch are issued before the first one is used: the row comes from L2 with one latency,
        // not one per loop trip (coherent loads: the producer may still be running when this kernel starts)
        constexpr int BATCH = 6;
        for (int base = 0; base < M * my_items; base += BATCH * IQ_THREADS) {
            float4 xv[BATCH];
#pragma unroll
            for (int i = 0; i < BATCH; ++i) {
                const int it0 = base + i * IQ_THREADS + tid;
                if (it0 < M * my_items) {
                    const int m = it0 / my_items, it = item_of(it0 - m * my_items);
                    xv[i] = __ldcg(reinterpret_cast<const float4 *>(p.x + (int64_t) m * p.ldx + (int64_t) it * 4));
                }
            }
#pragma unroll
            for (int i = 0; i < BATCH; ++i) {
                const int it0 = base + i * IQ_THREADS + tid;
                if (it0 < M * my_items) {   // warp-uniform: the item counts are multiples of 32
                    const int m = it0 / my_items, it = item_of(it0 - m * my_items);
                    quantize_item(xv[i], m, it);
                }
            }
        }
    } else if (p.prologue == 1) {
        // SwiGLU (src/core/ref/ops.cpp:383-425): (a / (1 + expf(-a))) * b, the arithmetic of swiglu_kernel
        constexpr int BATCH = 3;
        for (int base = 0; base < my_items; base += BATCH * IQ_THREADS) {
            float4 av[BATCH], bv[BATCH];
#pragma unroll
            for (int i = 0; i < BATCH; ++i) {
                const int li = base + i * IQ_THREADS + tid;
                if (li < my_items) {
                    av[i] = __ldcg(reinterpret_cast<const float4 *>(p.pa) + item_of(li));
                    bv[i] = __ldcg(reinterpret_cast<const float4 *>(p.pb) + item_of(li));
                }
            }
#pragma unroll
            for (int i = 0; i < BATCH; ++i) {
                const int li = base + i * IQ_THREADS + tid;
                const int it = item_of(li);
                if (li < my_items) {
                    const float4 a = av[i], b = bv[i];
                    float4 v;
                    v.x = __fmul_rn(__fdiv_rn(a.x, __fadd_rn(1.0f, expf(-a.x))), b.x);
                    v.y = __fmul_rn(__fdiv_rn(a.y, __fadd_rn(1.0f, expf(-a.y))), b.y);
                    v.z = __fmul_rn(__fdiv_rn(a.z, __fadd_rn(1.0f, expf(-a.z))), b.z);
                    v.w = __fmul_rn(__fdiv_rn(a.w, __fadd_rn(1.0f, expf(-a.w))), b.w);
                    quantize_item(v, 0, it);
                }
            }
        }
    } else {
        // (ADD_)RMS_NORM_MUL (src/core/ref/ops.cpp:466-519): every CTA (or pair of CTAs) normalises the row itself
        // (it reads it anyway); the row stays in registers between the two passes (the host bounds K for that)
        constexpr int MAXI = 4;
        float4 v[MAXI];
        double sq = 0.0;
        const bool writer = CL == 2 && share ? blockIdx.x < 2 : blockIdx.x == 0;   // who stores the side outputs
#pragma unroll
        for (int i = 0; i < MAXI; ++i) {
            const int li = tid + i * IQ_THREADS;
            const int it = item_of(li);
            v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (li < my_items) {
                v[i] = __ldcg(reinterpret_cast<const float4 *>(p.pa) + it);
                if (p.pb != nullptr) {
                    const float4 b = __ldcg(reinterpret_cast<const float4 *>(p.pb) + it);
                    v[i] = make_float4(__fadd_rn(v[i].x, b.x), __fadd_rn(v[i].y, b.y), __fadd_rn(v[i].z, b.z), __fadd_rn(v[i].w, b.w));
                }
                if (p.sum_out != nullptr && writer) reinterpret_cast<float4 *>(p.sum_out)[it] = v[i];
                sq += ((double) v[i].x * (double) v[i].x + (double) v[i].y * (double) v[i].y) +
                      ((double) v[i].z * (double) v[i].z + (double) v[i].w * (double) v[i].w);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        double * dred = reinterpret_cast<double *>(red);   // 16 + 2 doubles: the partial-output area is free before the first round
        if (lane == 0) dred[wid] = sq;
        __syncthreads();
        double tot = 0.0;
#pragma unroll
        for (int w = 0; w < IQ_WARPS * IQ_GROUPS; ++w) tot += dred[w];
        if (CL == 2 && share) {
            // the two CTAs exchange their halves of the sum of squares and add them in rank order (same bits in both)
            if (tid == 0) {
                dred[16 + cta_rank] = tot;
                uint32_t peer_slot;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer_slot) : "r"(iq_smem_addr(dred + 16 + cta_rank)), "r"(cta_rank ^ 1u));
                asm volatile("st.shared::cluster.f64 [%0], %1;" ::"r"(peer_slot), "d"(tot) : "memory");
            }
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
            tot = dred[16] + dred[17];
        }
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float) (tot / (double) (items * 4)), p.eps)));
#pragma unroll
        for (int i = 0; i < MAXI; ++i) {
            const int li = tid + i * IQ_THREADS;
            const int it = item_of(li);
            if (li < my_items) {   // warp-uniform: the item counts are multiples of 32
                const float4 w4 = __ldg(reinterpret_cast<const float4 *>(p.pw) + it);
                const float4 r = make_float4(__fmul_rn(__fmul_rn(v[i].x, scale), w4.x), __fmul_rn(__fmul_rn(v[i].y, scale), w4.y),
                                             __fmul_rn(__fmul_rn(v[i].z, scale), w4.z), __fmul_rn(__fmul_rn(v[i].w, scale), w4.w));
                if (p.x_out != nullptr && writer) reinterpret_cast<float4 *>(p.x_out)[it] = r;
                quantize_item(r, 0, it);
            }
        }
        __syncthreads();   // dred is part of `red`: everyone has read it before the rounds write there
    }
    if (CL == 2) {
        // both CTAs' halves are in place (release / acquire at cluster scope; also a barrier for this CTA's threads)
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    } else {
        __syncthreads();
    }
    pdl_launch_dependents();

    // per-lane views.  Pair j of a block feeds B columns 2j (h plane) and 2j+1 (l plane): lane (g, t) supplies
    // column g, so it reads plane g & 1 of pair g >> 1 and the zero bytes for the other pairs.
    const uint32_t xq0 = iq_smem_addr(xq);
    const uint32_t zero_addr = xq0 + xq_bytes;
    const uint32_t xq_live = xq0 + (uint32_t) (g >> 1) * 128 + (g & 1) * 64 + t * 16;   // + m * pairs * 128 + blk * 512
    const int live_pair = g >> 1;
    // the 24-bit scale field of lane t starts at byte 4 + 3 t of a 16-byte header
    const uint32_t fld_off = (uint32_t) (4 + 3 * t) & ~3u, fld_shift = ((uint32_t) (4 + 3 * t) & 3u) * 8u;
    const uint32_t xs0 = iq_smem_addr(xs2) + t * 16;
    float * my_red = red + group * (IQ_WARPS * 64);
    const int gtid = tid - group * (IQ_WARPS * 32);

    int rt = blockIdx.x * IQ_GROUPS + group, chunk = warp, cslot = 0;
    uint32_t cphase = 0;
    bool alive = true;

    // every group runs the same number of rounds so that the CTA-wide barriers match
    for (int round = blockIdx.x * IQ_GROUPS; round < p.n_tiles; round += rt_step) {
        float acc0[M], acc1[M];   // rows g and g + 8 of the tile
#pragma unroll
        for (int m = 0; m < M; ++m) acc0[m] = acc1[m] = 0.f;
        for (; alive && rt < p.n_tiles && chunk < p.chunks; chunk += IQ_WARPS) {
            // wait for the slot (bounded: a copy that never lands must not hang the GPU)
            {
                const uint32_t bar = bar0 + 8 * cslot;
                bool ok = iq_bar_try_wait(bar, cphase);
                for (uint32_t i = 0; !ok && i < IQ_WAIT_LIMIT; ++i) ok = iq_bar_try_wait(bar, cphase);
                if (!__all_sync(0xffffffffu, ok)) {
                    if (lane == 0) atomicExch(&g_iq_fault, 1);
                    alive = false;
                    break;
                }
            }
            const uint32_t tiles_lane = ring0 + cslot * IQ_SLOT_BYTES + lane * 16;
            const uint32_t hdr_lane = hdr0 + cslot * IQ_HDR_BYTES + g * 16;   // row g of the chunk's first block
#pragma unroll
            for (int b2 = 0; b2 < NB; ++b2) {
                const int blk = chunk * NB + b2;
                if (FULL || blk < p.blocks) {
                    int clo[M][4], chi[M][4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 wt = iq_lds128(tiles_lane + (b2 * 4 + j) * 512);   // x, y: row g k-halves 0, 1; z, w: row g + 8
#pragma unroll
                        for (int m = 0; m < M; ++m) {
                            const uint4 bf = iq_lds128(j == live_pair ? xq_live + (uint32_t) (m * p.pairs + blk * 4) * 128 : zero_addr);
                            if (j == 0) {
                                imma_16832_zero(clo[m], wt.x & 0x0F0F0F0Fu, wt.z & 0x0F0F0F0Fu, wt.y & 0x0F0F0F0Fu, wt.w & 0x0F0F0F0Fu, bf.x, bf.y);
                                imma_16832_zero(chi[m], wt.x & 0xF0F0F0F0u, wt.z & 0xF0F0F0F0u, wt.y & 0xF0F0F0F0u, wt.w & 0xF0F0F0F0u, bf.z, bf.w);
                            } else {
                                imma_16832(clo[m], wt.x & 0x0F0F0F0Fu, wt.z & 0x0F0F0F0Fu, wt.y & 0x0F0F0F0Fu, wt.w & 0x0F0F0F0Fu, bf.x, bf.y);
                                imma_16832(chi[m], wt.x & 0xF0F0F0F0u, wt.z & 0xF0F0F0F0u, wt.y & 0xF0F0F0F0u, wt.w & 0xF0F0F0F0u, bf.z, bf.w);
                            }
                        }
                    }
                    // per row: the (d, dmin) word and the two words that hold this lane's 24-bit scale field
                    const uint32_t ha = hdr_lane + b2 * 256, hb = ha + 128;
                    const IqHdr h0 = {iq_lds32(ha), iq_lds32(ha + fld_off), iq_lds32(ha + fld_off + 4)};
                    const IqHdr h1 = {iq_lds32(hb), iq_lds32(hb + fld_off), iq_lds32(hb + fld_off + 4)};
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        const uint4 sqb = iq_lds128(xs0 + (uint32_t) (m * p.pairs + blk * 4) * 16);
                        const float4 sq = make_float4(__uint_as_float(sqb.x), __uint_as_float(sqb.y), __uint_as_float(sqb.z), __uint_as_float(sqb.w));
                        acc0[m] += iq_row_term(h0, fld_shift, clo[m][0], clo[m][1], chi[m][0], chi[m][1], sq);
                        acc1[m] += iq_row_term(h1, fld_shift, clo[m][2], clo[m][3], chi[m][2], chi[m][3], sq);
                    }
                }
            }
            // the slot is consumed (its values sit in registers that the MMAs above have read): refill it
            __syncwarp();
            if (irt < p.n_tiles && ichunk < p.chunks) {
                request(irt, ichunk, cslot);
                ichunk += IQ_WARPS;
                if (ichunk >= p.chunks) { ichunk = warp; irt += rt_step; }
            }
            if (++cslot == R) { cslot = 0; cphase ^= 1u; }
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
        if (M == 1 && p.act != nullptr) {
            // group 0 holds tile T of gate, group 1 tile T of up (rt even / odd): one thread per row makes the activation
            if (group == 0 && gtid < 16 && rt + 1 < p.n_tiles) {
                const int row = gtid;
                float vg = 0.f, vu = 0.f;
#pragma unroll
                for (int w = 0; w < IQ_WARPS; ++w) {
                    vg += red[(w * 16 + row) * 4];
                    vu += red[IQ_WARPS * 64 + (w * 16 + row) * 4];
                }
                const int64_t at = (int64_t) (rt >> 1) * 16 + row;
                p.act[at] = __fmul_rn(__fdiv_rn(vg, __fadd_rn(1.0f, expf(-vg))), vu);
                if (p.y[0] != nullptr) p.y[0][at] = vg;
                if (p.y[1] != nullptr) p.y[1][at] = vu;
            }
        } else if (gtid < 64 && rt < p.n_tiles) {
            const int row = gtid >> 2, col = gtid & 3;
            if (col < M) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < IQ_WARPS; ++w) v += my_red[(w * 16 + row) * 4 + col];
                int ti, lrt;
                iq_locate(p, rt, ti, lrt);
                p.y[ti][(int64_t) col * p.ldy[ti] + (int64_t) lrt * 16 + row] = v;
            }
        }
        __syncthreads();
        rt += rt_step;
        chunk = warp;
    }

    // copies that were requested but never consumed (only after a fault) must land before the CTA's memory goes away
    if (!alive) {
        for (int s = 0; s < R; ++s)
            for (uint32_t i = 0; i < IQ_WAIT_LIMIT && !iq_bar_try_wait(bar0 + 8 * s, cphase); ++i) {}
    }
}

// ---------------------------------------------------------------------------------------------------------
// 3..8 activation columns: "tokens in columns".  The B operand's eight columns are the (h, l) planes of four
// tokens, so every lane supplies data and one MMA serves four tokens; each MMA covers one sub-block, whose scale is
// applied right away (lane (g, t) owns token t of the column group for rows g and g + 8 - no reduction inside the
// warp).  MG = column groups (1: up to 4 tokens, 2: up to 8).  One-block chunks keep the ring small next to the
// quantized activations of all tokens.
// ---------------------------------------------------------------------------------------------------------
// Quantizes the activation columns once for the whole launch that follows: the image has the shared-memory layout
// of matvec_q4k_imma_cols (per token and pair the B-fragment words, then (s, sum x) per sub-block), so that kernel
// fetches it with one bulk copy instead of having every CTA redo the work for every token.
__global__ void __launch_bounds__(256) q4k_quantize_cols(const float * x, int64_t ldx, int m_tokens, int mt, int pairs, uint32_t * img) {
    pdl_wait();
    pdl_launch_dependents();
    const int items = pairs * 16;
    // (scale, sum) pairs: one row of `pairs` 16-byte entries per token, padded by one entry so that the entries of the four
    // tokens a warp reads together lie in different shared-memory banks
    float2 * xs2 = reinterpret_cast<float2 *>(img + (size_t) mt * pairs * 32);
    for (int it0 = blockIdx.x * blockDim.x + threadIdx.x; it0 < mt * items; it0 += gridDim.x * blockDim.x) {   // whole warps: items is a multiple of 64
        const int m = it0 / items, it = it0 - m * items;
        const int sb = it >> 3, q = it & 7;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m < m_tokens) v = __ldcg(reinterpret_cast<const float4 *>(x + (int64_t) m * ldx + (int64_t) it * 4));
        uint32_t amax_bits = act_abs_bits(v);
        float sum = (v.x + v.y) + (v.z + v.w);
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, o));
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        float inv, s;
        act_group_scale(amax_bits, inv, s);
        const int x0 = __float_as_int(fmaf(v.x, inv, 12582912.0f)) - 0x4B400000, x1 = __float_as_int(fmaf(v.y, inv, 12582912.0f)) - 0x4B400000,
                  x2 = __float_as_int(fmaf(v.z, inv, 12582912.0f)) - 0x4B400000, x3 = __float_as_int(fmaf(v.w, inv, 12582912.0f)) - 0x4B400000;
        const int h0 = (x0 + 128) >> 8, h1 = (x1 + 128) >> 8, h2 = (x2 + 128) >> 8, h3 = (x3 + 128) >> 8;
        const uint32_t hp = __byte_perm(__byte_perm((uint32_t) h0, (uint32_t) h1, 0x0040), __byte_perm((uint32_t) h2, (uint32_t) h3, 0x0040), 0x5410);
        const uint32_t lp = __byte_perm(__byte_perm((uint32_t) x0, (uint32_t) x1, 0x0040), __byte_perm((uint32_t) x2, (uint32_t) x3, 0x0040), 0x5410);
        // per pair [plane][t][low sub-block b0, b1, high sub-block b0, b1]
        const size_t word = ((size_t) m * pairs + (sb >> 1)) * 32 + (q & 3) * 4 + (sb & 1) * 2 + (q >> 2);
        img[word] = hp;
        img[word + 16] = lp;
        if (q == 0) xs2[(size_t) m * (pairs + 1) * 2 + sb] = make_float2(s, sum);
    }
}

constexpr int IQ_SC_ROWS = 16 * 10;   // float2 entries of one warp's decoded scales: 16 rows of 8, padded to 10

template <int MG>
__global__ void __launch_bounds__(IQ_THREADS, 1) matvec_q4k_imma_cols(IqArgs p, int m_tokens, const uint32_t * img) {
    constexpr int MT = 4 * MG;                          // token slots
    constexpr uint32_t SLOT_BYTES = 4 * 512;            // weight tiles of one block
    constexpr uint32_t HDR_BYTES = 256;                 // its 16 block headers
    extern __shared__ __align__(128) uint8_t smem[];
    const int R = p.ring;
    const uint32_t xq_bytes = (uint32_t) MT * p.pairs * 128;
    uint32_t * xq = reinterpret_cast<uint32_t *>(smem);
    float2 * xs2 = reinterpret_cast<float2 *>(smem + xq_bytes);
    float * red = reinterpret_cast<float *>(smem + xq_bytes + (uint32_t) MT * (p.pairs + 1) * 16);   // [warp][16 rows][8 tokens]
    // [warp][16 rows][8 sub-blocks] (d sc, dmin m), rows 80 bytes apart: the eight rows a warp reads together cover all banks once
    float2 * scs = reinterpret_cast<float2 *>(red + IQ_WARPS * IQ_GROUPS * 128);
    uint64_t * bars = reinterpret_cast<uint64_t *>(scs + IQ_WARPS * IQ_GROUPS * IQ_SC_ROWS);   // [warp][R], then one for the activation image
    uint8_t * hdr = reinterpret_cast<uint8_t *>(bars + IQ_WARPS * IQ_GROUPS * R + 1);
    hdr += (128 - (iq_smem_addr(hdr) & 127)) & 127;
    uint8_t * ring = hdr + (uint32_t) IQ_WARPS * IQ_GROUPS * R * HDR_BYTES;
    const uint32_t img_bar = iq_smem_addr(bars + IQ_WARPS * IQ_GROUPS * R);

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int group = wid / IQ_WARPS, warp = wid % IQ_WARPS;
    const int g = lane >> 2, t = lane & 3;
    const int rt_step = gridDim.x * IQ_GROUPS;
    const uint32_t bar0 = iq_smem_addr(bars + wid * R);
    const uint32_t hdr0 = iq_smem_addr(hdr) + (uint32_t) wid * R * HDR_BYTES;
    const uint32_t ring0 = iq_smem_addr(ring) + (uint32_t) wid * R * SLOT_BYTES;

    if (lane == 0) {
        for (int s = 0; s < R; ++s) iq_bar_init(bar0 + 8 * s, 33);   // lane 0's expect_tx + 32 header arrivals
        if (tid == 0) iq_bar_init(img_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();   // the image barrier is polled by every thread

    const uint32_t rt_tile_bytes = (uint32_t) p.pairs * 512u, rt_hdr_bytes = (uint32_t) p.blocks * 256u;
    const uint32_t lane_hdr_off = (uint32_t) (lane & 15) * (uint32_t) p.blocks * 16u;
    auto request = [&](int rt, int blk, int s) {
        const uint32_t bar = bar0 + 8 * s;
        if (lane == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            iq_bar_expect_tx(bar, SLOT_BYTES);
            iq_bulk_g2s(ring0 + s * SLOT_BYTES, p.w[0] + (uint64_t) rt * rt_tile_bytes + (uint32_t) blk * SLOT_BYTES, SLOT_BYTES, bar);
        }
        if (lane < 16) iq_cp_async16(hdr0 + s * HDR_BYTES + lane * 16, p.w[0] + p.h_off[0] + (uint64_t) rt * rt_hdr_bytes + lane_hdr_off + (uint32_t) blk * 16u);
        iq_cp_async_arrive(bar);
    };
    int irt = blockIdx.x * IQ_GROUPS + group, iblk = warp, islot = 0;
    for (int i = 0; i < R; ++i) {
        if (irt < p.n_tiles && iblk < p.blocks) {
            request(irt, iblk, islot);
            if (++islot == R) islot = 0;
            iblk += IQ_WARPS;
            if (iblk >= p.blocks) { iblk = warp; irt += rt_step; }
        }
    }

    pdl_wait();

    // the quantized activation columns (made by q4k_quantize_cols, the predecessor on the stream): one bulk copy
    if (tid == 0) {
        const uint32_t bytes = xq_bytes + (uint32_t) MT * (p.pairs + 1) * 16;
        iq_bar_expect_tx(img_bar, bytes);
        iq_bulk_g2s(iq_smem_addr(xq), img, bytes, img_bar);
    }
    {
        bool ok = iq_bar_try_wait(img_bar, 0u);
        for (uint32_t i = 0; !ok && i < IQ_WAIT_LIMIT; ++i) ok = iq_bar_try_wait(img_bar, 0u);
        if (!ok) atomicExch(&g_iq_fault, 2);
    }
    pdl_launch_dependents();

    // lane (g, t) supplies B column g = plane (g & 1) of token (g >> 1) of each column group, and owns token t
    const uint32_t xq0 = iq_smem_addr(xq);
    const uint32_t xs0 = iq_smem_addr(xs2);
    float2 * my_sc = scs + wid * IQ_SC_ROWS;
    float * my_red = red + group * (IQ_WARPS * 128);
    const int gtid = tid - group * (IQ_WARPS * 32);

    int rt = blockIdx.x * IQ_GROUPS + group, blk = warp, cslot = 0;
    uint32_t cphase = 0;
    bool alive = true;
    for (int round = blockIdx.x * IQ_GROUPS; round < p.n_tiles; round += rt_step) {
        float acc0[MG], acc1[MG];   // rows g and g + 8, token t of each column group
#pragma unroll
        for (int cg = 0; cg < MG; ++cg) acc0[cg] = acc1[cg] = 0.f;
        for (; alive && rt < p.n_tiles && blk < p.blocks; blk += IQ_WARPS) {
            {
                const uint32_t bar = bar0 + 8 * cslot;
                bool ok = iq_bar_try_wait(bar, cphase);
                for (uint32_t i = 0; !ok && i < IQ_WAIT_LIMIT; ++i) ok = iq_bar_try_wait(bar, cphase);
                if (!__all_sync(0xffffffffu, ok)) {
                    if (lane == 0) atomicExch(&g_iq_fault, 1);
                    alive = false;
                    break;
                }
            }
            // decode the block's 16 headers for the warp: lane -> (row lane & 15, sub-blocks 4 (lane >> 4) .. + 3)
            {
                const uint4 h = iq_lds128(hdr0 + cslot * HDR_BYTES + (lane & 15) * 16);
                const float2 df = __half22float2(*reinterpret_cast<const __half2 *>(&h.x));
                const uint32_t f0 = lane < 16 ? h.y : __funnelshift_r(h.z, h.w, 16);            // field 0 or 2
                const uint32_t f1 = lane < 16 ? __funnelshift_r(h.y, h.z, 24) : h.w >> 8;         // field 1 or 3
                float2 * dst = my_sc + (lane & 15) * 10 + (lane >> 4) * 4;
                dst[0] = make_float2(df.x * (float) (f0 & 63u), df.y * (float) ((f0 >> 6) & 63u));
                dst[1] = make_float2(df.x * (float) ((f0 >> 12) & 63u), df.y * (float) ((f0 >> 18) & 63u));
                dst[2] = make_float2(df.x * (float) (f1 & 63u), df.y * (float) ((f1 >> 6) & 63u));
                dst[3] = make_float2(df.x * (float) ((f1 >> 12) & 63u), df.y * (float) ((f1 >> 18) & 63u));
            }
            __syncwarp();
            const uint32_t tiles_lane = ring0 + cslot * SLOT_BYTES + lane * 16;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 wt = iq_lds128(tiles_lane + j * 512);   // x, y: row g k-halves 0, 1; z, w: row g + 8
                const float4 sc0 = *reinterpret_cast<const float4 *>(my_sc + g * 10 + 2 * j);         // row g: (d sc, dmin m) of the pair's two sub-blocks
                const float4 sc1 = *reinterpret_cast<const float4 *>(my_sc + (g + 8) * 10 + 2 * j);   // row g + 8
                const float2 s_lo0 = make_float2(sc0.x, sc0.y), s_hi0 = make_float2(sc0.z, sc0.w);
                const float2 s_lo1 = make_float2(sc1.x, sc1.y), s_hi1 = make_float2(sc1.z, sc1.w);
#pragma unroll
                for (int cg = 0; cg < MG; ++cg) {
                    const uint32_t tok_b = (uint32_t) (cg * 4 + (g >> 1)), tok_c = (uint32_t) (cg * 4 + t);
                    const uint4 bf = iq_lds128(xq0 + (tok_b * p.pairs + (uint32_t) (blk * 4 + j)) * 128u + (uint32_t) (g & 1) * 64u + (uint32_t) t * 16u);
                    int clo[4], chi[4];
                    imma_16832_zero(clo, wt.x & 0x0F0F0F0Fu, wt.z & 0x0F0F0F0Fu, wt.y & 0x0F0F0F0Fu, wt.w & 0x0F0F0F0Fu, bf.x, bf.y);
                    imma_16832_zero(chi, wt.x & 0xF0F0F0F0u, wt.z & 0xF0F0F0F0u, wt.y & 0xF0F0F0F0u, wt.w & 0xF0F0F0F0u, bf.z, bf.w);
                    // (s, sum x) of the pair's two sub-blocks for the token this lane owns
                    const uint4 sqb = iq_lds128(xs0 + (tok_c * (uint32_t) (p.pairs + 1) + (uint32_t) (blk * 4 + j)) * 16u);
                    const float s_l = __uint_as_float(sqb.x), x_l = __uint_as_float(sqb.y), s_h = __uint_as_float(sqb.z), x_h = __uint_as_float(sqb.w);
                    const float vl0 = (float) (clo[0] * 256 + clo[1]), vl1 = (float) (clo[2] * 256 + clo[3]);
                    const float vh0 = (float) ((chi[0] * 256 + chi[1]) >> 4), vh1 = (float) ((chi[2] * 256 + chi[3]) >> 4);
                    acc0[cg] += (s_lo0.x * s_l) * vl0 - s_lo0.y * x_l + (s_hi0.x * s_h) * vh0 - s_hi0.y * x_h;
                    acc1[cg] += (s_lo1.x * s_l) * vl1 - s_lo1.y * x_l + (s_hi1.x * s_h) * vh1 - s_hi1.y * x_h;
                }
            }
            __syncwarp();
            if (irt < p.n_tiles && iblk < p.blocks) {
                request(irt, iblk, cslot);
                iblk += IQ_WARPS;
                if (iblk >= p.blocks) { iblk = warp; irt += rt_step; }
            }
            if (++cslot == R) { cslot = 0; cphase ^= 1u; }
        }
#pragma unroll
        for (int cg = 0; cg < MG; ++cg) {
            my_red[(warp * 16 + g) * 8 + cg * 4 + t] = acc0[cg];
            my_red[(warp * 16 + g + 8) * 8 + cg * 4 + t] = acc1[cg];
        }
        __syncthreads();
        if (gtid < 128 && rt < p.n_tiles) {
            const int row = gtid >> 3, col = gtid & 7;
            if (col < m_tokens && col < MT) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < IQ_WARPS; ++w) v += my_red[(w * 16 + row) * 8 + col];
                p.y[0][(int64_t) col * p.ldy[0] + (int64_t) rt * 16 + row] = v;
            }
        }
        __syncthreads();
        rt += rt_step;
        blk = warp;
    }
    if (!alive) {
        for (int s = 0; s < R; ++s)
            for (uint32_t i = 0; i < IQ_WAIT_LIMIT && !iq_bar_try_wait(bar0 + 8 * s, cphase); ++i) {}
    }
}

size_t iq_cols_smem_bytes(int pairs, int mt, int ring) {
    return (size_t) mt * (pairs * 128 + (pairs + 1) * 16) + (size_t) IQ_WARPS * IQ_GROUPS * 128 * 4 + (size_t) IQ_WARPS * IQ_GROUPS * IQ_SC_ROWS * 8 +
           (size_t) IQ_WARPS * IQ_GROUPS * ring * 8 + 8 + 128 + (size_t) IQ_WARPS * IQ_GROUPS * ring * (256 + 2048);
}

size_t iq_smem_bytes(int pairs, int m, int ring, int nb) {
    return (size_t) m * pairs * (128 + 16) + 16 + (size_t) IQ_WARPS * IQ_GROUPS * 64 * 4 + (size_t) IQ_WARPS * IQ_GROUPS * ring * 8 + 128 +
           (size_t) IQ_WARPS * IQ_GROUPS * ring * nb * (256 + 2048);
}

template <int M, int NB, bool FULL>
int launch_iq_full(cudaStream_t s, const IqArgs & a, size_t smem, int grid) {
    // always the device maximum: a smaller value set by a later launch would undercut kernel nodes already
    // recorded in a graph when a tool re-launches them
    static const int use_cluster = [] { const char * e = getenv("SM100_Q4K_CLUSTER"); return e != nullptr ? atoi(e) : 1; }();
    // measured: the pair pays off from K = 8192 on (K = 12288: 6440 -> 5270 cycles before the first MMA); below that the
    // cluster barrier and the remote stores cost more than the half row they save (K = 4096: 2240 -> 2850)
    if (use_cluster && M == 1 && NB == 2 && (use_cluster > 1 || a.pairs >= 128)) {
        if (smem > 48 * 1024)
            SM100_CUDA(cudaFuncSetAttribute(matvec_q4k_imma<M, NB, FULL, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        const int even = (grid + 1) & ~1;   // an extra CTA finds no row tile but still takes its half of the quantization
        return launch_cluster(matvec_q4k_imma<M, NB, FULL, 2>, dim3((unsigned) even), dim3(IQ_THREADS), smem, s, 2u, a);
    }
    if (smem > 48 * 1024)
        SM100_CUDA(cudaFuncSetAttribute(matvec_q4k_imma<M, NB, FULL, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    return launch(matvec_q4k_imma<M, NB, FULL, 1>, dim3((unsigned) grid), dim3(IQ_THREADS), smem, s, a);
}

template <int M, int NB>
int launch_iq(cudaStream_t s, const IqArgs & a, size_t smem, int grid) {
    return a.blocks % NB == 0 ? launch_iq_full<M, NB, true>(s, a, smem, grid) : launch_iq_full<M, NB, false>(s, a, smem, grid);
}

std::atomic<bool> g_iq_launched[MAX_DEVICES];   // per device, see sm100_common.cuh

}  // namespace


// Reads and clears the kernel's fault flag on the current device (set when a warp gave up waiting for a copy);
// called after a stream synchronisation.
int iq_poll_fault() {
    if (!g_iq_launched[current_device()].exchange(false, std::memory_order_relaxed)) return ST_OK;
    int v = 0;
    SM100_CUDA(cudaMemcpyFromSymbol(&v, g_iq_fault, sizeof(v)));
    if (v == 0) return ST_OK;
    const int zero = 0;
    SM100_CUDA(cudaMemcpyToSymbol(g_iq_fault, &zero, sizeof(zero)));
    return fail(ST_BACKEND, "mul_mat: the Q4_K matvec gave up waiting for a weight copy; its output is incomplete");
}

// Q4_K packed matvec (1 or 2 activation columns) over the full 16-row tiles of up to three tensors that share
// the activations; *handled = false when the shapes are left to the caller's other kernels.
// glu_out (optional): ws are the gate and up tensors (equal row counts, one column); glu_out receives swiglu(gate, up), ys[0]
// and ys[1] the projections themselves when they are non-null.
int matvec_q4k_imma_multi(cudaStream_t s, int count, const void * const * ws, const int64_t * ns, int64_t k, const float * x, int64_t ldx,
                          int64_t m, float * const * ys, const int64_t * ldys, bool * handled, const Q4KPrologue * pro, float * glu_out) {
    *handled = false;
    if (glu_out != nullptr && (count != 2 || m != 1 || ns[0] != ns[1] || ns[0] % 16 != 0 || ((uintptr_t) glu_out & 15) != 0)) return ST_OK;
    if (pro != nullptr && pro->mode != 0) {
        if (m != 1 || pro->a == nullptr) return ST_OK;
        const uintptr_t al = (uintptr_t) pro->a | (uintptr_t) pro->b | (uintptr_t) pro->norm_w | (uintptr_t) pro->sum_out | (uintptr_t) pro->x_out;
        if ((al & 15) != 0) return ST_OK;
        if (pro->mode == 1 && pro->b == nullptr) return ST_OK;
        if (pro->mode == 2 && (pro->norm_w == nullptr || k > 4 * 4 * IQ_THREADS)) return ST_OK;   // the row must fit the registers of one CTA
        x = pro->a;   // alignment checks below
    }
    if (count < 1 || count > IQ_MAX_TENSORS || m < 1 || m > 2 || k % 256 != 0 || k / 64 > 4096) return ST_OK;
    if (((uintptr_t) x & 15) != 0 || (m > 1 && (ldx & 3) != 0)) return ST_OK;
    int64_t tiles = 0;
    for (int i = 0; i < count; ++i) {
        if (ns[i] / 16 == 0 || ((uintptr_t) ws[i] & 15) != 0) return ST_OK;
        if (count > 1 && ns[i] % 16 != 0) return ST_OK;   // leftover rows are the single-tensor caller's business
        tiles += ns[i] / 16;
    }
    if (tiles > INT32_MAX / 2) return ST_OK;
    const int pairs = (int) (k / 64);
    // two CTAs per SM with one-block chunks on request, else one CTA per SM with two-block chunks
    static const int forced_nb = [] { const char * e = getenv("SM100_Q4K_NB"); return e != nullptr ? atoi(e) : 0; }();
    const int nb = forced_nb == 1 ? 1 : 2;
    int ring = 4;
    const size_t per_cta = nb == 1 ? (size_t) 113 * 1024 : (size_t) 227 * 1024;
    while (ring >= 2 && iq_smem_bytes(pairs, (int) m, ring, nb) > per_cta) --ring;
    if (ring < 2) return ST_OK;
    const size_t smem = iq_smem_bytes(pairs, (int) m, ring, nb);
    IqArgs a = {};
    int end = 0;
    for (int i = 0; i < IQ_MAX_TENSORS; ++i) {
        if (i < count) {
            a.w[i] = (const uint8_t *) ws[i];
            a.h_off[i] = ns[i] * (k / 256) * 128;
            a.y[i] = ys[i];
            a.ldy[i] = ldys[i];
            end += (int) (ns[i] / 16);
            a.tile_end[i] = end;
        } else {
            a.tile_end[i] = INT32_MAX;
        }
    }
    a.x = x;
    a.ldx = ldx;
    a.act = glu_out;
    if (pro != nullptr && pro->mode != 0) {
        a.prologue = pro->mode;
        a.pa = pro->a; a.pb = pro->b; a.pw = pro->norm_w; a.sum_out = pro->sum_out; a.x_out = pro->x_out; a.eps = pro->eps;
    }
    a.n_tiles = (int) tiles;
    a.pairs = pairs;
    a.blocks = (int) (k / 256);
    a.chunks = (a.blocks + nb - 1) / nb;
    a.ring = ring;
    int64_t grid = (int64_t) sm_count() * (nb == 1 ? 2 : 1);   // resident CTAs: each quantizes the activations once
    const int64_t rounds = (tiles + IQ_GROUPS - 1) / IQ_GROUPS;
    if (grid > rounds) grid = rounds;
    g_iq_launched[current_device()].store(true, std::memory_order_relaxed);
    int st;
    if (nb == 1) st = m == 1 ? launch_iq<1, 1>(s, a, smem, (int) grid) : launch_iq<2, 1>(s, a, smem, (int) grid);
    else st = m == 1 ? launch_iq<1, 2>(s, a, smem, (int) grid) : launch_iq<2, 2>(s, a, smem, (int) grid);
    *handled = st == ST_OK;
    return st;
}

// 3..8 activation columns of one packed Q4_K tensor over its full 16-row tiles; *handled = false when the shape
// (or the shared memory the quantized columns need) is left to the caller's other kernels.
int matvec_q4k_imma_cols_tiles(cudaStream_t s, const void * w, int64_t k, int64_t n, const float * x, int64_t ldx, int64_t m, float * y, int64_t ldy,
                               bool * handled) {
    *handled = false;
    const int64_t tiles = n / 16;
    if (tiles == 0 || m < 3 || m > 8 || k % 256 != 0 || k / 64 > 4096 || tiles > INT32_MAX / 2) return ST_OK;
    if (((uintptr_t) w & 15) != 0 || ((uintptr_t) x & 15) != 0 || (ldx & 3) != 0) return ST_OK;
    const int pairs = (int) (k / 64);
    const int mg = m > 4 ? 2 : 1;
    int ring = 4;
    while (ring >= 2 && iq_cols_smem_bytes(pairs, 4 * mg, ring) > (size_t) 227 * 1024) --ring;
    if (ring < 2) return ST_OK;
    const size_t smem = iq_cols_smem_bytes(pairs, 4 * mg, ring);
    IqArgs a = {};
    a.w[0] = (const uint8_t *) w;
    a.h_off[0] = n * (k / 256) * 128;
    a.y[0] = y;
    a.ldy[0] = ldy;
    a.tile_end[0] = (int) tiles;
    a.tile_end[1] = a.tile_end[2] = INT32_MAX;
    a.x = x;
    a.ldx = ldx;
    a.n_tiles = (int) tiles;
    a.pairs = pairs;
    a.blocks = (int) (k / 256);
    a.chunks = a.blocks;
    a.ring = ring;
    int64_t grid = sm_count();
    const int64_t rounds = (tiles + IQ_GROUPS - 1) / IQ_GROUPS;
    if (grid > rounds) grid = rounds;
    g_iq_launched[current_device()].store(true, std::memory_order_relaxed);
    const int mt = 4 * mg;
    void * img = nullptr;
    int st = device_scratch(2, (size_t) mt * (pairs * 128 + (pairs + 1) * 16), &img);
    if (st != ST_OK) return st;
    const int q_items = mt * pairs * 16;
    st = launch(q4k_quantize_cols, dim3((unsigned) ((q_items + 255) / 256)), dim3(256), 0, s, x, ldx, (int) m, mt, pairs, (uint32_t *) img);
    if (st != ST_OK) return st;
    if (mg == 1) {
        SM100_CUDA(cudaFuncSetAttribute(matvec_q4k_imma_cols<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        st = launch(matvec_q4k_imma_cols<1>, dim3((unsigned) grid), dim3(IQ_THREADS), smem, s, a, (int) m, (const uint32_t *) img);
    } else {
        SM100_CUDA(cudaFuncSetAttribute(matvec_q4k_imma_cols<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        st = launch(matvec_q4k_imma_cols<2>, dim3((unsigned) grid), dim3(IQ_THREADS), smem, s, a, (int) m, (const uint32_t *) img);
    }
    *handled = st == ST_OK;
    return st;
}

int matvec_q4k_imma_tiles(cudaStream_t s, const void * w, int64_t k, int64_t n, const float * x, int64_t ldx, int64_t m, float * y, int64_t ldy,
                          bool * handled) {
    return matvec_q4k_imma_multi(s, 1, &w, &n, k, x, ldx, m, &y, &ldy, handled, nullptr, nullptr);
}

}  // namespace sm100
