// Prefill MUL_MAT (M > 8 activation columns) on the fifth-generation tensor cores.
//
//   y[N, M] = W[K, N] . x[K, M]      W quantized (Q8_0, Q4_0, Q4_K) or F16, x and y f32
//
// replaces the reference's tiled GEMM (src/backends/opencl11/kernels/mul_mm.cl:271, dispatched from
// src/backends/opencl11/opencl_api.cpp for batches above the matvec limit) and has to agree with the CPU
// reference (src/core/ref/ops.cpp:891-984) to NMSE <= 1e-6.
//
// Two launches per call:
//
//  1. gemm_prep_x   converts the activations to f16 once, normalised per token by a power of two (so the
//                   largest element of a token sits in [8192, 16384) whatever its magnitude), and writes
//                   them in the shared-memory image the tensor core wants: per (token tile, 64-wide K chunk)
//                   one contiguous block of 8-token x 16-byte core matrices.  A consumer CTA then fetches a
//                   whole B stage with one bulk copy (cp.async.bulk, completion on an mbarrier).
//
//  2. gemm_tc       one CTA per 128 weight rows x TN tokens.  Warps 0-7 dequantize the weights of the
//                   CTA's rows chunk by chunk into f16 core matrices in shared memory (the A operand;
//                   weights are multiplied by 256 to keep small scales out of the f16 subnormals), warp 8
//                   issues the bulk copies of the B operand, one thread of warp 9 issues tcgen05.mma
//                   (kind::f16, 128 x TN x 16 per instruction) into a TMEM accumulator of TN columns and
//                   commits each stage back to the producers.  When the last commit lands, warps 0-7
//                   read the accumulator with tcgen05.ld, undo the two scalings and store y.
//
// f16 operands with f32 accumulation: each product carries two roundings of 2^-11 relative size, which
// puts the NMSE near 2e-7.  Every wait on an mbarrier is bounded; a CTA that gives up raises a fault flag
// (reported by the next stream synchronisation), drains its copies, frees its TMEM and returns.
#include "sm100_common.cuh"
#include "sm100_layout.h"

#include <atomic>
#include <cstdlib>
#include <mutex>
#include <vector>

namespace sm100 {

int device_scratch(int slot, size_t bytes, void ** out);

namespace {

constexpr int TM = 128;            // weight rows per CTA = rows of one tcgen05.mma = TMEM lanes
// Warp roles.  The MMA warp is warp 0: the scheduler favours older warps, and a young MMA warp was starved
// by the polling producers (each of its instructions took 50-80 cycles to issue).
constexpr int WARP_MMA = 0;        // owns TMEM and issues the MMAs
constexpr int WARP_BULK = 1;       // issues the bulk copies of the activation stages
constexpr int FIRST_PRODUCER = 2;  // warps 2-17 dequantize, then run the epilogue
constexpr int PRODUCER_WARPS = 16; // 512 threads = 512 (row, 32-weight block) tasks: one chunk of 128 K, or two of 64
constexpr int GEMM_THREADS = 32 * (FIRST_PRODUCER + PRODUCER_WARPS);
constexpr float W_PRESCALE = 256.0f;  // applied to quantized weights before they are rounded to f16
constexpr uint32_t WAIT_LIMIT = 1u << 21;  // polls of one mbarrier wait before the CTA gives up (~1 s)

__device__ int g_gemm_fault;  // 0, or 1 + the wait site that gave up


// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
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
// Bounded wait.  Returns false when the CTA is giving up (this wait ran out, or another one did).
// Waiters off the critical path (`patient`) sleep between polls so that they leave the issue slots alone.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int * abort_flag, int site, bool patient = true) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (patient || i >= 64) {
            if (*abort_flag != 0) return false;
            __nanosleep(patient ? 100 : 32);
        }
    }
    *abort_flag = 1 + site;
    atomicCAS(&g_gemm_fault, 0, 1 + site);
    return false;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// global -> shared bulk copy through the TMA unit; src, dst and bytes are multiples of 16
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void * src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}

// Shared-memory matrix descriptor of a K-major operand without swizzle (8-row x 16-byte core matrices), as two
// words.  Low: bits 0-13 start address >> 4, bits 16-29 (bytes between the two core matrices an instruction
// spans along K) >> 4.  High: bits 0-13 (bytes between 8-row groups) >> 4, bit 14 = descriptor version of sm_100;
// base offset, swizzle mode = 0.
// Instruction descriptor of kind::f16: f16 A and B, both K-major, f32 accumulator, M x N tile.
__host__ __device__ constexpr uint32_t instr_desc_f16(int m, int n) {
    return (1u << 4) | ((uint32_t) (n >> 3) << 17) | ((uint32_t) (m >> 4) << 24);
}
// D[tmem] (+)= A . B^T; both descriptors share their high word (same 8-row-group stride and version)
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives on `bar` when every MMA this thread issued so far has finished reading shared memory and writing TMEM
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 16 consecutive f32 columns of the accumulator: thread i of the warp receives lane (base lane + i)
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// Weight sources: 32 consecutive weights of one row (K block `kb` of 32) as 16 half2, times 256.
// load() only issues the global loads, so the caller can keep one block in flight while it converts
// the previous one.
// ---------------------------------------------------------------------------------------------
struct WeightRef {
    const uint8_t * base;
    Planes planes;       // packed layout
    int64_t row_stride;  // natural layout: bytes between rows
    int64_t blocks_per_row;
};

__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

// unsigned bytes b0, b1 of `w` (selected by `sel`) -> half2 (1024 + b0, 1024 + b1)
__device__ __forceinline__ __half2 bytes_to_h2_1024(uint32_t w, uint32_t sel) { return bits_h2(__byte_perm(w, 0x64646464u, sel)); }

__device__ __forceinline__ uint32_t ld_u16_any(const uint8_t * p) { return __ldg((const unsigned short *) p); }

template <bool PACKED>
struct SrcQ80 {
    static constexpr float PRESCALE = W_PRESCALE;
    struct Regs { uint32_t q[8]; uint32_t d; };
    __device__ static __forceinline__ void load(Regs & r, const WeightRef & W, int64_t row, int kb) {
        if (PACKED) {
            const int64_t t = row * W.blocks_per_row + kb;
            asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"  // 32-byte aligned: tensor base is
                         : "=r"(r.q[0]), "=r"(r.q[1]), "=r"(r.q[2]), "=r"(r.q[3]), "=r"(r.q[4]), "=r"(r.q[5]), "=r"(r.q[6]), "=r"(r.q[7])
                         : "l"(W.base + W.planes.off[0] + t * 32));
            r.d = ld_u16_any(W.base + W.planes.off[1] + t * 2);
        } else {
            const uint8_t * blk = W.base + row * W.row_stride + (int64_t) kb * 34;  // 2-byte aligned
            r.d = ld_u16_any(blk);
#pragma unroll
            for (int i = 0; i < 8; ++i) r.q[i] = ld_u16_any(blk + 2 + 4 * i) | ld_u16_any(blk + 4 + 4 * i) << 16;
        }
    }
    __device__ static __forceinline__ void convert(const Regs & r, uint32_t (&out)[16]) {
        const __half2 d2 = __half2half2(__float2half_rn(__half2float(__ushort_as_half((unsigned short) r.d)) * W_PRESCALE));
        const __half2 bias = __float2half2_rn(1152.0f);  // 1024 + 128
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t u = r.q[i] ^ 0x80808080u;  // int8 + 128
            out[2 * i] = h2_bits(__hmul2(__hsub2(bytes_to_h2_1024(u, 0x4140u), bias), d2));
            out[2 * i + 1] = h2_bits(__hmul2(__hsub2(bytes_to_h2_1024(u, 0x4342u), bias), d2));
        }
    }
};

template <bool PACKED>
struct SrcQ40 {
    static constexpr float PRESCALE = W_PRESCALE;
    struct Regs { uint32_t q[4]; uint32_t d; };
    __device__ static __forceinline__ void load(Regs & r, const WeightRef & W, int64_t row, int kb) {
        if (PACKED) {
            const int64_t t = row * W.blocks_per_row + kb;
            const uint4 a = __ldg((const uint4 *) (W.base + W.planes.off[0] + t * 16));
            r.q[0] = a.x; r.q[1] = a.y; r.q[2] = a.z; r.q[3] = a.w;
            r.d = ld_u16_any(W.base + W.planes.off[1] + t * 2);
        } else {
            const uint8_t * blk = W.base + row * W.row_stride + (int64_t) kb * 18;
            r.d = ld_u16_any(blk);
#pragma unroll
            for (int i = 0; i < 4; ++i) r.q[i] = ld_u16_any(blk + 2 + 4 * i) | ld_u16_any(blk + 4 + 4 * i) << 16;
        }
    }
    // weight i (< 16) is the low nibble of byte i, weight 16 + i its high nibble; value = (nibble - 8) * d
    __device__ static __forceinline__ void convert(const Regs & r, uint32_t (&out)[16]) {
        const __half2 d2 = __half2half2(__float2half_rn(__half2float(__ushort_as_half((unsigned short) r.d)) * W_PRESCALE));
        const __half2 bias = __float2half2_rn(1032.0f);  // 1024 + 8
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t p0 = __byte_perm(r.q[i], 0u, 0x4140u);  // b0 | b1 << 16
            const uint32_t p1 = __byte_perm(r.q[i], 0u, 0x4342u);  // b2 | b3 << 16
            out[2 * i] = h2_bits(__hmul2(__hsub2(bits_h2((p0 & 0x000f000fu) | 0x64006400u), bias), d2));
            out[2 * i + 1] = h2_bits(__hmul2(__hsub2(bits_h2((p1 & 0x000f000fu) | 0x64006400u), bias), d2));
            out[8 + 2 * i] = h2_bits(__hmul2(__hsub2(bits_h2(((p0 >> 4) & 0x000f000fu) | 0x64006400u), bias), d2));
            out[8 + 2 * i + 1] = h2_bits(__hmul2(__hsub2(bits_h2(((p1 >> 4) & 0x000f000fu) | 0x64006400u), bias), d2));
        }
    }
};

// F16 weights: rows of K halves, 2-byte aligned at worst
struct SrcF16 {
    static constexpr float PRESCALE = 1.0f;
    struct Regs { uint32_t h[16]; };
    __device__ static __forceinline__ void load(Regs & r, const WeightRef & W, int64_t row, int kb) {
        const uint8_t * p = W.base + row * W.row_stride + (int64_t) kb * 64;
        if ((((uintptr_t) p) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 a = __ldg((const uint4 *) p + i);
                r.h[4 * i] = a.x; r.h[4 * i + 1] = a.y; r.h[4 * i + 2] = a.z; r.h[4 * i + 3] = a.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) r.h[i] = ld_u16_any(p + 4 * i) | ld_u16_any(p + 4 * i + 2) << 16;
        }
    }
    __device__ static __forceinline__ void convert(const Regs & r, uint32_t (&out)[16]) {
#pragma unroll
        for (int i = 0; i < 16; ++i) out[i] = r.h[i];  // already f16: used as they are, no prescale
    }
};

// Q4_K, packed layout only.  K block kb = 8 * block + sub; sub-blocks 2p (low nibbles) and 2p + 1 (high
// nibbles) share the 32 quant bytes of pair p, which the tile-ordered Q plane spreads over four lanes.
struct SrcQ4K {
    static constexpr float PRESCALE = W_PRESCALE;
    struct Regs { uint32_t q[8]; uint4 h; };
    __device__ static __forceinline__ void load(Regs & r, const WeightRef & W, int64_t row, int kb) {
        const int64_t b = kb >> 3;
        const int pair = (kb & 7) >> 1;
        const Planes & P = W.planes;
        const int64_t full = (P.n_rows / 16) * 16;
        if (row < full) {
            const uint8_t * tile = W.base + P.off[0] + ((row >> 4) * (P.blocks_per_row * 4) + b * 4 + pair) * 512 + (row & 7) * 64 +
                                   ((row >> 3) & 1) * 8;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const uint2 v = __ldg((const uint2 *) (tile + t * 16));  // bytes [4t, 4t+4) and [16+4t, 16+4t+4) of the pair
                r.q[t] = v.x;
                r.q[4 + t] = v.y;
            }
        } else {
            const uint4 * src = (const uint4 *) (W.base + P.off[0] + full * P.blocks_per_row * 128 +
                                                 ((row - full) * P.blocks_per_row + b) * 128 + pair * 32);
            const uint4 a = __ldg(src), c = __ldg(src + 1);
            r.q[0] = a.x; r.q[1] = a.y; r.q[2] = a.z; r.q[3] = a.w;
            r.q[4] = c.x; r.q[5] = c.y; r.q[6] = c.z; r.q[7] = c.w;
        }
        r.h = __ldg((const uint4 *) (W.base + P.off[1] + (row * P.blocks_per_row + b) * 16));
    }
    __device__ static __forceinline__ void convert(const Regs & r, int kb, uint32_t (&out)[16]) {
        const int sub = kb & 7;
        const float d = __half2float(__ushort_as_half((unsigned short) (r.h.x & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short) (r.h.x >> 16)));
        // four 24-bit fields follow d and dmin: field p = sc[2p] | m[2p] << 6 | sc[2p+1] << 12 | m[2p+1] << 18
        uint32_t field;
        switch (sub >> 1) {
            case 0: field = r.h.y; break;
            case 1: field = __funnelshift_r(r.h.y, r.h.z, 24); break;
            case 2: field = __funnelshift_r(r.h.z, r.h.w, 16); break;
            default: field = r.h.w >> 8; break;
        }
        field = (field >> ((sub & 1) * 12)) & 0xfffu;
        const float sc = (float) (field & 63u), mn = (float) (field >> 6);
        const __half2 d1 = __float2half2_rn(d * sc * W_PRESCALE);
        const __half2 m1 = __float2half2_rn(-(dmin * mn * W_PRESCALE));
        const __half2 bias = __float2half2_rn(1024.0f);
        const int shift = (sub & 1) * 4;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t w = r.q[i] >> shift;
            const uint32_t p0 = __byte_perm(w, 0u, 0x4140u), p1 = __byte_perm(w, 0u, 0x4342u);
            out[2 * i] = h2_bits(__hfma2(__hsub2(bits_h2((p0 & 0x000f000fu) | 0x64006400u), bias), d1, m1));
            out[2 * i + 1] = h2_bits(__hfma2(__hsub2(bits_h2((p1 & 0x000f000fu) | 0x64006400u), bias), d1, m1));
        }
    }
};

// uniform call shape over the sources
template <typename S>
struct SrcTraits {
    __device__ static __forceinline__ void convert(const typename S::Regs & r, int, uint32_t (&out)[16]) { S::convert(r, out); }
};
template <>
struct SrcTraits<SrcQ4K> {
    __device__ static __forceinline__ void convert(const SrcQ4K::Regs & r, int kb, uint32_t (&out)[16]) { SrcQ4K::convert(r, kb, out); }
};

// ---------------------------------------------------------------------------------------------
// Shared memory of one CTA
// ---------------------------------------------------------------------------------------------
template <int TN, int KC, int STAGES>
struct GemmSmem {
    static constexpr int A_BYTES = TM * KC * 2;
    static constexpr int B_BYTES = TN * KC * 2;
    uint8_t a[STAGES][A_BYTES];  // [k / 8][row][8 halves]
    uint8_t b[STAGES][B_BYTES];  // [k / 8][token][8 halves]
    uint64_t full[STAGES];       // -> MMA: one arrival per producer warp of the stage's group, plus the bulk copy's bytes
    uint64_t empty[STAGES];      // MMA commit -> producers and the bulk warp
    uint64_t accum;              // last commit -> epilogue
    uint32_t tmem_base;
    int abort_flag;
};

struct GemmArgs {
    WeightRef w;
    const __half * xh;       // prepared activations of this pass
    const float * tokscale;  // per token: 1 / token scale
    float out_scale;         // 1 / weight prescale
    float * y;
    int64_t ldy;
    int n, m;      // weight rows; tokens of this pass
    int nchunks;   // ceil(K / KC)
    int kblocks;   // K / 32
    int m_tiles;
};

template <typename S, int TN, int KC, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tc(const GemmArgs g) {
    // a chunk of KC weights per row is 4 KC tasks; the 512 producer threads form 512 / (4 KC) groups that
    // take the chunks in turn
    constexpr int GROUPS = PRODUCER_WARPS * 32 / (4 * KC);
    constexpr int GROUP_WARPS = PRODUCER_WARPS / GROUPS;
    static_assert(GROUPS >= 1 && STAGES % GROUPS == 0, "each producer group owns every GROUPS-th stage");
    extern __shared__ __align__(128) uint8_t smem_raw[];
    using Smem = GemmSmem<TN, KC, STAGES>;
    Smem & sm = *reinterpret_cast<Smem *>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mt = blockIdx.x % g.m_tiles, nt = blockIdx.x / g.m_tiles;
    const int n0 = nt * TM, m0 = mt * TN;
    volatile int * abort_flag = &sm.abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_addr(&sm.full[s]), GROUP_WARPS + 1);  // the group's warps + the bulk copy's expect_tx
            mbar_init(smem_addr(&sm.empty[s]), 1);
        }
        mbar_init(smem_addr(&sm.accum), 1);
        sm.abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == WARP_MMA) {
        tmem_alloc(smem_addr(&sm.tmem_base), TN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *(volatile uint32_t *) &sm.tmem_base;
    // barrier addresses advance by 8 bytes per stage, operand stages by their byte size
    const uint32_t full0 = smem_addr(&sm.full[0]), empty0 = smem_addr(&sm.empty[0]);
    const uint32_t a_smem = smem_addr(sm.a[0]), b_smem = smem_addr(sm.b[0]);

    // everything above overlaps the tail of the previous kernel; the activations it wrote are read below
    pdl_wait();

    if (warp >= FIRST_PRODUCER) {
        // ---- A operand.  A task is (row, 32-weight block), one per thread of a producer group; with 64-wide
        // chunks group 0 (warps 2-9) takes the even chunks and group 1 the odd ones, so each has two chunk times
        // for its convert-store-fence sequence.  Eight warps cover the 128 rows for two adjacent blocks: warp w
        // owns rows 16 w .. 16 w + 15, lane l takes row (l & 7) + 8 (l >> 4), block (l >> 3) & 1, so one warp-wide
        // load touches the 16 rows' adjacent halves (whole 32/64-byte runs per row) and every group of 8 lanes
        // stores one complete 128-byte core matrix (no bank conflicts).  DEPTH of the group's chunks are kept
        // in flight in registers to cover the L2/HBM latency.
        constexpr int DEPTH = 2;
        constexpr int BLOCKS = KC / 32;  // 32-weight blocks per row and chunk
        const int pw = warp - FIRST_PRODUCER;
        const int group = pw / GROUP_WARPS;
        const int gw = pw % GROUP_WARPS;
        const int row_in = 16 * (gw & 7) + (lane & 7) + 8 * (lane >> 4);
        const int blk = ((lane >> 3) & 1) + 2 * (gw >> 3);
        const int64_t row = n0 + row_in;
        const bool row_ok = row < g.n;
        const uint32_t dst0 = a_smem + (blk * 4) * (TM * 16) + row_in * 16;
        typename S::Regs ring[DEPTH];
#pragma unroll
        for (int d = 0; d < DEPTH; ++d) {
            const int kb = (GROUPS * d + group) * BLOCKS + blk;
            if (row_ok && kb < g.kblocks) S::load(ring[d], g.w, row, kb);
        }
        bool alive = true;
        int s = group;  // this group's stage: advances by GROUPS, wraps at STAGES
        uint32_t phase = 0;
        for (int c0 = group; c0 < g.nchunks && alive; c0 += GROUPS * DEPTH) {
#pragma unroll
            for (int d = 0; d < DEPTH; ++d) {
                const int c = c0 + GROUPS * d;
                if (c >= g.nchunks) break;
                const int kb = c * BLOCKS + blk;
                uint32_t out[16];
                if (row_ok && kb < g.kblocks) {
                    SrcTraits<S>::convert(ring[d], kb, out);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) out[i] = 0u;
                }
                const int kb_next = kb + GROUPS * DEPTH * BLOCKS;
                if (row_ok && kb_next < g.kblocks) S::load(ring[d], g.w, row, kb_next);
                // the stage is free once the MMAs of the chunk that used it last have retired
                bool ok = mbar_try_wait(empty0 + 8 * s, phase ^ 1u);
                if (!ok) ok = mbar_wait(empty0 + 8 * s, phase ^ 1u, abort_flag, 0);
                if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
                const uint32_t dst = dst0 + s * Smem::A_BYTES;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + j * (TM * 16)), "r"(out[4 * j]), "r"(out[4 * j + 1]),
                                 "r"(out[4 * j + 2]), "r"(out[4 * j + 3])
                                 : "memory");
                fence_proxy_async();  // generic-proxy stores -> visible to the tensor core's async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(full0 + 8 * s);
                s += GROUPS;
                if (s >= STAGES) { s -= STAGES; phase ^= 1u; }
            }
        }
        pdl_launch_dependents();

        // ---- epilogue: a warp may read the TMEM lanes 32 (warp % 4) ..; four consecutive producer warps cover
        // the four lane quarters, and each such set takes a quarter of the columns ----
        bool acc_ok = alive;
        if (acc_ok) {
            acc_ok = mbar_try_wait(smem_addr(&sm.accum), 0u);
            if (!acc_ok) acc_ok = mbar_wait(smem_addr(&sm.accum), 0u, abort_flag, 1);
        }
        if (__all_sync(0xffffffffu, acc_ok)) {
            tc_fence_after();
            const int lane_base = 32 * (warp & 3);
            const int col_base = (pw >> 2) * (TN / 4);
            const int64_t n_out = n0 + lane_base + lane;
#pragma unroll 1
            for (int cc = 0; cc < TN / 4; cc += 16) {
                uint32_t r[16];
                tmem_ld16(tmem + ((uint32_t) lane_base << 16) + (uint32_t) (col_base + cc), r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int tok = m0 + col_base + cc + j;
                    if (tok < g.m && n_out < g.n) g.y[(int64_t) tok * g.ldy + n_out] = __uint_as_float(r[j]) * (__ldcg(g.tokscale + tok) * g.out_scale);
                }
            }
        }
    } else if (warp == WARP_BULK) {
        // ---- B operand: one bulk copy per stage, issued as soon as the stage is free ----
        if (lane == 0) {
            const uint8_t * src = reinterpret_cast<const uint8_t *>(g.xh) + (int64_t) mt * g.nchunks * Smem::B_BYTES;
            int issued = 0, s = 0;
            uint32_t phase = 0;
            for (int c = 0; c < g.nchunks; ++c) {
                if (!mbar_try_wait(empty0 + 8 * s, phase ^ 1u) && !mbar_wait(empty0 + 8 * s, phase ^ 1u, abort_flag, 2)) break;
                mbar_expect_tx(full0 + 8 * s, Smem::B_BYTES);
                bulk_g2s(b_smem + s * Smem::B_BYTES, src + (int64_t) c * Smem::B_BYTES, Smem::B_BYTES, full0 + 8 * s);
                issued = c + 1;
                if (++s == STAGES) { s = 0; phase ^= 1u; }
            }
            // copies still in flight must land before the CTA's shared memory goes away
            for (int c = issued > STAGES ? issued - STAGES : 0; c < issued; ++c) {
                const uint32_t bar = full0 + 8 * (c % STAGES);
                for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try_wait(bar, (uint32_t) (c / STAGES) & 1u); ++i) __nanosleep(64);
            }
        }
        __syncwarp();
    } else {
        // ---- MMA warp (warp 0).  This loop is one warp's serial instruction stream and bounds the kernel,
        // so it is kept lean: one barrier per stage, descriptors are a base plus compile-time offsets in
        // their low word, stage and phase are counters. ----
        constexpr uint32_t IDESC = instr_desc_f16(TM, TN);
        constexpr uint32_t DESC_HI = (128u >> 4) | (1u << 14);  // 128 bytes between 8-row groups; descriptor version 1
        const uint32_t a_lo0 = (a_smem >> 4) | ((uint32_t) (TM * 16) >> 4) << 16;  // start address | bytes between K halves
        const uint32_t b_lo0 = (b_smem >> 4) | ((uint32_t) (TN * 16) >> 4) << 16;
        bool alive = true;
        int s = 0;
        uint32_t phase = 0, accumulate = 0;
        for (int c = 0; c < g.nchunks; ++c) {
            bool ok = mbar_try_wait(full0 + 8 * s, phase);
            if (!ok) ok = mbar_wait(full0 + 8 * s, phase, abort_flag, 3, false);
            if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
            tc_fence_after();
            if (lane == 0) {
                const uint32_t a_lo = a_lo0 + s * (Smem::A_BYTES >> 4), b_lo = b_lo0 + s * (Smem::B_BYTES >> 4);
#pragma unroll
                for (int ks = 0; ks < KC / 16; ++ks) {
                    mma_f16(tmem, a_lo + ks * (2 * TM * 16 >> 4), b_lo + ks * (2 * TN * 16 >> 4), DESC_HI, IDESC, accumulate);
                    accumulate = 1u;
                }
                mma_commit(empty0 + 8 * s);
            }
            __syncwarp();
            if (++s == STAGES) { s = 0; phase ^= 1u; }
        }
        if (lane == 0) {
            // the accumulator is complete (or abandoned) once everything issued so far has retired
            mma_commit(smem_addr(&sm.accum));
            if (!alive) {
                for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try_wait(smem_addr(&sm.accum), 0u); ++i) __nanosleep(64);
            }
        }
        __syncwarp();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == WARP_MMA) {
        tc_fence_after();
        tmem_dealloc(tmem, TN);
    }
}

// ---------------------------------------------------------------------------------------------
// Activation preparation: f32 [M, K] (column stride ldx) -> normalised f16 stage images + token factors
// ---------------------------------------------------------------------------------------------
template <int TN, int KC>
__global__ void __launch_bounds__(256) gemm_prep_x(const float * x, int64_t ldx, int m, int k, int nchunks, int kslices, float * tokscale,
                                                   __half * xh) {
    pdl_wait();
    __shared__ float s_scale[8];
    const int group = blockIdx.x / kslices, slice = blockIdx.x % kslices;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    {
        const int tok = group * 8 + warp;
        float amax = 0.0f;
        if (tok < m) {
            const float4 * row = reinterpret_cast<const float4 *>(x + (int64_t) tok * ldx);
            for (int i = lane; i < k / 4; i += 32) {
                const float4 v = __ldcg(row + i);
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        int sh = 0;
        if (amax > 0.0f && amax <= 3.0e38f) {
            sh = 13 - ilogbf(amax);
            sh = sh > 100 ? 100 : sh < -100 ? -100 : sh;
        }
        if (lane == 0) {
            s_scale[warp] = ldexpf(1.0f, sh);
            if (slice == 0) tokscale[tok] = ldexpf(1.0f, -sh);
        }
    }
    __syncthreads();
    pdl_launch_dependents();
    const int t = threadIdx.x & 7;
    const int tok = group * 8 + t;
    const float scale = s_scale[t];
    constexpr int UPC = KC / 8;       // 8-element K units per chunk
    const int units = nchunks * UPC;  // per token, K padded to whole chunks
    const int per_slice = (units + kslices - 1) / kslices;
    const int u_end = (slice + 1) * per_slice < units ? (slice + 1) * per_slice : units;
    const int mt = tok / TN, tt = tok % TN;
    for (int u = slice * per_slice + (threadIdx.x >> 3); u < u_end; u += 32) {
        const int k0 = u * 8;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (tok < m && k0 < k) {
            const float4 * p = reinterpret_cast<const float4 *>(x + (int64_t) tok * ldx + k0);
            a = __ldcg(p);
            b = __ldcg(p + 1);
        }
        const __half2 h0 = __floats2half2_rn(a.x * scale, a.y * scale), h1 = __floats2half2_rn(a.z * scale, a.w * scale);
        const __half2 h2 = __floats2half2_rn(b.x * scale, b.y * scale), h3 = __floats2half2_rn(b.z * scale, b.w * scale);
        __half * dst = xh + ((int64_t) mt * nchunks + u / UPC) * (TN * KC) + (u % UPC) * (TN * 8) + tt * 8;
        *reinterpret_cast<uint4 *>(dst) = make_uint4(h2_bits(h0), h2_bits(h1), h2_bits(h2), h2_bits(h3));
    }
}

std::atomic<bool> g_gemm_launched{false};

template <typename S, int TN, int KC, int STAGES>
int launch_gemm(cudaStream_t s, GemmArgs g, int n_tiles) {
    g.out_scale = 1.0f / S::PRESCALE;
    using Smem = GemmSmem<TN, KC, STAGES>;
    static std::mutex mu;
    static std::vector<char> configured;
    int dev = 0;
    SM100_CUDA(cudaGetDevice(&dev));
    {
        std::lock_guard<std::mutex> lock(mu);
        if ((int) configured.size() <= dev) configured.resize(dev + 1, 0);
        if (!configured[dev]) {
            SM100_CUDA(cudaFuncSetAttribute(gemm_tc<S, TN, KC, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sizeof(Smem)));
            configured[dev] = 1;
        }
    }
    g_gemm_launched.store(true, std::memory_order_relaxed);
    return launch(gemm_tc<S, TN, KC, STAGES>, dim3((unsigned) (n_tiles * g.m_tiles)), dim3(GEMM_THREADS), sizeof(Smem), s, g);
}

template <int TN, int KC, int STAGES>
int launch_gemm_dtype(cudaStream_t s, int dtype, int layout, const GemmArgs & g, int n_tiles) {
    const bool packed = layout == LAYOUT_PACKED;
    switch (dtype) {
        case DT_Q8_0:
            return packed ? launch_gemm<SrcQ80<true>, TN, KC, STAGES>(s, g, n_tiles) : launch_gemm<SrcQ80<false>, TN, KC, STAGES>(s, g, n_tiles);
        case DT_Q4_0:
            return packed ? launch_gemm<SrcQ40<true>, TN, KC, STAGES>(s, g, n_tiles) : launch_gemm<SrcQ40<false>, TN, KC, STAGES>(s, g, n_tiles);
        case DT_Q4_K: return launch_gemm<SrcQ4K, TN, KC, STAGES>(s, g, n_tiles);
        case DT_F16: return launch_gemm<SrcF16, TN, KC, STAGES>(s, g, n_tiles);
    }
    return fail(ST_UNSUPPORTED, "gemm: no tensor-core source for dtype %d", dtype);
}

template <int TN, int KC, int STAGES>
int gemm_passes(cudaStream_t s, int dtype, int layout, GemmArgs g, const float * x, int64_t ldx, int64_t m, int64_t k, float * y, int n_tiles) {
    g.nchunks = (int) ((k + KC - 1) / KC);
    // tokens per pass: the prepared activations of one pass stay below 64 MiB
    int64_t pass = ((int64_t) 64 << 20) / ((int64_t) g.nchunks * KC * 2) / TN * TN;
    if (pass < TN) pass = TN;
    for (int64_t c0 = 0; c0 < m; c0 += pass) {
        const int64_t mm = m - c0 < pass ? m - c0 : pass;
        const int m_tiles = (int) ((mm + TN - 1) / TN);
        const int64_t mpad = (int64_t) m_tiles * TN;
        const size_t scale_bytes = ((size_t) mpad * sizeof(float) + 255) / 256 * 256;
        const size_t bytes = scale_bytes + (size_t) mpad * g.nchunks * KC * sizeof(__half);
        void * ws = nullptr;
        int st = device_scratch(1, bytes, &ws);
        if (st != ST_OK) return st;
        float * tokscale = (float *) ws;
        __half * xh = (__half *) ((uint8_t *) ws + scale_bytes);
        const int groups = (int) (mpad / 8);
        int kslices = (2 * sm_count() + groups - 1) / groups;
        if (kslices < 1) kslices = 1;
        if (kslices > g.nchunks) kslices = g.nchunks;
        st = launch(gemm_prep_x<TN, KC>, dim3((unsigned) (groups * kslices)), dim3(256), 0, s, x + c0 * ldx, ldx, (int) mm, (int) k, g.nchunks,
                    kslices, tokscale, xh);
        if (st != ST_OK) return st;
        g.xh = xh;
        g.tokscale = tokscale;
        g.y = y + c0 * g.ldy;
        g.m = (int) mm;
        g.m_tiles = m_tiles;
        st = launch_gemm_dtype<TN, KC, STAGES>(s, dtype, layout, g, n_tiles);
        if (st != ST_OK) return st;
    }
    return ST_OK;
}

}  // namespace

// Reads and clears the fault flag of the tensor-core GEMM on the current device; called after a stream
// synchronisation.  Costs nothing until a GEMM has been launched.
int gemm_poll_fault() {
    if (!g_gemm_launched.exchange(false, std::memory_order_relaxed)) return ST_OK;
    int v = 0;
    SM100_CUDA(cudaMemcpyFromSymbol(&v, g_gemm_fault, sizeof(v)));
    if (v == 0) return ST_OK;
    const int zero = 0;
    SM100_CUDA(cudaMemcpyToSymbol(g_gemm_fault, &zero, sizeof(zero)));
    return fail(ST_BACKEND, "mul_mat: the tensor-core GEMM gave up waiting on a pipeline barrier (site %d); its output is incomplete", v - 1);
}

// Tensor-core MUL_MAT.  *handled = false (and ST_OK) when the shape or dtype is left to the caller's fallback.
int gemm_tc_mul_mat(cudaStream_t s, int dtype, int layout, const void * w, int64_t w_row_stride, int64_t k, int64_t n, const float * x,
                    int64_t ldx, int64_t m, float * y, int64_t ldy, bool * handled) {
    *handled = false;
    const bool packed = layout == LAYOUT_PACKED;
    if (!(dtype == DT_Q8_0 || dtype == DT_Q4_0 || dtype == DT_F16 || (dtype == DT_Q4_K && packed))) return ST_OK;
    if (k % 32 != 0 || (dtype == DT_Q4_K && k % 256 != 0)) return ST_OK;
    if (n > INT32_MAX - TM || k > INT32_MAX - 128 || m > INT32_MAX / 2) return ST_OK;
    if ((((uintptr_t) x) & 15) != 0 || ldx % 4 != 0) return ST_OK;
    if (packed && (((uintptr_t) w) & 31) != 0) return ST_OK;
    const int be = block_elems(dtype);
    if (w_row_stride == 0) w_row_stride = k / be * block_bytes(dtype);

    const int n_tiles = (int) ((n + TM - 1) / TM);
    GemmArgs g = {};
    g.w.base = (const uint8_t *) w;
    g.w.planes = packed ? planes_for(dtype, n, k) : Planes{};
    g.w.row_stride = w_row_stride;
    g.w.blocks_per_row = k / be;
    g.n = (int) n;
    g.kblocks = (int) (k / 32);
    g.ldy = ldy;
    // 256-token tiles halve the dequantization work and the weight traffic per output, but a CTA then owns
    // all of an SM: worth it once there are enough tiles to fill the machine
    static const int forced_tn = [] { const char * e = getenv("SM100_GEMM_TN"); return e != nullptr ? atoi(e) : 0; }();
    const int64_t tiles256 = (int64_t) n_tiles * ((m + 255) / 256);
    const bool wide = forced_tn != 0 ? forced_tn == 256 : tiles256 >= (int64_t) sm_count();
    const int st = wide ? gemm_passes<256, 64, 4>(s, dtype, layout, g, x, ldx, m, k, y, n_tiles)
                        : gemm_passes<128, 64, 6>(s, dtype, layout, g, x, ldx, m, k, y, n_tiles);
    if (st != ST_OK) return st;
    *handled = true;
    return ST_OK;
}

}  // namespace sm100
