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
//  2. gemm_tc       one CTA per 128 weight rows x TN tokens (TN = 128 or 256).  Warp 0 owns the tensor memory
//                   and issues tcgen05.mma (kind::f16, 128 x TN x 16 per instruction, f32 accumulator of TN
//                   TMEM columns), warps 1-3 issue the bulk copies of the B stages in turn (a warp gets one
//                   bulk copy through per ~530 cycles), warps 4-27 dequantize the CTA's weight rows chunk by
//                   chunk to f16 (weights are multiplied by 256 to keep small scales out of the f16
//                   subnormals) - by default straight into tensor memory with tcgen05.st, from where the MMA
//                   reads its A operand, so that shared memory carries the activations only; optionally
//                   into shared-memory core matrices.  Weight stages and activation stages are two rings
//                   with their own full/empty mbarriers; tcgen05.commit hands both back.  When the last
//                   commit lands, warps 4-19 read the accumulator with tcgen05.ld, undo the two scalings
//                   and store y.
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
// Warp roles.  The MMA warp is warp 0: as a young warp it was starved by the polling producers (each of its
// instructions took 50-80 cycles to issue).
constexpr int WARP_MMA = 0;        // owns TMEM and issues the MMAs
constexpr int WARP_BULK = 1;       // warps 1-3 issue the bulk copies of the activation stages, a chunk each in turn
constexpr int BULK_WARPS = 3;
constexpr int FIRST_PRODUCER = 4;  // warps 4.. dequantize; the first 16 of them then run the epilogue
// Producer warps: 8 warps = 256 (row, 32-weight block) tasks = one 64-wide chunk of the 128 rows, so 24 warps are three
// groups that take the chunks in turn.  A producer's instruction stream is a dependent chain (~7 cycles per
// instruction), so the third group buys throughput that the issue slots still have.
constexpr int PRODUCER_WARPS = 24;
constexpr int EPILOGUE_WARPS = 16;
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
// non-blocking look at a barrier phase
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
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
// D[tmem] (+)= A . B^T; both descriptors share their high word (same 8-row-group stride and version).
// Executed by a whole (converged) warp: one elected lane issues.  Keeping the warp converged around the issue lets the
// operands live in uniform registers - issued from inside a divergent `if (lane == 0)` each MMA cost ~86 cycles.
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, e;\n\t.reg .b64 da, db;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same with the A operand in tensor memory: lane = row, 32-bit column j of the 8 columns at `a_tmem` = the row's
// K elements 2j (low half) and 2j + 1.
__device__ __forceinline__ void mma_f16_ta(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, e;\n\t.reg .b64 db;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The four MMAs of a 64-wide chunk (A in tensor memory) as one block of instructions: the issuing lane is given as a
// flag, the descriptors and addresses of the K steps are derived inside.  `b_desc` is the whole 64-bit descriptor
// of the first K step, `b_step` what a K step adds to it.
__device__ __forceinline__ void mma4_f16_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint64_t b_step, uint32_t idesc, uint32_t accumulate,
                                            uint32_t issuer) {
    asm volatile(
        "{\n\t.reg .pred pi, pacc, pone;\n\t.reg .b64 d1, d2, d3;\n\t.reg .b32 a1, a2, a3;\n\t"
        "elect.sync _|pi, 0xffffffff;\n\t"
        "setp.ne.b32 pacc, %5, 0;\n\t"
        "setp.eq.b32 pone, %6, %6;\n\t"
        "add.u64 d1, %2, %3;\n\t"
        "add.u64 d2, d1, %3;\n\t"
        "add.u64 d3, d2, %3;\n\t"
        "add.u32 a1, %1, 8;\n\t"
        "add.u32 a2, %1, 16;\n\t"
        "add.u32 a3, %1, 24;\n\t"
        "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %4, pacc;\n\t"
        "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], d1, %4, pone;\n\t"
        "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], d2, %4, pone;\n\t"
        "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], d3, %4, pone;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "l"(b_step), "r"(idesc), "r"(accumulate), "r"(issuer)
        : "memory");
}
// two commits (weight stage, activation stage) by the issuing lane
__device__ __forceinline__ void mma_commit2(uint32_t bar_a, uint32_t bar_b, uint32_t issuer) {
    asm volatile(
        "{\n\t.reg .pred pi;\n\t"
        "elect.sync _|pi, 0xffffffff;\n\t"
        "@pi tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "@pi tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%1];\n\t}" ::"r"(bar_a),
        "r"(bar_b), "r"(issuer)
        : "memory");
}
// 16 consecutive 32-bit columns of this thread's own TMEM lane (lane = base lane of the warp's quarter + lane id)
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(addr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// arrives on `bar` when every MMA issued so far by the elected lane has finished reading shared memory and writing
// TMEM (whole converged warp, like mma_f16: elect.sync picks the same lane)
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile(
        "{\n\t.reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar)
        : "memory");
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
template <int TN, int KC, int STAGES, int RT, bool ATM>
struct GemmSmem {
    static constexpr int A_BYTES = TM * KC * 2;   // one row tile of a stage
    static constexpr int B_BYTES = TN * KC * 2;
    // Weight stages: in tensor memory (ATM) as many as the columns left by the accumulators hold, at most 8;
    // in shared memory as many as activation stages.  The two rings have their own barriers: the activation copies
    // are the long-latency side (~2 us under load) and want every byte of shared memory in flight.
    static constexpr int SA = !ATM ? STAGES : (512 - RT * TN) / (RT * (KC / 2)) < 8 ? (512 - RT * TN) / (RT * (KC / 2)) : 8;
    uint8_t a[SA][ATM ? 16 : RT * A_BYTES];  // [row tile][k / 8][row][8 halves]; unused when A lives in tensor memory
    uint8_t b[STAGES][B_BYTES];  // [k / 8][token][8 halves]
    uint64_t full_a[SA];         // producers -> MMA: one arrival per producer warp and row tile
    uint64_t empty_a[SA];        // MMA commit -> producers
    uint64_t full_b[STAGES];     // bulk copy -> MMA: the issuing lane's expect_tx arrival + the bytes
    uint64_t empty_b[STAGES];    // MMA commit -> bulk warp
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

// RT row tiles of 128 weight rows per CTA (RT accumulators of TN columns in TMEM) share one activation stage: the
// activation bytes a CTA pulls from L2 per multiply-add halve with RT = 2, and that traffic is what bounds the kernel.
//
// ATM: the dequantized weights go to tensor memory instead of shared memory (tcgen05.st by the producers, A operand
// of the MMA read from TMEM).  Shared memory then carries only the activation stages: its data pipe - 128 bytes per
// cycle, shared by the producers' stores, the bulk copies and the MMA's operand reads - is what bounds the
// shared-memory variant (a 128 x 128 x 64 chunk moves 64 KB through it = 512 cycles, against 256 cycles of MMA).
// TMEM columns: RT accumulators of TN, then per stage and row tile KC / 2 columns of A (two f16 per column).
template <typename S, int TN, int KC, int STAGES, int RT, bool ATM>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tc(const GemmArgs g) {
    // a chunk of KC weights per row is 4 KC tasks; the 512 producer threads form 512 / (4 KC) groups that
    // take the chunks in turn
    constexpr int GROUPS = PRODUCER_WARPS * 32 / (4 * KC);
    constexpr int GROUP_WARPS = PRODUCER_WARPS / GROUPS;
    static_assert(GROUPS >= 1 && GROUPS * 4 * KC == PRODUCER_WARPS * 32, "whole producer groups of one chunk's tasks each");
    extern __shared__ __align__(128) uint8_t smem_raw[];
    using Smem = GemmSmem<TN, KC, STAGES, RT, ATM>;
    constexpr int ACC_COLS = RT * TN;
    constexpr int A_COLS = KC / 2;                                   // per stage and row tile
    constexpr int SA = Smem::SA;
    static_assert(SA >= 2, "at least two weight stages");
    constexpr int USED_COLS = ACC_COLS + (ATM ? SA * RT * A_COLS : 0);
    constexpr int TMEM_COLS = USED_COLS <= 32 ? 32 : USED_COLS <= 64 ? 64 : USED_COLS <= 128 ? 128 : USED_COLS <= 256 ? 256 : 512;
    static_assert(USED_COLS <= 512, "accumulators and weight stages exceed the tensor memory");
    Smem & sm = *reinterpret_cast<Smem *>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mt = blockIdx.x % g.m_tiles, nt = blockIdx.x / g.m_tiles;
    const int n0 = nt * (TM * RT), m0 = mt * TN;
    volatile int * abort_flag = &sm.abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SA; ++s) {
            mbar_init(smem_addr(&sm.full_a[s]), RT * GROUP_WARPS);
            mbar_init(smem_addr(&sm.empty_a[s]), 1);
        }
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_addr(&sm.full_b[s]), 1);
            mbar_init(smem_addr(&sm.empty_b[s]), 1);
        }
        mbar_init(smem_addr(&sm.accum), 1);
        sm.abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == WARP_MMA) {
        tmem_alloc(smem_addr(&sm.tmem_base), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *(volatile uint32_t *) &sm.tmem_base;
    // barrier addresses advance by 8 bytes per stage, operand stages by their byte size
    const uint32_t full_a0 = smem_addr(&sm.full_a[0]), empty_a0 = smem_addr(&sm.empty_a[0]);
    const uint32_t full_b0 = smem_addr(&sm.full_b[0]), empty_b0 = smem_addr(&sm.empty_b[0]);
    const uint32_t a_smem = smem_addr(sm.a[0]), b_smem = smem_addr(sm.b[0]);

    // Everything above, and the weight side below, overlaps the activation preparation that precedes this kernel
    // in the stream: only the bulk-copy warp (prepared activations) and the epilogue (token factors, output) wait
    // for it.  That kernel itself starts only after everything before it has completed, so nothing older is in flight.

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
        // ATM: a thread may only write its warp's quarter of the TMEM lanes (32 (warp % 4) ..), so a warp takes 32
        // consecutive rows of one block; the group's eight consecutive warps cover the four quarters for both blocks
        const int row_in = ATM ? 32 * (warp & 3) + lane : 16 * (gw & 7) + (lane & 7) + 8 * (lane >> 4);
        const int blk = ATM ? gw >> 2 : ((lane >> 3) & 1) + 2 * (gw >> 3);
        // The work unit is (chunk, row tile): unit u = chunk * RT + row tile, and group g takes the units g, g + GROUPS, ...
        // Rows past the tensor and blocks past K are clamped to the last valid ones instead of zero-filled: such rows
        // are never stored, and the activation image is zero where K is padded (the weights read there are finite).
        const int units = g.nchunks * RT;
        const int kb_last = g.kblocks - 1;
        const uint32_t dst0 = a_smem + (blk * 4) * (TM * 16) + row_in * 16;
        auto unit_row = [&](int u) -> int64_t {
            const int64_t row = (int64_t) n0 + (u % RT) * TM + row_in;
            return row < g.n ? row : (int64_t) g.n - 1;
        };
        auto unit_kb = [&](int u) -> int {
            const int kb = (u / RT) * BLOCKS + blk;
            return kb < kb_last ? kb : kb_last;
        };
        typename S::Regs ring[DEPTH];
#pragma unroll
        for (int d = 0; d < DEPTH; ++d) {
            const int u = group + GROUPS * d;
            S::load(ring[d], g.w, unit_row(u), unit_kb(u));
        }
        bool alive = true;
        for (int u0 = group; u0 < units && alive; u0 += GROUPS * DEPTH) {
#pragma unroll
            for (int d = 0; d < DEPTH; ++d) {
                const int u = u0 + GROUPS * d;
                if (u >= units) break;
                const int c = u / RT, rt = u % RT;
                uint32_t out[16];
                SrcTraits<S>::convert(ring[d], unit_kb(u), out);
                const int u_next = u + GROUPS * DEPTH;   // past the end: a clamped, unused load
                S::load(ring[d], g.w, unit_row(u_next), unit_kb(u_next));
                // the stage is free once the MMAs of the chunk that used it last have retired
                const int s = c % SA;
                const uint32_t phase = (uint32_t) (c / SA) & 1u;
                bool ok = mbar_try_wait(empty_a0 + 8 * s, phase ^ 1u);
                if (!ok) ok = mbar_wait(empty_a0 + 8 * s, phase ^ 1u, abort_flag, 0);
                if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
                if (ATM) {
                    tc_fence_after();   // the stage's previous MMAs (observed through the barrier) precede these stores
                    tmem_st16(tmem + ((uint32_t) (32 * (warp & 3)) << 16) + (uint32_t) (ACC_COLS + (s * RT + rt) * A_COLS + blk * 16), out);
                    tmem_st_wait();
                    tc_fence_before();   // the stores are ordered before the MMA that the arrival releases
                } else {
                    const uint32_t dst = dst0 + (s * RT + rt) * Smem::A_BYTES;
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + j * (TM * 16)), "r"(out[4 * j]), "r"(out[4 * j + 1]),
                                     "r"(out[4 * j + 2]), "r"(out[4 * j + 3])
                                     : "memory");
                    fence_proxy_async();  // generic-proxy stores -> visible to the tensor core's async proxy
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(full_a0 + 8 * s);
            }
        }
        // the dependency wait (long satisfied: the activations have been flowing) comes before the successor is
        // released, as in every kernel of this library: a successor's early section then overlaps this kernel only
        pdl_wait();
        pdl_launch_dependents();

        // ---- epilogue: a warp may read the TMEM lanes 32 (warp % 4) ..; four consecutive producer warps cover
        // the four lane quarters, and each such set takes a quarter of the columns ----
        bool acc_ok = alive;
        if (acc_ok) {
            acc_ok = mbar_try_wait(smem_addr(&sm.accum), 0u);
            if (!acc_ok) acc_ok = mbar_wait(smem_addr(&sm.accum), 0u, abort_flag, 1);
        }
        if (__all_sync(0xffffffffu, acc_ok) && pw < EPILOGUE_WARPS) {
            tc_fence_after();
            const int lane_base = 32 * (warp & 3);
            const int col_base = (pw >> 2) * (TN / 4);
#pragma unroll 1
            for (int rt = 0; rt < RT; ++rt) {
                const int64_t n_out = (int64_t) n0 + rt * TM + lane_base + lane;
#pragma unroll 1
                for (int cc = 0; cc < TN / 4; cc += 16) {
                    uint32_t r[16];
                    tmem_ld16(tmem + ((uint32_t) lane_base << 16) + (uint32_t) (rt * TN + col_base + cc), r);
                    // the token factors are fetched before any store: a load after a store to memory that may alias
                    // is not moved up by the compiler, and 16 dependent trips to L2 per pass cost ~5 us per CTA
                    float f[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) f[j] = __ldcg(g.tokscale + m0 + col_base + cc + j) * g.out_scale;   // allocated for whole tiles
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int tok = m0 + col_base + cc + j;
                        if (tok < g.m && n_out < g.n) g.y[(int64_t) tok * g.ldy + n_out] = __uint_as_float(r[j]) * f[j];
                    }
                }
            }
        }
    } else if (warp >= WARP_BULK) {
        // ---- B operand: one bulk copy per stage, issued as soon as the stage is free.  A warp gets one bulk copy
        // through per ~530 cycles whatever its size (measured: 16 KB copies from one thread 31 B/cycle, from four
        // warps 113 B/cycle), so the chunks go round BULK_WARPS issuing warps. ----
        if (lane == 0) {
            pdl_wait();
            const uint8_t * src = reinterpret_cast<const uint8_t *>(g.xh) + (int64_t) mt * g.nchunks * Smem::B_BYTES;
            int last = -1;
            for (int c = warp - WARP_BULK; c < g.nchunks; c += BULK_WARPS) {
                const int s = c % STAGES;
                const uint32_t phase = (uint32_t) (c / STAGES) & 1u;
                if (!mbar_try_wait(empty_b0 + 8 * s, phase ^ 1u) && !mbar_wait(empty_b0 + 8 * s, phase ^ 1u, abort_flag, 2)) break;
                mbar_expect_tx(full_b0 + 8 * s, Smem::B_BYTES);
                bulk_g2s(b_smem + s * Smem::B_BYTES, src + (int64_t) c * Smem::B_BYTES, Smem::B_BYTES, full_b0 + 8 * s);
                last = c;
            }
            // Every copy has landed once the MMA warp has passed its stage's barrier, which it does for every chunk
            // before the CTA ends.  Only a CTA that is giving up can have copies in flight when it leaves: wait,
            // briefly, for this warp's last ones so that they do not land in freed shared memory.
            if (*abort_flag != 0) {
                for (int c = last; c >= 0 && c > last - STAGES; c -= BULK_WARPS) {
                    const uint32_t bar = full_b0 + 8 * (c % STAGES);
                    for (uint32_t i = 0; i < (1u << 14) && !mbar_try_wait(bar, (uint32_t) (c / STAGES) & 1u); ++i) __nanosleep(64);
                }
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
        const uint32_t issuer = lane == 0 ? 1u : 0u;   // the lane that issues the MMAs and the commits (always the same one)
        int sa = 0, sb = 0;                       // stage of the weight ring and of the activation ring
        uint32_t pa = 0, pb = 0, accumulate = 0;
        // Both rings run several stages ahead, so the barriers of a chunk are almost always complete when this warp
        // gets to it - but asking costs a round trip (~250 cycles per barrier for this lone warp, two thirds of
        // the loop).  The look at chunk c + 1's barriers is therefore issued before chunk c's MMAs and its answer
        // used an iteration later; only a "not yet" takes the waiting path.
        uint32_t ready = (mbar_test_wait(full_b0, 0u) ? 1u : 0u) & (mbar_test_wait(full_a0, 0u) ? 1u : 0u);
        for (int c = 0; c < g.nchunks; ++c) {
            if (ready == 0u) {
                bool ok = mbar_try_wait(full_b0 + 8 * sb, pb);
                if (!ok) ok = mbar_wait(full_b0 + 8 * sb, pb, abort_flag, 3, false);
                if (ok) {
                    ok = mbar_try_wait(full_a0 + 8 * sa, pa);
                    if (!ok) ok = mbar_wait(full_a0 + 8 * sa, pa, abort_flag, 4, false);
                }
                if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
            }
            tc_fence_after();
            // next chunk's stages
            int sa_n = sa + 1, sb_n = sb + 1;
            uint32_t pa_n = pa, pb_n = pb;
            if (sa_n == SA) { sa_n = 0; pa_n ^= 1u; }
            if (sb_n == STAGES) { sb_n = 0; pb_n ^= 1u; }
            const uint32_t rb = mbar_test_wait(full_b0 + 8 * sb_n, pb_n) ? 1u : 0u;   // read after this chunk's MMAs are issued
            const uint32_t ra = mbar_test_wait(full_a0 + 8 * sa_n, pa_n) ? 1u : 0u;
            {
                const uint32_t a_lo = ATM ? 0u : a_lo0 + sa * (RT * Smem::A_BYTES >> 4), b_lo = b_lo0 + sb * (Smem::B_BYTES >> 4);
                if (ATM && KC == 64) {
                    const uint64_t b_desc = ((uint64_t) DESC_HI << 32) | b_lo;
#pragma unroll
                    for (int rt = 0; rt < RT; ++rt)
                        mma4_f16_ta(tmem + rt * TN, tmem + ACC_COLS + (sa * RT + rt) * A_COLS, b_desc, (uint64_t) (2 * TN * 16 >> 4), IDESC, accumulate, issuer);
                    accumulate = 1u;
                    mma_commit2(empty_a0 + 8 * sa, empty_b0 + 8 * sb, issuer);   // each commit covers every MMA issued so far
                } else {
#pragma unroll
                    for (int rt = 0; rt < RT; ++rt) {
#pragma unroll
                        for (int ks = 0; ks < KC / 16; ++ks) {
                            if (ATM)
                                mma_f16_ta(tmem + rt * TN, tmem + ACC_COLS + (sa * RT + rt) * A_COLS + ks * 8, b_lo + ks * (2 * TN * 16 >> 4), DESC_HI,
                                           IDESC, ks == 0 ? accumulate : 1u);
                            else
                                mma_f16(tmem + rt * TN, a_lo + rt * (Smem::A_BYTES >> 4) + ks * (2 * TM * 16 >> 4), b_lo + ks * (2 * TN * 16 >> 4),
                                        DESC_HI, IDESC, ks == 0 ? accumulate : 1u);
                        }
                    }
                    accumulate = 1u;
                    mma_commit(empty_a0 + 8 * sa);   // each commit covers every MMA issued so far
                    mma_commit(empty_b0 + 8 * sb);
                }
            }
            ready = c + 1 < g.nchunks ? (ra & rb) : 1u;
            sa = sa_n; pa = pa_n; sb = sb_n; pb = pb_n;
        }
        __syncwarp();
        // the accumulator is complete (or abandoned) once everything issued so far has retired
        mma_commit(smem_addr(&sm.accum));
        if (!alive && lane == 0) {
            for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try_wait(smem_addr(&sm.accum), 0u); ++i) __nanosleep(64);
        }
        __syncwarp();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == WARP_MMA) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// Activation preparation: f32 [M, K] (column stride ldx) -> normalised f16 stage images + token factors
// ---------------------------------------------------------------------------------------------
// A CTA takes `toks` consecutive tokens (a power of two, 1..8) with 256 / toks threads each and keeps their rows in
// registers (up to PREP_MAX_V float4 per thread, all requested at once): one trip to memory gives both the
// token's largest magnitude and, after the scale is known, the f16 image.  Rows too long for the registers
// (K > 32768 / toks at toks = 1) take the two-pass path: the same loop twice.
constexpr int PREP_MAX_V = 32;

template <int TN, int KC>
__global__ void __launch_bounds__(256) gemm_prep_x(const float * x, int64_t ldx, int m, int k, int nchunks, int toks, float * tokscale,
                                                   __half * xh) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float s_amax[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tpt = 256 / toks;                  // threads per token: 32, 64, 128 or 256
    const int tok = blockIdx.x * toks + threadIdx.x / tpt;
    const int r = threadIdx.x % tpt;
    const int kpad4 = nchunks * (KC / 4);        // float4 per token in the image (K padded to whole chunks)
    const int k4 = k / 4;
    const bool in_regs = kpad4 <= PREP_MAX_V * tpt;
    const float4 * row = reinterpret_cast<const float4 *>(x + (int64_t) tok * ldx);
    const bool tok_ok = tok < m;
    float4 v[PREP_MAX_V];
    float amax = 0.0f;
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < PREP_MAX_V; ++i) {
            const int idx = r + i * tpt;
            v[i] = tok_ok && idx < k4 ? __ldcg(row + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < PREP_MAX_V; ++i)
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
    } else if (tok_ok) {
#pragma unroll 8
        for (int idx = r; idx < k4; idx += tpt) {
            const float4 t = __ldcg(row + idx);
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(t.x), fabsf(t.y)), fmaxf(fabsf(t.z), fabsf(t.w))));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) s_amax[warp] = amax;
    __syncthreads();
    const int wpt = tpt / 32, w0 = (threadIdx.x / tpt) * wpt;   // the token's warps
    amax = 0.0f;
    for (int w = 0; w < wpt; ++w) amax = fmaxf(amax, s_amax[w0 + w]);
    int sh = 0;
    if (amax > 0.0f && amax <= 3.0e38f) {
        sh = 13 - ilogbf(amax);
        sh = sh > 100 ? 100 : sh < -100 ? -100 : sh;
    }
    const float scale = ldexpf(1.0f, sh);
    if (r == 0) tokscale[tok] = ldexpf(1.0f, -sh);
    // image: [token tile][chunk][k / 8][token in tile][8 halves]; a float4 is half of one 16-byte unit
    const int mt = tok / TN, tt = tok % TN;
    __half * img = xh + (int64_t) mt * nchunks * (TN * KC) + tt * 8;
    auto put = [&](int idx, const float4 & t) {
        const int kk = idx * 4, c = kk / KC, u = (kk % KC) >> 3;
        const __half2 h0 = __floats2half2_rn(t.x * scale, t.y * scale), h1 = __floats2half2_rn(t.z * scale, t.w * scale);
        *reinterpret_cast<uint2 *>(img + (int64_t) c * (TN * KC) + u * (TN * 8) + (kk & 4)) = make_uint2(h2_bits(h0), h2_bits(h1));
    };
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < PREP_MAX_V; ++i) {
            const int idx = r + i * tpt;
            if (idx < kpad4) put(idx, v[i]);
        }
    } else {
#pragma unroll 8
        for (int idx = r; idx < kpad4; idx += tpt) put(idx, tok_ok && idx < k4 ? __ldcg(row + idx) : make_float4(0.f, 0.f, 0.f, 0.f));
    }
}

std::atomic<bool> g_gemm_launched[MAX_DEVICES];   // per device, see sm100_common.cuh

template <typename S, int TN, int KC, int STAGES, int RT, bool ATM>
int launch_gemm(cudaStream_t s, GemmArgs g, int n_tiles) {
    g.out_scale = 1.0f / S::PRESCALE;
    using Smem = GemmSmem<TN, KC, STAGES, RT, ATM>;
    static std::mutex mu;
    static std::vector<char> configured;
    int dev = 0;
    SM100_CUDA(cudaGetDevice(&dev));
    {
        std::lock_guard<std::mutex> lock(mu);
        if ((int) configured.size() <= dev) configured.resize(dev + 1, 0);
        if (!configured[dev]) {
            SM100_CUDA(cudaFuncSetAttribute(gemm_tc<S, TN, KC, STAGES, RT, ATM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sizeof(Smem)));
            configured[dev] = 1;
        }
    }
    g_gemm_launched[current_device()].store(true, std::memory_order_relaxed);
    return launch(gemm_tc<S, TN, KC, STAGES, RT, ATM>, dim3((unsigned) (n_tiles * g.m_tiles)), dim3(GEMM_THREADS), sizeof(Smem), s, g);
}

template <int TN, int KC, int STAGES, int RT, bool ATM>
int launch_gemm_dtype(cudaStream_t s, int dtype, int layout, const GemmArgs & g, int n_tiles) {
    const bool packed = layout == LAYOUT_PACKED;
    switch (dtype) {
        case DT_Q8_0:
            return packed ? launch_gemm<SrcQ80<true>, TN, KC, STAGES, RT, ATM>(s, g, n_tiles) : launch_gemm<SrcQ80<false>, TN, KC, STAGES, RT, ATM>(s, g, n_tiles);
        case DT_Q4_0:
            return packed ? launch_gemm<SrcQ40<true>, TN, KC, STAGES, RT, ATM>(s, g, n_tiles) : launch_gemm<SrcQ40<false>, TN, KC, STAGES, RT, ATM>(s, g, n_tiles);
        case DT_Q4_K: return launch_gemm<SrcQ4K, TN, KC, STAGES, RT, ATM>(s, g, n_tiles);
        case DT_F16: return launch_gemm<SrcF16, TN, KC, STAGES, RT, ATM>(s, g, n_tiles);
    }
    return fail(ST_UNSUPPORTED, "gemm: no tensor-core source for dtype %d", dtype);
}

template <int TN, int KC, int STAGES, int RT, bool ATM>
int gemm_passes(cudaStream_t s, int dtype, int layout, GemmArgs g, const float * x, int64_t ldx, int64_t m, int64_t k, float * y) {
    const int n_tiles = (g.n + TM * RT - 1) / (TM * RT);
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
        // tokens per CTA: as many (up to 8) as keep a token's share of the row within the registers of its threads
        int toks = 8;
        while (toks > 1 && (int64_t) g.nchunks * (KC / 4) > (int64_t) PREP_MAX_V * (256 / toks)) toks >>= 1;
        st = launch(gemm_prep_x<TN, KC>, dim3((unsigned) (mpad / toks)), dim3(256), 0, s, x + c0 * ldx, ldx, (int) mm, (int) k, g.nchunks,
                    toks, tokscale, xh);
        if (st != ST_OK) return st;
        g.xh = xh;
        g.tokscale = tokscale;
        g.y = y + c0 * g.ldy;
        g.m = (int) mm;
        g.m_tiles = m_tiles;
        st = launch_gemm_dtype<TN, KC, STAGES, RT, ATM>(s, dtype, layout, g, n_tiles);
        if (st != ST_OK) return st;
    }
    return ST_OK;
}

}  // namespace

// Reads and clears the fault flag of the tensor-core GEMM on the current device; called after a stream
// synchronisation.  Costs nothing until a GEMM has been launched.

int gemm_poll_fault() {
    if (!g_gemm_launched[current_device()].exchange(false, std::memory_order_relaxed)) return ST_OK;
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
    // Tile choice.  128 weight rows x 256 tokens per CTA once such tiles fill the SMs: per multiply-add it pulls 20 %
    // fewer bytes into the SM than 128 x 128, and the kernel is bound by what an SM can take in (activation stages by
    // bulk copy + quantized weights by loads, ~50 bytes per cycle measured).  Two row tiles per CTA (256 x 128) pull
    // less still but are bound by the dequantizing warps instead; they stay selectable for experiments.
    static const int forced_tn = [] { const char * e = getenv("SM100_GEMM_TN"); return e != nullptr ? atoi(e) : 0; }();
    static const int forced_rt = [] { const char * e = getenv("SM100_GEMM_RT"); return e != nullptr ? atoi(e) : 0; }();
    // weights staged in tensor memory (default) or in shared memory
    static const int use_atm = [] { const char * e = getenv("SM100_GEMM_TMEM_A"); return e != nullptr ? atoi(e) : 1; }();
    int tn = (int64_t) n_tiles * ((m + 255) / 256) >= (int64_t) sm_count() ? 256 : 128;
    if (forced_tn == 128 || forced_tn == 256) tn = forced_tn;
    const int rt = forced_rt == 2 ? 2 : 1;
    int st;
    if (use_atm) {
        // more activation stages than these in flight slow the weight loads down by more than they hide
        if (rt == 2) st = gemm_passes<128, 64, 8, 2, true>(s, dtype, layout, g, x, ldx, m, k, y);   // 2 x 128 accumulator columns + 4 weight stages
        else st = tn == 256 ? gemm_passes<256, 64, 6, 1, true>(s, dtype, layout, g, x, ldx, m, k, y) : gemm_passes<128, 64, 8, 1, true>(s, dtype, layout, g, x, ldx, m, k, y);
    } else if (rt == 2) {
        st = tn == 256 ? gemm_passes<256, 64, 3, 2, false>(s, dtype, layout, g, x, ldx, m, k, y) : gemm_passes<128, 64, 4, 2, false>(s, dtype, layout, g, x, ldx, m, k, y);
    } else {
        st = tn == 256 ? gemm_passes<256, 64, 4, 1, false>(s, dtype, layout, g, x, ldx, m, k, y) : gemm_passes<128, 64, 6, 1, false>(s, dtype, layout, g, x, ldx, m, k, y);
    }
    if (st != ST_OK) return st;
    *handled = true;
    return ST_OK;
}

}  // namespace sm100
