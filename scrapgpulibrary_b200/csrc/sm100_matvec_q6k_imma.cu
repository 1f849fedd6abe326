// Q6_K decode MUL_MAT (one activation column) on the integer tensor-core path, packed layout.
//
// Same scheme as the Q4_K / Q4_0 / Q8_0 kernels: activations become 16-bit integers (two signed-byte planes, here
// with one f32 scale per 16 elements because Q6_K scales its weights in groups of 16), the 6-bit weights go into
// mma.sync.m16n8k32 (u8 x s8) as stored (q + 32), and the group scale is applied to an exact integer dot product:
//   y[n] = sum_groups d[n, block] sc[n, group] s_group ((256 H + L) - 32 Sx_group)
// (values of src/core/ref/quant.cpp:84-108 and src/core/ref/ops.cpp:891-984 of the reference; NMSE ~1e-9).
//
// The packed layout (sm100_layout.h) stores a block as four 64-weight units; a unit is 32 bytes of low nibbles,
// 16 bytes of high bit pairs and 4 group scales, and holds 4 groups of 16 weights.  A warp takes 16 rows x 1 unit:
// lane (g, t) assembles group t of rows g and g + 8 (16 bytes each) and feeds it into its eight k-slots of two
// MMAs; the four groups that share an MMA are kept apart by the B operand (group c's activations in columns 2c,
// 2c + 1, zeros elsewhere - a fixed pattern per lane).  Each warp walks a contiguous range of units of its row
// tile, so the half-used sectors of the bit-pair and scale planes are found in L1 by the next iteration.
#include "sm100_quant_units.cuh"

#include <cstdlib>

namespace sm100 {

namespace {

constexpr int SQ_WARPS = 8;    // warps that share one row tile (they split K)
constexpr int SQ_GROUPS = 2;   // row tiles a CTA works on at a time
constexpr int SQ_THREADS = SQ_WARPS * SQ_GROUPS * 32;

struct SqArgs {
    const uint8_t * w;                      // packed tensor base
    int64_t x_off, s_off, d_off;            // byte offsets of the bit-pair, scale and d planes (nibble plane at 0)
    const float * x;
    float * y;
    int64_t ldx, ldy;   // floats between consecutive activation / result columns (multi-column kernel)
    int n_tiles;        // full 16-row tiles
    int blocks;         // K / 256
    int units;          // K / 64
    int units_per_warp; // ceil(units / 8)
};

__device__ __forceinline__ void sq_imma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// one lane's share of a (row, unit): the 16 bytes that hold its group's nibbles, the unit's bit pairs, its scales
struct SqPiece {
    uint4 nib, hb;
    uint32_t sc, d;   // the unit's four group scales; the block's f16 d
};

// activations -> 16-bit integers per 16-element group (shared by the kernels below); the caller synchronises the CTA
__device__ __forceinline__ void sq_quantize_x(const float * x, uint32_t * xq, float2 * xs, int ngroups, int tid) {
    // activations -> 16-bit integers per 16-element group.  One item = 4 consecutive elements; the 4 items of a
    // group sit in 4 consecutive lanes.
    if (tid < 8) xq[ngroups * 8 + tid] = 0u;
    // all loads of a batch are issued before the first one is used: one L2 latency per batch, not per trip
    constexpr int BATCH = 6;
    for (int base = 0; base < ngroups * 4; base += BATCH * SQ_THREADS) {
        float4 xv[BATCH];
#pragma unroll
        for (int i = 0; i < BATCH; ++i) {
            const int it = base + i * SQ_THREADS + tid;
            if (it < ngroups * 4) xv[i] = __ldcg(reinterpret_cast<const float4 *>(x) + it);   // coherent: the producer may still be running when this kernel starts
        }
#pragma unroll
        for (int i = 0; i < BATCH; ++i) {
            const int it = base + i * SQ_THREADS + tid;
            if (it >= ngroups * 4) continue;   // warp-uniform: the item count is a multiple of 32
            const float4 v = xv[i];
            const int grp = it >> 2, q = it & 3;
            uint32_t amax_bits = act_abs_bits(v);
            amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, 1));
            amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, 2));
            float inv, s;
            act_group_scale(amax_bits, inv, s);
            // round to nearest (even) without the conversion unit: 1.5 * 2^23 + x keeps the integer in the mantissa (|x| <= 32512)
        const int x0 = __float_as_int(fmaf(v.x, inv, 12582912.0f)) - 0x4B400000, x1 = __float_as_int(fmaf(v.y, inv, 12582912.0f)) - 0x4B400000,
                  x2 = __float_as_int(fmaf(v.z, inv, 12582912.0f)) - 0x4B400000, x3 = __float_as_int(fmaf(v.w, inv, 12582912.0f)) - 0x4B400000;
            int isum = (x0 + x1) + (x2 + x3);
            isum += __shfl_xor_sync(0xffffffffu, isum, 1);
            isum += __shfl_xor_sync(0xffffffffu, isum, 2);
            // 16-bit integer = 256 h + l with h, l signed bytes: h = (x + 128) >> 8, l = low byte of x
            const int h0 = (x0 + 128) >> 8, h1 = (x1 + 128) >> 8, h2 = (x2 + 128) >> 8, h3 = (x3 + 128) >> 8;
            xq[grp * 8 + q] = __byte_perm(__byte_perm((uint32_t) h0, (uint32_t) h1, 0x0040), __byte_perm((uint32_t) h2, (uint32_t) h3, 0x0040), 0x5410);
            xq[grp * 8 + 4 + q] = __byte_perm(__byte_perm((uint32_t) x0, (uint32_t) x1, 0x0040), __byte_perm((uint32_t) x2, (uint32_t) x3, 0x0040), 0x5410);
            if (q == 0) xs[grp] = make_float2(s, __int_as_float(32 * isum));
        }
    }
}

// Shared memory of one CTA, per activation column (M of them, one after the other):
//   xq   [K/16][2 planes][16 B]   quantized activations, natural order inside a group; 32 zero bytes follow
//   xs   [K/16] (float s, int 32 * sum of the group's integers)
// then
//   red  [column][group][warp][16 rows] float    partial outputs of the warps of one row tile
// M > 1: the weights of a step are assembled once and multiplied with every column in turn (two MMAs and the scale terms
// per column), which is what makes a batch cheaper than one launch per column: the 6-bit assembly is the expensive part.
template <int M>
__global__ void __launch_bounds__(SQ_THREADS, 1) matvec_q6k_imma(SqArgs p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int ngroups = p.units * 4;
    const uint32_t col_bytes = (uint32_t) ngroups * 40u + 32u;   // one column's xq, zero bytes and xs
    uint32_t * xq = reinterpret_cast<uint32_t *>(smem);
    float2 * xs = reinterpret_cast<float2 *>(smem + (size_t) ngroups * 32 + 32);
    float * red = reinterpret_cast<float *>(smem + (size_t) M * col_bytes);

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int group = wid / SQ_WARPS, warp = wid % SQ_WARPS;
    const int g = lane >> 2, t = lane & 3;
    const int rt_step = gridDim.x * SQ_GROUPS;
    const int u_begin = warp * p.units_per_warp;
    const int u_end = u_begin + p.units_per_warp < p.units ? u_begin + p.units_per_warp : p.units;
    const uint32_t nib_shift = (uint32_t) (t >> 1) * 4u, hb_shift = (uint32_t) t * 2u, sc_shift = 24u - 8u * (uint32_t) t;

    auto load = [&](int rt_, int unit, SqPiece & p0, SqPiece & p1) {
        const int64_t blk0 = ((int64_t) rt_ * 16 + g) * p.blocks + (unit >> 2);   // block of row g
        const int64_t blk1 = blk0 + 8 * (int64_t) p.blocks;                        // block of row g + 8
        const int u = unit & 3;
        p0.nib = ldg_stream(p.w + blk0 * 128 + u * 32 + (t & 1) * 16);
        p1.nib = ldg_stream(p.w + blk1 * 128 + u * 32 + (t & 1) * 16);
        p0.hb = __ldg(reinterpret_cast<const uint4 *>(p.w + p.x_off + blk0 * 64 + u * 16));
        p1.hb = __ldg(reinterpret_cast<const uint4 *>(p.w + p.x_off + blk1 * 64 + u * 16));
        p0.sc = __ldg(reinterpret_cast<const uint32_t *>(p.w + p.s_off + blk0 * 16 + u * 4));
        p1.sc = __ldg(reinterpret_cast<const uint32_t *>(p.w + p.s_off + blk1 * 16 + u * 4));
        p0.d = __ldg(reinterpret_cast<const unsigned short *>(p.w + p.d_off) + blk0);
        p1.d = __ldg(reinterpret_cast<const unsigned short *>(p.w + p.d_off) + blk1);
    };

    SqPiece cur0, cur1, nxt0, nxt1;
    int rt = blockIdx.x * SQ_GROUPS + group, unit = u_begin;
    if (rt < p.n_tiles && unit < u_end) load(rt, unit, cur0, cur1);

    pdl_wait();

#pragma unroll 1
    for (int m = 0; m < M; ++m)
        sq_quantize_x(p.x + m * p.ldx, reinterpret_cast<uint32_t *>(smem + (size_t) m * col_bytes),
                      reinterpret_cast<float2 *>(smem + (size_t) m * col_bytes + (size_t) ngroups * 32 + 32), ngroups, tid);
    __syncthreads();
    pdl_launch_dependents();

    // B operand: lane (g, t) supplies column g; it is group t's plane (g & 1) when t == g / 2 and zero otherwise
    const bool live = t == (g >> 1);
    const uint32_t xq0 = (uint32_t) __cvta_generic_to_shared(xq);
    const uint32_t zero_addr = xq0 + (uint32_t) ngroups * 32u;
    const uint32_t lane_off = (uint32_t) t * 64u + (uint32_t) (g & 1) * 16u;   // group +2t of the unit, plane g & 1
    float * my_red = red + group * (SQ_WARPS * 16);   // column m: + m * SQ_GROUPS * SQ_WARPS * 16
    const int gtid = tid - group * (SQ_WARPS * 32);

    // every group runs the same number of rounds so that the CTA-wide barriers match
    for (int round = blockIdx.x * SQ_GROUPS; round < p.n_tiles; round += rt_step) {
        float acc0[M], acc1[M];   // rows g and g + 8, this lane's groups, per column
#pragma unroll
        for (int m = 0; m < M; ++m) acc0[m] = acc1[m] = 0.f;
        for (; rt < p.n_tiles && unit < u_end; ++unit) {
            int nrt = rt, nunit = unit + 1;
            if (nunit >= u_end) { nrt = rt + rt_step; nunit = u_begin; }
            if (nrt < p.n_tiles && nunit < u_end) load(nrt, nunit, nxt0, nxt1);
            const float d0 = __half2float(__ushort_as_half((unsigned short) cur0.d)), d1 = __half2float(__ushort_as_half((unsigned short) cur1.d));
            // group index of (block, unit, t): 16 block + 8 (unit / 2) + (unit & 1) + 2 t
            const int u = unit & 3;
            const uint32_t grp0 = (uint32_t) (unit >> 2) * 16u + (uint32_t) (u >> 1) * 8u + (uint32_t) (u & 1);
            const uint32_t n0[4] = {cur0.nib.x, cur0.nib.y, cur0.nib.z, cur0.nib.w}, n1[4] = {cur1.nib.x, cur1.nib.y, cur1.nib.z, cur1.nib.w};
            const uint32_t h0[4] = {cur0.hb.x, cur0.hb.y, cur0.hb.z, cur0.hb.w}, h1[4] = {cur1.hb.x, cur1.hb.y, cur1.hb.z, cur1.hb.w};
            uint32_t q0[4], q1[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                q0[i] = ((n0[i] >> nib_shift) & 0x0F0F0F0Fu) | (((h0[i] >> hb_shift) & 0x03030303u) << 4);
                q1[i] = ((n1[i] >> nib_shift) & 0x0F0F0F0Fu) | (((h1[i] >> hb_shift) & 0x03030303u) << 4);
            }
            const int s0 = ((int) (cur0.sc << sc_shift)) >> 24, s1 = ((int) (cur1.sc << sc_shift)) >> 24;   // signed byte t
            const float ds0 = d0 * (float) s0, ds1 = d1 * (float) s1;
#pragma unroll
            for (int m = 0; m < M; ++m) {
                uint4 bx = make_uint4(0u, 0u, 0u, 0u);
                {
                    const uint32_t addr = live ? xq0 + (uint32_t) m * col_bytes + grp0 * 32u + lane_off : zero_addr;
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(bx.x), "=r"(bx.y), "=r"(bx.z), "=r"(bx.w) : "r"(addr));
                }
                int c[4] = {0, 0, 0, 0};
                sq_imma(c, q0[0], q1[0], q0[1], q1[1], bx.x, bx.y);
                sq_imma(c, q0[2], q1[2], q0[3], q1[3], bx.z, bx.w);
                // columns 2t, 2t + 1 of this lane: (H, L) of group t
                const float2 sq = *reinterpret_cast<const float2 *>(reinterpret_cast<const uint8_t *>(xs + grp0 + 2 * t) + (size_t) m * col_bytes);
                const int sx32 = __float_as_int(sq.y);
                const float v0 = (float) (c[0] * 256 + c[1] - sx32), v1 = (float) (c[2] * 256 + c[3] - sx32);
                acc0[m] = fmaf(ds0 * sq.x, v0, acc0[m]);
                acc1[m] = fmaf(ds1 * sq.x, v1, acc1[m]);
            }
            cur0 = nxt0;
            cur1 = nxt1;
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float a0 = acc0[m], a1 = acc1[m];
            a0 += __shfl_xor_sync(0xffffffffu, a0, 1);
            a0 += __shfl_xor_sync(0xffffffffu, a0, 2);
            a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
            a1 += __shfl_xor_sync(0xffffffffu, a1, 2);
            if (t == 0) {
                my_red[m * (SQ_GROUPS * SQ_WARPS * 16) + warp * 16 + g] = a0;
                my_red[m * (SQ_GROUPS * SQ_WARPS * 16) + warp * 16 + g + 8] = a1;
            }
        }
        __syncthreads();
        if (gtid < 16 * M && rt < p.n_tiles) {
            const int m = gtid >> 4, row = gtid & 15;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < SQ_WARPS; ++w) v += my_red[m * (SQ_GROUPS * SQ_WARPS * 16) + w * 16 + row];
            p.y[m * p.ldy + (int64_t) rt * 16 + row] = v;
        }
        __syncthreads();
        rt += rt_step;
        unit = u_begin;
    }
}

// The same product with SQ_DEPTH steps (16 rows x one 64-weight unit each) of a warp in flight in registers instead of
// two, the first SQ_DEPTH requested before the dependency wait.  Needs whole batches: every warp's unit range a
// multiple of SQ_DEPTH long.
constexpr int SQ_DEPTH = 4;

__global__ void __launch_bounds__(SQ_THREADS, 1) matvec_q6k_imma_deep(SqArgs p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int ngroups = p.units * 4;
    uint32_t * xq = reinterpret_cast<uint32_t *>(smem);
    float2 * xs = reinterpret_cast<float2 *>(smem + (size_t) ngroups * 32 + 32);
    float * red = reinterpret_cast<float *>(xs + ngroups);

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int group = wid / SQ_WARPS, warp = wid % SQ_WARPS;
    const int g = lane >> 2, t = lane & 3;
    const int rt_step = gridDim.x * SQ_GROUPS;
    const int u_begin = warp * p.units_per_warp;
    const int u_end = u_begin + p.units_per_warp < p.units ? u_begin + p.units_per_warp : p.units;
    const uint32_t nib_shift = (uint32_t) (t >> 1) * 4u, hb_shift = (uint32_t) t * 2u, sc_shift = 24u - 8u * (uint32_t) t;

    auto load = [&](int rt_, int unit, SqPiece & p0, SqPiece & p1) {
        const int64_t blk0 = ((int64_t) rt_ * 16 + g) * p.blocks + (unit >> 2);   // block of row g
        const int64_t blk1 = blk0 + 8 * (int64_t) p.blocks;                        // block of row g + 8
        const int u = unit & 3;
        p0.nib = ldg_stream(p.w + blk0 * 128 + u * 32 + (t & 1) * 16);
        p1.nib = ldg_stream(p.w + blk1 * 128 + u * 32 + (t & 1) * 16);
        p0.hb = __ldg(reinterpret_cast<const uint4 *>(p.w + p.x_off + blk0 * 64 + u * 16));
        p1.hb = __ldg(reinterpret_cast<const uint4 *>(p.w + p.x_off + blk1 * 64 + u * 16));
        p0.sc = __ldg(reinterpret_cast<const uint32_t *>(p.w + p.s_off + blk0 * 16 + u * 4));
        p1.sc = __ldg(reinterpret_cast<const uint32_t *>(p.w + p.s_off + blk1 * 16 + u * 4));
        p0.d = __ldg(reinterpret_cast<const unsigned short *>(p.w + p.d_off) + blk0);
        p1.d = __ldg(reinterpret_cast<const unsigned short *>(p.w + p.d_off) + blk1);
    };

    SqPiece slot0[SQ_DEPTH], slot1[SQ_DEPTH];   // rows g and g + 8 of the steps in flight
    int rt = blockIdx.x * SQ_GROUPS + group;
    // load cursor: runs SQ_DEPTH steps ahead of the multiply over the same (row tile, unit) sequence
    int lrt = rt, lunit = u_begin;
    auto advance = [&]() {
        if (++lunit >= u_end) { lunit = u_begin; lrt += rt_step; }
    };
#pragma unroll
    for (int i = 0; i < SQ_DEPTH; ++i) {
        if (lrt < p.n_tiles) load(lrt, lunit, slot0[i], slot1[i]);
        advance();
    }

    pdl_wait();

    sq_quantize_x(p.x, xq, xs, ngroups, tid);
    __syncthreads();
    pdl_launch_dependents();

    // B operand: lane (g, t) supplies column g; it is group t's plane (g & 1) when t == g / 2 and zero otherwise
    const bool live = t == (g >> 1);
    const uint32_t xq0 = (uint32_t) __cvta_generic_to_shared(xq);
    const uint32_t zero_addr = xq0 + (uint32_t) ngroups * 32u;
    const uint32_t lane_off = (uint32_t) t * 64u + (uint32_t) (g & 1) * 16u;   // group +2t of the unit, plane g & 1
    float * my_red = red + group * (SQ_WARPS * 16);
    const int gtid = tid - group * (SQ_WARPS * 32);

    // every group runs the same number of rounds so that the CTA-wide barriers match
    for (int round = blockIdx.x * SQ_GROUPS; round < p.n_tiles; round += rt_step) {
        float acc0 = 0.f, acc1 = 0.f;   // rows g and g + 8, this lane's groups
        for (int ub = u_begin; rt < p.n_tiles && ub < u_end; ub += SQ_DEPTH) {
#pragma unroll
          for (int si = 0; si < SQ_DEPTH; ++si) {
            const int unit = ub + si;
            const SqPiece & cur0 = slot0[si];
            const SqPiece & cur1 = slot1[si];
            const float d0 = __half2float(__ushort_as_half((unsigned short) cur0.d)), d1 = __half2float(__ushort_as_half((unsigned short) cur1.d));
            // group index of (block, unit, t): 16 block + 8 (unit / 2) + (unit & 1) + 2 t
            const int u = unit & 3;
            const uint32_t grp0 = (uint32_t) (unit >> 2) * 16u + (uint32_t) (u >> 1) * 8u + (uint32_t) (u & 1);
            uint4 bx = make_uint4(0u, 0u, 0u, 0u);
            {
                const uint32_t addr = live ? xq0 + grp0 * 32u + lane_off : zero_addr;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(bx.x), "=r"(bx.y), "=r"(bx.z), "=r"(bx.w) : "r"(addr));
            }
            const uint32_t n0[4] = {cur0.nib.x, cur0.nib.y, cur0.nib.z, cur0.nib.w}, n1[4] = {cur1.nib.x, cur1.nib.y, cur1.nib.z, cur1.nib.w};
            const uint32_t h0[4] = {cur0.hb.x, cur0.hb.y, cur0.hb.z, cur0.hb.w}, h1[4] = {cur1.hb.x, cur1.hb.y, cur1.hb.z, cur1.hb.w};
            uint32_t q0[4], q1[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                q0[i] = ((n0[i] >> nib_shift) & 0x0F0F0F0Fu) | (((h0[i] >> hb_shift) & 0x03030303u) << 4);
                q1[i] = ((n1[i] >> nib_shift) & 0x0F0F0F0Fu) | (((h1[i] >> hb_shift) & 0x03030303u) << 4);
            }
            int c[4] = {0, 0, 0, 0};
            sq_imma(c, q0[0], q1[0], q0[1], q1[1], bx.x, bx.y);
            sq_imma(c, q0[2], q1[2], q0[3], q1[3], bx.z, bx.w);
            // columns 2t, 2t + 1 of this lane: (H, L) of group t
            const float2 sq = xs[grp0 + 2 * t];
            const int sx32 = __float_as_int(sq.y);
            const int s0 = ((int) (cur0.sc << sc_shift)) >> 24, s1 = ((int) (cur1.sc << sc_shift)) >> 24;   // signed byte t
            const float v0 = (float) (c[0] * 256 + c[1] - sx32), v1 = (float) (c[2] * 256 + c[3] - sx32);
            acc0 = fmaf(d0 * (float) s0 * sq.x, v0, acc0);
            acc1 = fmaf(d1 * (float) s1 * sq.x, v1, acc1);
            // the slot is free: its step SQ_DEPTH ahead goes in
            if (lrt < p.n_tiles) load(lrt, lunit, slot0[si], slot1[si]);
            advance();
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
            for (int w = 0; w < SQ_WARPS; ++w) v += my_red[w * 16 + gtid];
            p.y[(int64_t) rt * 16 + gtid] = v;
        }
        __syncthreads();
        rt += rt_step;
    }
}

size_t sq_smem_bytes(int units, int cols = 1) { return (size_t) cols * ((size_t) units * 4 * 40 + 32) + (size_t) cols * SQ_WARPS * SQ_GROUPS * 16 * 4; }

}  // namespace

// Q6_K packed matvec, one activation column, over the full 16-row tiles of the tensor; *handled = false when the
// shape is left to the caller's other kernels.
int matvec_q6k_imma_tiles(cudaStream_t s, const void * w, int64_t k, int64_t n, const float * x, float * y, bool * handled) {
    *handled = false;
    const int64_t tiles = n / 16;
    if (tiles == 0 || k % 256 != 0 || k > (int64_t) 1 << 18 || tiles > INT32_MAX / 2) return ST_OK;
    if (((uintptr_t) w & 15) != 0 || ((uintptr_t) x & 15) != 0) return ST_OK;
    const int units = (int) (k / 64);
    const size_t smem = sq_smem_bytes(units);
    if (smem > (size_t) 227 * 1024) return ST_OK;
    const Planes P = planes_for(DT_Q6_K, n, k);
    SqArgs a;
    a.w = (const uint8_t *) w;
    a.x_off = P.off[1];
    a.s_off = P.off[2];
    a.d_off = P.off[3];
    a.x = x;
    a.y = y;
    a.ldx = k;
    a.ldy = n;
    a.n_tiles = (int) tiles;
    a.blocks = (int) (k / 256);
    a.units = units;
    a.units_per_warp = (units + SQ_WARPS - 1) / SQ_WARPS;
    int64_t grid = sm_count();
    const int64_t rounds = (tiles + SQ_GROUPS - 1) / SQ_GROUPS;
    if (grid > rounds) grid = rounds;
    static const int deep_ok = [] { const char * e = getenv("SM100_Q6K_DEEP"); return e != nullptr ? atoi(e) : 1; }();
    int st;
    if (deep_ok && units % SQ_WARPS == 0 && a.units_per_warp % SQ_DEPTH == 0) {
        if (smem > 48 * 1024) SM100_CUDA(cudaFuncSetAttribute(matvec_q6k_imma_deep, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        st = launch(matvec_q6k_imma_deep, dim3((unsigned) grid), dim3(SQ_THREADS), smem, s, a);
    } else {
        if (smem > 48 * 1024) SM100_CUDA(cudaFuncSetAttribute(matvec_q6k_imma<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        st = launch(matvec_q6k_imma<1>, dim3((unsigned) grid), dim3(SQ_THREADS), smem, s, a);
    }
    *handled = st == ST_OK;
    return st;
}

// The same for 2..8 activation columns: the columns are served in launches of 8, 4, 2 or 1 (as many as fit the shared
// memory: a column of K = 12288 takes 30 KB), each launch assembling the weights once for all its columns.
template <int M>
static int launch_q6k_cols(cudaStream_t s, SqArgs a, int grid) {
    const size_t smem = sq_smem_bytes(a.units, M);
    if (smem > 48 * 1024) SM100_CUDA(cudaFuncSetAttribute(matvec_q6k_imma<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    return launch(matvec_q6k_imma<M>, dim3((unsigned) grid), dim3(SQ_THREADS), smem, s, a);
}

int matvec_q6k_imma_cols(cudaStream_t s, const void * w, int64_t k, int64_t n, const float * x, int64_t ldx, int m, float * y, int64_t ldy, bool * handled) {
    *handled = false;
    const int64_t tiles = n / 16;
    if (m < 2 || m > 8 || tiles == 0 || k % 256 != 0 || k > (int64_t) 1 << 18 || tiles > INT32_MAX / 2) return ST_OK;
    if (((uintptr_t) w & 15) != 0 || ((uintptr_t) x & 15) != 0 || ldx % 4 != 0) return ST_OK;
    const int units = (int) (k / 64);
    if (sq_smem_bytes(units, 1) > (size_t) 227 * 1024) return ST_OK;
    const Planes P = planes_for(DT_Q6_K, n, k);
    SqArgs a;
    a.w = (const uint8_t *) w;
    a.x_off = P.off[1];
    a.s_off = P.off[2];
    a.d_off = P.off[3];
    a.ldx = ldx;
    a.ldy = ldy;
    a.n_tiles = (int) tiles;
    a.blocks = (int) (k / 256);
    a.units = units;
    a.units_per_warp = (units + SQ_WARPS - 1) / SQ_WARPS;
    int64_t grid = sm_count();
    const int64_t rounds = (tiles + SQ_GROUPS - 1) / SQ_GROUPS;
    if (grid > rounds) grid = rounds;
    for (int done = 0; done < m;) {
        int take = 8;
        while (take > m - done || sq_smem_bytes(units, take) > (size_t) 227 * 1024) take /= 2;
        a.x = x + (int64_t) done * ldx;
        a.y = y + (int64_t) done * ldy;
        int st;
        switch (take) {
            case 8: st = launch_q6k_cols<8>(s, a, (int) grid); break;
            case 4: st = launch_q6k_cols<4>(s, a, (int) grid); break;
            case 2: st = launch_q6k_cols<2>(s, a, (int) grid); break;
            default: st = launch_q6k_cols<1>(s, a, (int) grid); break;
        }
        if (st != ST_OK) return st;
        done += take;
    }
    *handled = true;
    return ST_OK;
}

}  // namespace sm100
