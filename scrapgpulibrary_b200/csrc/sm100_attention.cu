// Fused decode attention for sm_100a: the values of scrapgpu_scaled_dot_product_attention
// (src/core/attention.cpp:558-678 of the reference; contract include/scrapgpu/attention.h:11-46), which the
// reference composes per head from CPY(V^T) + MUL_MAT(K.Q) + SOFT_MAX(+host-built mask) + MUL_MAT with a
// host round trip per tile.  Here: one pass over the KV cache, split along the key axis so that all SMs
// stream K and V (flash-decoding), query heads of a KV group processed together (GQA), f32 throughout.
//
//   scores[k] = (sum_d K[d,k,hk] Q[d,q,h]) * scale (+ mask[k,q,h]),  key k visible iff !causal or k <= offset + q
//   out[dv,q,h] = sum_k softmax(scores)[k] V[dv,k,hk];  a query with no visible key gives zeros (:497-516)
//
// Kernel 1 writes per split an un-normalised partial (running max m, sum l, accumulator o[Dv]) into a
// scratch buffer; kernel 2 merges the splits.  HBM-bound: algorithmic bytes = 2 * 4 * D * visible keys * Hkv.
#include "sm100_common.cuh"

#include <cstdlib>
#include <mutex>
#include <vector>

namespace sm100 {

constexpr int ATT_MAX_GROUP = 8;    // query heads per KV head handled together (reference limit: ops_matmul.cpp:19)
constexpr int ATT_CHUNK = 512;      // keys per split at most (scores of a split live in shared memory)
constexpr int ATT_THREADS = 256;

struct AttnArgs {
    const float * q; const float * k; const float * v; const float * mask; float * out; float * scratch;
    const int32_t * positions;
    int * counters;   // one per (query, KV head): splits that have delivered their partial (fused merge), or null
    int64_t d, dv, nq, nk, hq, hkv, offset;
    int64_t mask_heads;
    int splits, chunk, causal;
    // KV-cache calls: only the last `fresh_keys` visible keys of a query may have been written since the stream's last
    // point of full serialization, every earlier key (and `positions`) is older than that, so those rows can be
    // requested before the dependency wait.  -1: no such promise, everything is read after the wait.
    int fresh_keys;
    float scale;
    // Decode step with the new token's head post-processing in the same launch (attn_fast_kernel<.., POST = true>): q is the
    // RAW query projection; every warp applies the per-head RMS norm (when q_w is set) and the NEOX rotation to the query heads
    // it uses, and the CTA whose split ends at the newest position does the same for the new key (k_new, k_w), stores it and
    // the new value (v_new) into row positions[0] of the caches (k, v) and then reads them like any other row.
    const float * k_new; const float * v_new; const float * q_w; const float * k_w;
    const float * table;            // (cos, sin) per (position - table_first, pair), or null: computed from theta_scale
    int64_t table_first; int table_n;
    float eps, theta_scale;
};

// scratch layout per (q, h, split): [m, l, o[dv]]
// A split's partial of one (query, head) is [m, l, unused, unused, o[dv]]: the accumulator starts 16 bytes in, so
// that it can be moved as float4 when dv is a multiple of 4.
constexpr int ATT_HDR = 4;

__device__ __forceinline__ int64_t scratch_index(const AttnArgs & a, int64_t q, int64_t h, int split) {
    return ((q * a.hq + h) * a.splits + split) * (a.dv + ATT_HDR);
}

__device__ __forceinline__ int64_t visible_keys(const AttnArgs & a, int64_t q) {
    if (!a.causal) return a.nk;
    const int64_t off = a.positions != nullptr ? (int64_t) a.positions[0] : a.offset;
    const int64_t vis = off + q + 1;
    return vis < a.nk ? (vis < 0 ? 0 : vis) : a.nk;
}

__global__ void __launch_bounds__(ATT_THREADS) attn_partial_kernel(AttnArgs a) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float smem[];
    const int split = blockIdx.x;
    const int64_t hk = blockIdx.y, q = blockIdx.z;
    const int group = (int) (a.hq / a.hkv);
    float * sq = smem;                                  // [group][d]
    float * ss = sq + (int64_t) group * a.d;            // [group][chunk]
    float * sred = ss + (int64_t) group * a.chunk;      // [2][group][dv] partial accumulators of the two key halves
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;

    // the visible keys (known only on the device when the offset comes from `positions`) are spread evenly over
    // the splits; the planned chunk is the upper bound the shared memory was sized for
    const int64_t n_vis = visible_keys(a, q);
    const int64_t chunk = (n_vis + a.splits - 1) / a.splits;
    const int64_t k0 = (int64_t) split * chunk;
    const int64_t k1 = k0 + chunk < n_vis ? k0 + chunk : n_vis;
    const int64_t count = k1 > k0 ? k1 - k0 : 0;

    for (int64_t i = tid; i < (int64_t) group * a.d; i += blockDim.x) {
        const int64_t g = i / a.d, dd = i % a.d;
        sq[i] = a.q[((hk * group + g) * a.nq + q) * a.d + dd];
    }
    __syncthreads();

    // scores: one warp per key, all query heads of the group at once
    for (int64_t kk = warp; kk < count; kk += nwarps) {
        const float * kr = a.k + (hk * a.nk + k0 + kk) * a.d;
        float acc[ATT_MAX_GROUP];
#pragma unroll
        for (int g = 0; g < ATT_MAX_GROUP; ++g) acc[g] = 0.f;
        for (int64_t dd = lane; dd < a.d; dd += 32) {
            const float kvv = kr[dd];
#pragma unroll
            for (int g = 0; g < ATT_MAX_GROUP; ++g)
                if (g < group) acc[g] = fmaf(kvv, sq[g * a.d + dd], acc[g]);
        }
#pragma unroll
        for (int g = 0; g < ATT_MAX_GROUP; ++g) {
            if (g < group) {
                float v = acc[g];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) {
                    v *= a.scale;
                    if (a.mask != nullptr) {
                        const int64_t mh = a.mask_heads == 1 ? 0 : hk * group + g;
                        v += a.mask[(mh * a.nq + q) * a.nk + k0 + kk];
                    }
                    ss[g * a.chunk + kk] = v;
                }
            }
        }
    }
    __syncthreads();

    // per head: max, exponentials, sum (warp g handles head g; group <= 8 = warps)
    for (int g = warp; g < group; g += nwarps) {
        float m = -INFINITY;
        for (int64_t kk = lane; kk < count; kk += 32) m = fmaxf(m, ss[g * a.chunk + kk]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float l = 0.f;
        for (int64_t kk = lane; kk < count; kk += 32) {
            const float e = m == -INFINITY ? 0.f : expf(ss[g * a.chunk + kk] - m);
            ss[g * a.chunk + kk] = e;
            l += e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        if (lane == 0) {
            float * dst = a.scratch + scratch_index(a, q, hk * group + g, split);
            dst[0] = m;
            dst[1] = l;
        }
    }
    __syncthreads();

    // o[g][dv] = sum_k e[g][k] V[dv,k]: threads cover dv, the two halves of the block take alternate keys
    const int halves = blockDim.x >= 2 * a.dv ? 2 : 1;
    const int half = halves == 2 ? (int) (tid / a.dv) : 0;
    for (int64_t dv0 = 0; dv0 < a.dv; dv0 += blockDim.x / halves) {
        const int64_t dvi = dv0 + (halves == 2 ? tid % a.dv : tid);
        const bool active = dvi < a.dv && half < halves;
        float o[ATT_MAX_GROUP];
#pragma unroll
        for (int g = 0; g < ATT_MAX_GROUP; ++g) o[g] = 0.f;
        if (active) {
            for (int64_t kk = half; kk < count; kk += halves) {
                const float vv = a.v[(hk * a.nk + k0 + kk) * a.dv + dvi];
#pragma unroll
                for (int g = 0; g < ATT_MAX_GROUP; ++g)
                    if (g < group) o[g] = fmaf(ss[g * a.chunk + kk], vv, o[g]);
            }
        }
        if (halves == 2) {
            if (active && half == 1)
                for (int g = 0; g < group; ++g) sred[g * a.dv + dvi] = o[g];
            __syncthreads();
            if (active && half == 0)
                for (int g = 0; g < group; ++g) a.scratch[scratch_index(a, q, hk * group + g, split) + ATT_HDR + dvi] = o[g] + sred[g * a.dv + dvi];
            __syncthreads();
        } else if (active) {
            for (int g = 0; g < group; ++g) a.scratch[scratch_index(a, q, hk * group + g, split) + ATT_HDR + dvi] = o[g];
        }
    }
}

// Merge of the splits of one (query, head), by one CTA: thread s first turns split s's (m, l) into its weight
// exp(m_s - m) in shared memory (one round of independent loads), then the threads cover dv and sum the weighted
// partial accumulators, again with independent loads.  Loads bypass L1: the partials may come from other CTAs of
// the same launch.
constexpr int ATT_MAX_SPLITS = 1024;

__device__ __forceinline__ void attn_merge_head(const AttnArgs & a, int64_t q, int64_t h, float * s_w, float (*s_red)[32]) {
    const float * base = a.scratch + scratch_index(a, q, h, 0);
    const int64_t stride = a.dv + ATT_HDR;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    __syncthreads();   // s_w / s_red may still be read from a previous head
    float m = -INFINITY;
    for (int s = tid; s < a.splits; s += blockDim.x) {
        const float ms = __ldcg(base + s * stride);
        s_w[s] = ms;
        m = fmaxf(m, ms);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) s_red[0][warp] = m;
    __syncthreads();
    m = -INFINITY;
    for (int w = 0; w < nwarps; ++w) m = fmaxf(m, s_red[0][w]);
    float l = 0.f;
    for (int s = tid; s < a.splits; s += blockDim.x) {
        const float ms = s_w[s];
        const float e = ms != -INFINITY ? expf(ms - m) : 0.f;
        s_w[s] = e;
        if (ms != -INFINITY) l += __ldcg(base + s * stride + 1) * e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) s_red[1][warp] = l;
    __syncthreads();
    l = 0.f;
    for (int w = 0; w < nwarps; ++w) l += s_red[1][w];
    for (int64_t dvi = tid; dvi < a.dv; dvi += blockDim.x) {
        float o = 0.f;
        if (m != -INFINITY) {
            // unconditional loads (every split wrote its accumulator, zeros if it had no key): they pipeline
#pragma unroll 8
            for (int s = 0; s < a.splits; ++s) o = fmaf(__ldcg(base + s * stride + ATT_HDR + dvi), s_w[s], o);
            o = o / l;
        }
        a.out[(h * a.nq + q) * a.dv + dvi] = o;
    }
}

// The same merge for the G heads of a KV group at once, by the CTA that delivered the group's last partial
// (splits <= ATT_FUSED_SPLITS, dv = 128 D4).  It is one round trip to L2 deep: every thread first requests its
// share of the accumulators (a float4 column of one head, a 1/P share of the splits, up to ATT_MERGE_BATCH loads in
// flight), then warp g turns head g's (m, l) pairs - one float2 load per split - into the weights exp(m_s - m) in
// shared memory, and only then are the requested accumulators weighted and summed.
constexpr int ATT_FUSED_SPLITS = 128;
constexpr int ATT_MERGE_BATCH = 20;

template <int G, int D4>
__device__ __forceinline__ void attn_merge_group(const AttnArgs & a, int64_t q, int64_t hk, float * s_w, float * s_l, float4 * s_part) {
    constexpr int COLS = 32 * D4;                      // float4 columns per head
    constexpr int ITEMS = G * COLS;
    constexpr int P = ITEMS >= ATT_THREADS ? 1 : ATT_THREADS / ITEMS;   // threads per column, each with a share of the splits
    constexpr int ROUNDS = (ITEMS + ATT_THREADS - 1) / ATT_THREADS;
    constexpr int ACTIVE = ITEMS < ATT_THREADS ? ITEMS : ATT_THREADS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t stride = a.dv + ATT_HDR;
    const int64_t st4 = stride / 4;
    const float * gbase = a.scratch + scratch_index(a, q, hk * G, 0);   // head g of the group: + g * splits * stride
    const int item = tid % ACTIVE, part = tid / ACTIVE;
    const int per = (a.splits + P - 1) / P;
    const int s_begin = part * per;
    const int s_end = s_begin + per < a.splits ? s_begin + per : a.splits;
    const float4 * col0 = reinterpret_cast<const float4 *>(gbase + (int64_t) (item / COLS) * a.splits * stride + ATT_HDR) + item % COLS;
    float4 pre[ATT_MERGE_BATCH];
#pragma unroll
    for (int i = 0; i < ATT_MERGE_BATCH; ++i)
        pre[i] = s_begin + i < s_end ? __ldcg(col0 + (int64_t) (s_begin + i) * st4) : make_float4(0.f, 0.f, 0.f, 0.f);

    if (warp < G) {
        const float * base = gbase + (int64_t) warp * a.splits * stride;
        float2 ml[ATT_FUSED_SPLITS / 32];
        float m = -INFINITY;
#pragma unroll
        for (int i = 0; i < ATT_FUSED_SPLITS / 32; ++i) {
            const int sp = lane + 32 * i;
            ml[i] = sp < a.splits ? __ldcg(reinterpret_cast<const float2 *>(base + (int64_t) sp * stride)) : make_float2(-INFINITY, 0.f);
            m = fmaxf(m, ml[i].x);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        float l = 0.f;
#pragma unroll
        for (int i = 0; i < ATT_FUSED_SPLITS / 32; ++i) {
            const int sp = lane + 32 * i;
            const float e = ml[i].x != -INFINITY ? expf(ml[i].x - m) : 0.f;
            if (sp < a.splits) s_w[warp * ATT_FUSED_SPLITS + sp] = e;
            l = fmaf(ml[i].y, e, l);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
        if (lane == 0) s_l[warp] = m == -INFINITY ? 0.f : l;   // 0: no visible key at all
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < ROUNDS; ++r) {
        const int it = item + r * ATT_THREADS;     // ROUNDS > 1 only with P == 1
        const int g = it / COLS, c = it % COLS;
        const float * w = s_w + g * ATT_FUSED_SPLITS;
        const float4 * col = reinterpret_cast<const float4 *>(gbase + (int64_t) g * a.splits * stride + ATT_HDR) + c;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int sp = s_begin;
        if (r == 0) {
#pragma unroll
            for (int i = 0; i < ATT_MERGE_BATCH; ++i) {
                const float ws = s_begin + i < s_end ? w[s_begin + i] : 0.f;
                acc.x = fmaf(pre[i].x, ws, acc.x); acc.y = fmaf(pre[i].y, ws, acc.y);
                acc.z = fmaf(pre[i].z, ws, acc.z); acc.w = fmaf(pre[i].w, ws, acc.w);
            }
            sp = s_begin + ATT_MERGE_BATCH;
        }
#pragma unroll 8
        for (; sp < s_end; ++sp) {
            const float4 v = __ldcg(col + (int64_t) sp * st4);
            const float ws = w[sp];
            acc.x = fmaf(v.x, ws, acc.x); acc.y = fmaf(v.y, ws, acc.y);
            acc.z = fmaf(v.z, ws, acc.z); acc.w = fmaf(v.w, ws, acc.w);
        }
        if (P > 1) {
            if (part > 0) s_part[(part - 1) * ITEMS + item] = acc;
            __syncthreads();
            if (part == 0) {
#pragma unroll
                for (int pp = 1; pp < P; ++pp) {
                    const float4 v = s_part[(pp - 1) * ITEMS + item];
                    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                }
            }
        }
        if (part == 0) {
            const float l = s_l[g];
            reinterpret_cast<float4 *>(a.out + ((hk * G + g) * a.nq + q) * a.dv)[c] =
                l != 0.f ? make_float4(acc.x / l, acc.y / l, acc.z / l, acc.w / l) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
}

__global__ void attn_combine_kernel(AttnArgs a) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float s_w[ATT_MAX_SPLITS];
    __shared__ float s_red[2][32];
    attn_merge_head(a, blockIdx.y, blockIdx.x, s_w, s_red);
}

// Single-pass partial for head dimensions that are multiples of 128 (D = Dv = 128 D4) and G = 1, 2, 4 or 8 query
// heads per KV head.  A warp takes every 8th key of the split: the key's K and V rows are requested together
// (one float4 per lane and 128 elements), the scores of the G heads are warp-reduced, and a running
// (max, sum, accumulator) per head is updated in registers (online softmax) - one trip to memory per key instead of
// the three phases of the generic kernel.  The 8 warps are merged through shared memory into the split's partial;
// the CTA that delivers the last partial of a (query, KV head) merges the splits right away (counter in global
// memory, reset for the next call), so no second launch is needed.

// RMS norm (optional) and NEOX rotation of one head of 128 D4 elements held by a warp as float4 per lane and 128-element
// slab (elements 4 lane .. 4 lane + 3 of slab i), with the arithmetic of head_post_kernel (sm100_ops.cu): the values of
// RMS_NORM_MUL (src/core/ref/ops.cpp:466-492) and ROPE (:530-634) for one token.  The rotation pairs element j with j + D/2:
// for D = 128 that is the lane 16 away, for D = 256 the other slab of the same lane.
template <int D4>
__device__ __forceinline__ void post_head(const float * src, const float * w, const AttnArgs & a, int32_t pos, int lane, float4 (&out)[D4]) {
    constexpr int D = 128 * D4, HP = D / 2;
    float4 x[D4];
    double sum = 0.0;
#pragma unroll
    for (int i = 0; i < D4; ++i) {
        x[i] = __ldcg(reinterpret_cast<const float4 *>(src) + lane + 32 * i);
        sum += ((double) x[i].x * (double) x[i].x + (double) x[i].y * (double) x[i].y) + ((double) x[i].z * (double) x[i].z + (double) x[i].w * (double) x[i].w);
    }
    if (w != nullptr) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float) (sum * (1.0 / (double) D)), a.eps)));   // D is a power of two: the same double as sum / D
#pragma unroll
        for (int i = 0; i < D4; ++i) {
            const float4 g = __ldg(reinterpret_cast<const float4 *>(w) + lane + 32 * i);
            x[i] = make_float4(__fmul_rn(__fmul_rn(x[i].x, scale), g.x), __fmul_rn(__fmul_rn(x[i].y, scale), g.y),
                               __fmul_rn(__fmul_rn(x[i].z, scale), g.z), __fmul_rn(__fmul_rn(x[i].w, scale), g.w));
        }
    }
    // pair index of this lane's component c: j0 + c
    const int j0 = D4 == 1 ? 4 * (lane & 15) : 4 * lane;
    const int64_t rel = (int64_t) pos - a.table_first;
    const bool in_table = a.table != nullptr && rel >= 0 && rel < a.table_n;
    float cs[4], sn[4];
    if (in_table) {
        const float4 t0 = __ldg(reinterpret_cast<const float4 *>(a.table + (rel * HP + j0) * 2));
        const float4 t1 = __ldg(reinterpret_cast<const float4 *>(a.table + (rel * HP + j0) * 2) + 1);
        cs[0] = t0.x; sn[0] = t0.y; cs[1] = t0.z; sn[1] = t0.w; cs[2] = t1.x; sn[2] = t1.y; cs[3] = t1.z; sn[3] = t1.w;
    } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float theta = (float) pos;
            for (int q = 0; q < j0 + c; ++q) theta = __fmul_rn(theta, a.theta_scale);
            cs[c] = cosf(theta);
            sn[c] = sinf(theta);
        }
    }
    if (D4 == 1) {
        const bool lower = lane < 16;
        const float4 p = make_float4(__shfl_xor_sync(0xffffffffu, x[0].x, 16), __shfl_xor_sync(0xffffffffu, x[0].y, 16),
                                     __shfl_xor_sync(0xffffffffu, x[0].z, 16), __shfl_xor_sync(0xffffffffu, x[0].w, 16));
        const float mine[4] = {x[0].x, x[0].y, x[0].z, x[0].w}, other[4] = {p.x, p.y, p.z, p.w};
        float y[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float v0 = lower ? mine[c] : other[c], v1 = lower ? other[c] : mine[c];
            y[c] = lower ? __fsub_rn(__fmul_rn(v0, cs[c]), __fmul_rn(v1, sn[c])) : __fadd_rn(__fmul_rn(v0, sn[c]), __fmul_rn(v1, cs[c]));
        }
        out[0] = make_float4(y[0], y[1], y[2], y[3]);
    } else {
        const float v0[4] = {x[0].x, x[0].y, x[0].z, x[0].w}, v1[4] = {x[D4 - 1].x, x[D4 - 1].y, x[D4 - 1].z, x[D4 - 1].w};
        float y0[4], y1[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            y0[c] = __fsub_rn(__fmul_rn(v0[c], cs[c]), __fmul_rn(v1[c], sn[c]));
            y1[c] = __fadd_rn(__fmul_rn(v0[c], sn[c]), __fmul_rn(v1[c], cs[c]));
        }
        out[0] = make_float4(y0[0], y0[1], y0[2], y0[3]);
        out[D4 - 1] = make_float4(y1[0], y1[1], y1[2], y1[3]);
    }
}

template <int G, int D4, bool POST>
__global__ void __launch_bounds__(ATT_THREADS) attn_fast_kernel(AttnArgs a) {
    constexpr int D = 128 * D4;
    extern __shared__ __align__(16) float smem[];   // [8 warps][G][ATT_HDR + D]
    constexpr int SROW = ATT_HDR + D;
    __shared__ float s_w[ATT_MAX_SPLITS];
    __shared__ float s_red[2][32];
    __shared__ int s_last;
    __shared__ float4 s_q[POST ? G * D4 * 32 : 1];   // POST: the group's query heads after norm and rotation
    const int split = blockIdx.x;
    const int64_t hk = blockIdx.y, q = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int NW = ATT_THREADS / 32;
    // A warp takes NKB consecutive keys per trip: their K and V rows are requested together, the G x NKB partial
    // dot products are reduced over the lanes with a halving exchange (NV values cost NV - 1 + log2(32 / NV)
    // shuffles instead of 5 NV) and handed to all lanes through the warp's own shared-memory slot.
    constexpr int NKB = D4 == 1 ? 4 : 2;
    constexpr int NV = G * NKB;

    const bool early = a.fresh_keys >= 0;   // warp-uniform: see AttnArgs
    if (!early) pdl_wait();

    // the visible keys (known only on the device when the offset comes from `positions`) are spread evenly over the splits
    const int64_t n_vis = visible_keys(a, q);
    const int64_t chunk = (n_vis + a.splits - 1) / a.splits;
    const int64_t k0 = (int64_t) split * chunk;
    const int64_t k1 = k0 + chunk < n_vis ? k0 + chunk : n_vis;
    const int count = k1 > k0 ? (int) (k1 - k0) : 0;
    const float4 * kbase = reinterpret_cast<const float4 *>(a.k + (hk * a.nk + k0) * D) + lane;
    const float4 * vbase = reinterpret_cast<const float4 *>(a.v + (hk * a.nk + k0) * D) + lane;

    float4 kv[NKB][D4], vv[NKB][D4];
    int kb = warp * NKB;
    if (early) {
        // the first trip's stable rows are on their way while the preceding kernel finishes
        const int64_t stable = n_vis - a.fresh_keys - k0;   // keys of this split below this index are stable
#pragma unroll
        for (int j = 0; j < NKB; ++j) {
            const bool in = kb + j < count && kb + j < stable;
#pragma unroll
            for (int i = 0; i < D4; ++i) {
                kv[j][i] = in ? kbase[(int64_t) (kb + j) * (D / 4) + 32 * i] : make_float4(0.f, 0.f, 0.f, 0.f);
                vv[j][i] = in ? vbase[(int64_t) (kb + j) * (D / 4) + 32 * i] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        pdl_wait();
        if constexpr (POST) {
            // The new token's heads, once per CTA: warp t takes query head t of this KV head's group (normalised and rotated
            // into shared memory, from where every warp fetches all G of them); in the CTA whose split ends at the newest
            // position two more tasks make and store the new key and copy the new value into the caches (CTA-uniform
            // condition), where the loop below finds them like any other row.
            const int32_t pos = a.positions[0];
            const bool owns_newest = n_vis > 0 && n_vis - 1 >= k0 && n_vis - 1 < k1 && pos >= 0 && pos < a.nk;
            const int tasks = G + (owns_newest ? 2 : 0);
            for (int task = warp; task < tasks; task += NW) {
                if (task < G) {
                    float4 qn[D4];
                    post_head<D4>(a.q + (hk * G + task) * D, a.q_w, a, pos, lane, qn);
#pragma unroll
                    for (int i = 0; i < D4; ++i) s_q[(task * D4 + i) * 32 + lane] = qn[i];
                } else if (task == G) {
                    float4 kn[D4];
                    post_head<D4>(a.k_new + hk * D, a.k_w, a, pos, lane, kn);
                    float4 * dst = reinterpret_cast<float4 *>(const_cast<float *>(a.k) + (hk * a.nk + pos) * D);
#pragma unroll
                    for (int i = 0; i < D4; ++i) dst[lane + 32 * i] = kn[i];
                } else {
                    const float4 * src = reinterpret_cast<const float4 *>(a.v_new + hk * D);
                    float4 * dst = reinterpret_cast<float4 *>(const_cast<float *>(a.v) + (hk * a.nk + pos) * D);
#pragma unroll
                    for (int i = 0; i < D4; ++i) dst[lane + 32 * i] = __ldcg(src + lane + 32 * i);
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int j = 0; j < NKB; ++j) {
            const bool in = kb + j < count && kb + j >= stable;
            if (in) {
#pragma unroll
                for (int i = 0; i < D4; ++i) {
                    kv[j][i] = POST ? __ldcg(kbase + (int64_t) (kb + j) * (D / 4) + 32 * i) : kbase[(int64_t) (kb + j) * (D / 4) + 32 * i];
                    vv[j][i] = POST ? __ldcg(vbase + (int64_t) (kb + j) * (D / 4) + 32 * i) : vbase[(int64_t) (kb + j) * (D / 4) + 32 * i];
                }
            }
        }
    }
    pdl_launch_dependents();

    float4 qr[G][D4];
    if constexpr (POST) {
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int i = 0; i < D4; ++i) qr[g][i] = s_q[(g * D4 + i) * 32 + lane];
    } else {
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int i = 0; i < D4; ++i) qr[g][i] = reinterpret_cast<const float4 *>(a.q + ((hk * G + g) * a.nq + q) * D)[lane + 32 * i];
    }

    float m[G], l[G];
    float4 o[G][D4];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < D4; ++i) o[g][i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float * my_scores = smem + warp * G * SROW;   // first NV floats of the area this warp fills after the loop
    bool have = early;   // the first trip's rows are already requested
    for (; kb < count; kb += NW * NKB) {
        if (!have) {
#pragma unroll
            for (int j = 0; j < NKB; ++j) {
                const bool in = kb + j < count;
#pragma unroll
                for (int i = 0; i < D4; ++i) {
                    // (POST: the newest row was stored by this CTA a moment ago: read past L1)
                    kv[j][i] = !in ? make_float4(0.f, 0.f, 0.f, 0.f) : POST ? __ldcg(kbase + (int64_t) (kb + j) * (D / 4) + 32 * i) : kbase[(int64_t) (kb + j) * (D / 4) + 32 * i];
                    vv[j][i] = !in ? make_float4(0.f, 0.f, 0.f, 0.f) : POST ? __ldcg(vbase + (int64_t) (kb + j) * (D / 4) + 32 * i) : vbase[(int64_t) (kb + j) * (D / 4) + 32 * i];
                }
            }
        }
        have = false;
        float part[NV];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int j = 0; j < NKB; ++j) {
                float sc = 0.f;
#pragma unroll
                for (int i = 0; i < D4; ++i)
                    sc += (kv[j][i].x * qr[g][i].x + kv[j][i].y * qr[g][i].y) + (kv[j][i].z * qr[g][i].z + kv[j][i].w * qr[g][i].w);
                part[g * NKB + j] = sc;
            }
        // halving exchange: after the step with offset o a lane keeps the half selected by its bit o
        int n = NV;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            if (n > 1) {
                const bool upper = (lane & off) != 0;
#pragma unroll
                for (int i = 0; i < NV / 2; ++i) {
                    if (i < n / 2) {
                        const float keep = upper ? part[i + n / 2] : part[i];
                        const float give = upper ? part[i] : part[i + n / 2];
                        part[i] = keep + __shfl_xor_sync(0xffffffffu, give, off);
                    }
                }
                n >>= 1;
            } else {
                part[0] += __shfl_xor_sync(0xffffffffu, part[0], off);
            }
        }
        // this lane holds the complete sum of value index (lane * NV) / 32
        __syncwarp();
        my_scores[(lane * NV) >> 5] = part[0];
        __syncwarp();
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float sc[NKB];
            float mx = m[g];
#pragma unroll
            for (int j = 0; j < NKB; ++j) {
                sc[j] = my_scores[g * NKB + j] * a.scale;
                if (a.mask != nullptr && kb + j < count) {
                    const int64_t mh = a.mask_heads == 1 ? 0 : hk * G + g;
                    sc[j] += a.mask[(mh * a.nq + q) * a.nk + k0 + kb + j];
                }
                if (kb + j >= count) sc[j] = -INFINITY;
                mx = fmaxf(mx, sc[j]);
            }
            if (mx != -INFINITY) {   // warp-uniform: every lane holds the same scores
                const float corr = m[g] == -INFINITY ? 0.f : expf(m[g] - mx);
                float pr[NKB], psum = 0.f;
#pragma unroll
                for (int j = 0; j < NKB; ++j) {
                    pr[j] = expf(sc[j] - mx);   // exp(-inf) = 0 for hidden keys
                    psum += pr[j];
                }
                l[g] = fmaf(l[g], corr, psum);
                m[g] = mx;
#pragma unroll
                for (int i = 0; i < D4; ++i) {
                    float4 acc = make_float4(o[g][i].x * corr, o[g][i].y * corr, o[g][i].z * corr, o[g][i].w * corr);
#pragma unroll
                    for (int j = 0; j < NKB; ++j) {
                        acc.x = fmaf(pr[j], vv[j][i].x, acc.x);
                        acc.y = fmaf(pr[j], vv[j][i].y, acc.y);
                        acc.z = fmaf(pr[j], vv[j][i].z, acc.z);
                        acc.w = fmaf(pr[j], vv[j][i].w, acc.w);
                    }
                    o[g][i] = acc;
                }
            }
        }
    }
    __syncwarp();
    // warps -> shared memory: per (warp, head) [m, l, -, -, o[D]]
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float * dst = smem + (warp * G + g) * SROW;
        if (lane == 0) {
            dst[0] = m[g];
            dst[1] = l[g];
        }
#pragma unroll
        for (int i = 0; i < D4; ++i) reinterpret_cast<float4 *>(dst + ATT_HDR)[lane + 32 * i] = o[g][i];
    }
    __syncthreads();
    // weight of each warp's partial within the split, exp(m_w - max_w m_w), computed once per (head, warp)
    float * s_f = s_w;
    if (tid < G * NW) {
        const int g = tid / NW, w = tid % NW;
        float mm = -INFINITY;
#pragma unroll
        for (int w2 = 0; w2 < NW; ++w2) mm = fmaxf(mm, smem[(w2 * G + g) * SROW]);
        const float mw = smem[(w * G + g) * SROW];
        s_f[tid] = mw == -INFINITY ? 0.f : expf(mw - mm);
    }
    __syncthreads();
    // merge the warps into the split's partial per head, a float4 column per thread
    for (int item = tid; item < G * (D / 4); item += ATT_THREADS) {
        const int g = item / (D / 4), c = item - g * (D / 4);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float f = s_f[g * NW + w];
            const float4 v = reinterpret_cast<const float4 *>(smem + (w * G + g) * SROW + ATT_HDR)[c];
            acc.x = fmaf(v.x, f, acc.x); acc.y = fmaf(v.y, f, acc.y);
            acc.z = fmaf(v.z, f, acc.z); acc.w = fmaf(v.w, f, acc.w);
        }
        float * dst = a.scratch + scratch_index(a, q, hk * G + g, split);
        if (c == 0) {
            float mm = -INFINITY, ll = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) {
                mm = fmaxf(mm, smem[(w * G + g) * SROW]);
                ll = fmaf(smem[(w * G + g) * SROW + 1], s_f[g * NW + w], ll);
            }
            *reinterpret_cast<float2 *>(dst) = make_float2(mm, ll);
        }
        reinterpret_cast<float4 *>(dst + ATT_HDR)[c] = acc;
    }
    if (a.counters == nullptr) return;   // the caller merges with a second launch
    // the CTA's partial is complete once all its threads passed the barrier; thread 0 publishes it (the fence is
    // cumulative over what the barrier ordered before it) and takes a ticket
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const int last = atomicAdd(a.counters + q * a.hkv + hk, 1) == a.splits - 1 ? 1 : 0;
        if (last) __threadfence();
        s_last = last;
    }
    __syncthreads();
    if (s_last == 0) return;
    attn_merge_group<G, D4>(a, q, hk, s_w, &s_red[0][0], reinterpret_cast<float4 *>(smem));
    if (tid == 0) a.counters[q * a.hkv + hk] = 0;
}


int device_scratch(int slot, size_t bytes, void ** out);

static int workspace(size_t bytes, float ** out) {
    void * p = nullptr;
    const int st = device_scratch(0, bytes, &p);
    *out = (float *) p;
    return st;
}

constexpr int ATT_COUNTER_SLOTS = 16384;   // ints at the start of the scratch: one per (query, KV head) of a call

template <int G, int D4>
static int launch_fast(cudaStream_t s, const AttnArgs & a) {
    const size_t smem = (size_t) (ATT_THREADS / 32) * G * (128 * D4 + ATT_HDR) * sizeof(float);
    if (a.k_new != nullptr) {
        if (smem > 48 * 1024) SM100_CUDA(cudaFuncSetAttribute(attn_fast_kernel<G, D4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        return launch(attn_fast_kernel<G, D4, true>, dim3((unsigned) a.splits, (unsigned) a.hkv, (unsigned) a.nq), dim3(ATT_THREADS), smem, s, a);
    }
    if (smem > 48 * 1024) SM100_CUDA(cudaFuncSetAttribute(attn_fast_kernel<G, D4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
    return launch(attn_fast_kernel<G, D4, false>, dim3((unsigned) a.splits, (unsigned) a.hkv, (unsigned) a.nq), dim3(ATT_THREADS), smem, s, a);
}

// `scratch` is the raw scratch area: counters first, partials behind them
int attention_launch(cudaStream_t s, AttnArgs a, float * scratch) {
    const int group = (int) (a.hq / a.hkv);
    a.counters = nullptr;
    a.scratch = scratch + ATT_COUNTER_SLOTS;
    static const int use_fast = [] { const char * e = getenv("SM100_ATTN_FAST"); return e != nullptr ? atoi(e) : 1; }();
    const bool aligned = (((uintptr_t) a.q | (uintptr_t) a.k | (uintptr_t) a.v | (uintptr_t) a.out | (uintptr_t) scratch) & 15) == 0;
    if (use_fast && a.d == a.dv && (a.d == 128 || a.d == 256) && aligned && (group == 1 || group == 2 || group == 4 || group == 8)) {
        const bool fused = a.nq * a.hkv <= ATT_COUNTER_SLOTS && a.splits <= ATT_FUSED_SPLITS;
        if (fused) a.counters = reinterpret_cast<int *>(scratch);
        int st;
        const int d4 = (int) (a.d / 128);
        switch (group * 10 + d4) {
            case 11: st = launch_fast<1, 1>(s, a); break;
            case 12: st = launch_fast<1, 2>(s, a); break;
            case 21: st = launch_fast<2, 1>(s, a); break;
            case 22: st = launch_fast<2, 2>(s, a); break;
            case 41: st = launch_fast<4, 1>(s, a); break;
            case 42: st = launch_fast<4, 2>(s, a); break;
            case 81: st = launch_fast<8, 1>(s, a); break;
            default: st = launch_fast<8, 2>(s, a); break;
        }
        if (st != ST_OK || fused) return st;
    } else {
        const size_t smem = ((size_t) group * a.d + (size_t) group * a.chunk + (size_t) group * a.dv) * sizeof(float);
        if (smem > 48 * 1024) {
            SM100_CUDA(cudaFuncSetAttribute(attn_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
        }
        const int st = launch(attn_partial_kernel, dim3((unsigned) a.splits, (unsigned) a.hkv, (unsigned) a.nq), dim3(ATT_THREADS), smem, s, a);
        if (st != ST_OK) return st;
    }
    const int ct = a.dv >= 256 ? 256 : a.dv >= 128 ? 128 : 64;
    return launch(attn_combine_kernel, dim3((unsigned) a.hq, (unsigned) a.nq), dim3(ct), 0, s, a);
}

int attention_check(const AttnArgs & a) {
    if (a.q == nullptr || a.k == nullptr || a.v == nullptr || a.out == nullptr) return fail(ST_INVALID, "attention: null tensor pointer");
    if (a.d <= 0 || a.dv <= 0 || a.nq <= 0 || a.nk <= 0 || a.hq <= 0 || a.hkv <= 0) return fail(ST_INVALID, "attention: dimensions must be positive");
    if (a.hq % a.hkv != 0) return fail(ST_INVALID, "attention: Hq must be divisible by Hkv");
    if (a.nk > (int64_t) ATT_CHUNK * ATT_MAX_SPLITS) return fail(ST_UNSUPPORTED, "attention: more than %d keys", ATT_CHUNK * ATT_MAX_SPLITS);
    if (a.hq / a.hkv > ATT_MAX_GROUP) return fail(ST_UNSUPPORTED, "attention: more than 8 query heads per KV head");
    if (a.nq > 65535 || a.hkv > 65535) return fail(ST_UNSUPPORTED, "attention: too many queries or KV heads for one launch");
    if (a.d > 1024 || a.dv > 1024) return fail(ST_UNSUPPORTED, "attention: head dimension above 1024");
    return ST_OK;
}

size_t attention_scratch_bytes(const AttnArgs & a) {
    return ((size_t) ATT_COUNTER_SLOTS + (size_t) a.nq * a.hq * a.splits * (a.dv + ATT_HDR)) * sizeof(float);
}

void attention_plan(AttnArgs & a) {
    // enough splits to occupy the SMs, at most ATT_CHUNK keys per split
    const int64_t ctas_wanted = (int64_t) sm_count() * 2;
    int64_t per_head = a.hkv * a.nq;
    int64_t splits = (ctas_wanted + per_head - 1) / per_head;
    int64_t chunk = (a.nk + splits - 1) / splits;
    if (chunk < 32) chunk = 32;
    if (chunk > ATT_CHUNK) chunk = ATT_CHUNK;   // attention_check bounds nk so that this leaves at most ATT_MAX_SPLITS splits
    a.chunk = (int) chunk;
    a.splits = (int) ((a.nk + chunk - 1) / chunk);
}

}  // namespace sm100

using namespace sm100;

static int attention_entry(sm100_stream_t s, const float * q, const float * k, const float * v, const float * mask, int64_t mask_heads,
                           float * out, int64_t d, int64_t dv, int64_t nq, int64_t nk, int64_t hq, int64_t hkv, int causal, int64_t offset,
                           const int32_t * positions, float scale, int fresh_keys) {
    AttnArgs a = {};
    a.q = q; a.k = k; a.v = v; a.mask = mask; a.out = out; a.positions = positions;
    a.d = d; a.dv = dv; a.nq = nq; a.nk = nk; a.hq = hq; a.hkv = hkv; a.offset = offset;
    a.mask_heads = mask_heads <= 1 ? 1 : mask_heads;
    a.causal = causal; a.scale = scale;
    a.fresh_keys = fresh_keys;
    const int st = attention_check(a);
    if (st != ST_OK) return st;
    attention_plan(a);
    float * ws = nullptr;
    const int sw = workspace(attention_scratch_bytes(a), &ws);
    if (sw != ST_OK) return sw;
    return attention_launch((cudaStream_t) s, a, ws);
}

extern "C" int sm100_attention(sm100_stream_t s, const float * q, const float * k, const float * v, const float * mask, int64_t mask_heads,
                               float * out, int64_t d, int64_t dv, int64_t nq, int64_t nk, int64_t hq, int64_t hkv, int causal,
                               int64_t offset, const int32_t * positions, float scale) {
    return attention_entry(s, q, k, v, mask, mask_heads, out, d, dv, nq, nk, hq, hkv, causal, offset, positions, scale, -1);
}

extern "C" int sm100_attention_kvcache(sm100_stream_t s, const float * q, const float * k, const float * v, const float * mask,
                                       int64_t mask_heads, float * out, int64_t d, int64_t dv, int64_t nq, int64_t nk, int64_t hq, int64_t hkv,
                                       int causal, int64_t offset, const int32_t * positions, float scale, int fresh_keys) {
    if (fresh_keys < 0) return sm100::fail(sm100::ST_INVALID, "attention (KV cache): fresh_keys must not be negative");
    return attention_entry(s, q, k, v, mask, mask_heads, out, d, dv, nq, nk, hq, hkv, causal, offset, positions, scale, fresh_keys);
}



extern "C" int sm100_attention_decode(sm100_stream_t s, float * q, float * k_new, const float * v_new, const float * q_norm_w, const float * k_norm_w,
                                      const int32_t * positions, const float * table, int32_t table_first, int32_t table_n, float * k_cache,
                                      float * v_cache, float * out, int64_t head_dim, int64_t q_heads, int64_t kv_heads, int64_t cache_rows, float eps,
                                      float freq_base, int neox, float scale) {
    using namespace sm100;
    if (q == nullptr || k_new == nullptr || v_new == nullptr || positions == nullptr || k_cache == nullptr || v_cache == nullptr || out == nullptr)
        return fail(ST_INVALID, "attention_decode: null pointer");
    if (head_dim <= 0 || q_heads <= 0 || kv_heads <= 0 || cache_rows <= 0 || q_heads % kv_heads != 0) return fail(ST_INVALID, "attention_decode: bad shape");
    const int64_t group = q_heads / kv_heads;
    static const int fuse = [] { const char * e = getenv("SM100_ATTN_POST"); return e != nullptr ? atoi(e) : 1; }();
    const bool aligned = (((uintptr_t) q | (uintptr_t) k_new | (uintptr_t) v_new | (uintptr_t) q_norm_w | (uintptr_t) k_norm_w | (uintptr_t) table |
                           (uintptr_t) k_cache | (uintptr_t) v_cache | (uintptr_t) out) & 15) == 0;
    if (fuse && neox && aligned && (head_dim == 128 || head_dim == 256) && (group == 1 || group == 2 || group == 4 || group == 8)) {
        AttnArgs a = {};
        a.q = q; a.k = k_cache; a.v = v_cache; a.out = out; a.positions = positions;
        a.d = head_dim; a.dv = head_dim; a.nq = 1; a.nk = cache_rows; a.hq = q_heads; a.hkv = kv_heads; a.offset = 0;
        a.mask_heads = 1;
        a.causal = 1; a.scale = scale;
        a.fresh_keys = 1;
        a.k_new = k_new; a.v_new = v_new; a.q_w = q_norm_w; a.k_w = k_norm_w; a.table = table; a.table_first = table_first; a.table_n = (int) table_n;
        a.eps = eps;
        a.theta_scale = powf(freq_base, -2.0f / (float) head_dim);
        int st = attention_check(a);
        if (st != ST_OK) return st;
        attention_plan(a);
        if ((int64_t) a.nq * a.hkv <= ATT_COUNTER_SLOTS && a.splits <= ATT_FUSED_SPLITS) {   // the single-launch form of the fast kernel
            float * ws = nullptr;
            st = workspace(attention_scratch_bytes(a), &ws);
            if (st != ST_OK) return st;
            return attention_launch((cudaStream_t) s, a, ws);
        }
    }
    // the separate launches
    const int st = sm100_head_post(s, q, k_new, v_new, q_norm_w, k_norm_w, positions, table, table_first, table_n, k_cache, v_cache, head_dim, q_heads,
                                   kv_heads, cache_rows, eps, freq_base, neox);
    if (st != ST_OK) return st;
    return sm100_attention_kvcache(s, q, k_cache, v_cache, nullptr, 1, out, head_dim, head_dim, 1, cache_rows, q_heads, kv_heads, 1, 0, positions, scale, 1);
}

// ---------------------------------------------------------------------------------------------------------
// Attention without any allocation.
//
// Some hosts may not allocate device memory when they call in: a serving loop that has already handed every byte
// of HBM to its own pools, a real-time thread that must not take the driver's allocator lock, code running under
// a memory budget enforced from outside.  For them the split-key partials live in a fixed array that is part of
// this library's image: every GPU that loads the library carries these 4 MiB until the process exits.
//
// In host code the name of a __device__ array is only a stand-in symbol, not a device address, so the address is
// looked up with cudaGetSymbolAddress once per device (with that device current) and cached; the FIRST call on a
// device does this look-up, so make that first call outside of any stream capture.  All calls on a device share
// the one array: two calls whose kernels overlap on the GPU (different streams) race on it.
//
// What must start at zero: the first ATT_COUNTER_SLOTS ints of the array are the ticket counters of the single-launch
// merge, one per (query, KV head): the CTA that draws the last ticket merges the splits and puts the counter back
// to zero.  A call that raced with another one, or a launch that ended between drawing and resetting, would leave
// a counter non-zero and every later call on that device would merge too early or never.  So this entry does not
// rely on what the previous call left behind: it clears the counters it is going to use with a memset on the
// caller's stream in front of the launch (a memset node, no allocation).  The partials behind the counters need no
// clearing: every entry the merge reads is written by the same call first.  The counters take 64 KiB of the array;
// the partials of one call may use the remaining 4 MiB - 64 KiB.
// ---------------------------------------------------------------------------------------------------------
namespace sm100 {

constexpr size_t ATT_STATIC_FLOATS = (size_t) 1 << 20;   // 4 MiB
static __device__ __align__(256) float g_attn_static_scratch[ATT_STATIC_FLOATS];

constexpr int ATT_STATIC_MAX_DEVICES = 64;
static std::mutex g_static_mutex;
static float * g_static_ptr[ATT_STATIC_MAX_DEVICES] = {};

static int static_scratch(float ** out) {
    int dev = 0;
    SM100_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= ATT_STATIC_MAX_DEVICES) return fail(ST_UNSUPPORTED, "attention (static scratch): device ordinal %d is beyond the table of %d", dev, ATT_STATIC_MAX_DEVICES);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_ptr[dev] == nullptr) {
        void * p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_attn_static_scratch);   // the current device's copy of the array
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(attention scratch)");
        if (p == nullptr) return fail(ST_BACKEND, "attention (static scratch): the symbol has no device address");
        g_static_ptr[dev] = static_cast<float *>(p);
    }
    *out = g_static_ptr[dev];
    return ST_OK;
}

}  // namespace sm100

extern "C" int sm100_attention_static(sm100_stream_t s, const float * q, const float * k, const float * v, const float * mask, int64_t mask_heads,
                                      float * out, int64_t d, int64_t dv, int64_t nq, int64_t nk, int64_t hq, int64_t hkv, int causal,
                                      int64_t offset, const int32_t * positions, float scale) {
    AttnArgs a = {};
    a.q = q; a.k = k; a.v = v; a.mask = mask; a.out = out; a.positions = positions;
    a.d = d; a.dv = dv; a.nq = nq; a.nk = nk; a.hq = hq; a.hkv = hkv; a.offset = offset;
    a.mask_heads = mask_heads <= 1 ? 1 : mask_heads;
    a.causal = causal; a.scale = scale;
    a.fresh_keys = -1;
    const int st = attention_check(a);
    if (st != ST_OK) return st;
    attention_plan(a);
    const size_t need = attention_scratch_bytes(a);
    if (need > ATT_STATIC_FLOATS * sizeof(float))
        return fail(ST_UNSUPPORTED, "attention (static scratch): this shape needs %zu bytes of split-key partials, the built-in array holds %zu; use sm100_attention",
                    need, ATT_STATIC_FLOATS * sizeof(float));
    float * ws = nullptr;
    const int sw = static_scratch(&ws);
    if (sw != ST_OK) return sw;
    const size_t used_counters = (size_t) a.nq * a.hkv < (size_t) ATT_COUNTER_SLOTS ? (size_t) a.nq * a.hkv : (size_t) ATT_COUNTER_SLOTS;
    SM100_CUDA(cudaMemsetAsync(ws, 0, used_counters * sizeof(int), (cudaStream_t) s));   // see above: never trust the last call's counters
    return attention_launch((cudaStream_t) s, a, ws);
}

extern "C" size_t sm100_attention_static_capacity(void) { return sm100::ATT_STATIC_FLOATS * sizeof(float); }

extern "C" int sm100_attention_static_prepare(void ** device_address_out) {
    float * ws = nullptr;
    const int sw = sm100::static_scratch(&ws);
    if (sw != sm100::ST_OK) return sw;
    if (device_address_out != nullptr) *device_address_out = ws;
    return sm100::ST_OK;
}
