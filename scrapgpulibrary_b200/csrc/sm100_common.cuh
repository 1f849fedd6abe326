// Shared declarations of libscrapgpu_sm100: status codes, error reporting, launch helpers.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "scrapgpu_sm100.h"

namespace sm100 {

// scrapgpu_status values (include/scrapgpu/status.h:10-17 of the reference)
enum : int { ST_OK = 0, ST_UNSUPPORTED = 1, ST_INVALID = 2, ST_OOM = 3, ST_BACKEND = 4, ST_LOST = 5 };

// scrapgpu_dtype values (include/scrapgpu/tensor.h:10-22)
enum : int { DT_F32 = 0, DT_F16 = 1, DT_I32 = 2, DT_Q4_0 = 16, DT_Q8_0 = 17, DT_Q4_K = 32, DT_Q6_K = 33 };

enum : int { LAYOUT_NATURAL = 0, LAYOUT_PACKED = 1 };

int fail(int status, const char * fmt, ...);
int cuda_fail(cudaError_t e, const char * what);

#define SM100_CUDA(call)                                          \
    do {                                                          \
        cudaError_t e_ = (call);                                  \
        if (e_ != cudaSuccess) return ::sm100::cuda_fail(e_, #call); \
    } while (0)

inline int block_elems(int dtype) {
    switch (dtype) {
        case DT_Q4_0: case DT_Q8_0: return 32;
        case DT_Q4_K: case DT_Q6_K: return 256;
        case DT_F32: case DT_F16: case DT_I32: return 1;
        default: return 0;
    }
}

inline int block_bytes(int dtype) {
    switch (dtype) {
        case DT_Q4_0: return 18;
        case DT_Q8_0: return 34;
        case DT_Q4_K: return 144;
        case DT_Q6_K: return 210;
        case DT_F32: case DT_I32: return 4;
        case DT_F16: return 2;
        default: return 0;
    }
}

inline bool is_quant(int dtype) { return block_elems(dtype) > 1; }

// producer of a matvec's activation column folded into the matvec (sm100_mul_mat_fused)
struct Q4KPrologue {
    int mode;             // 0 none, 1 x = swiglu(a, b), 2 s = a (+ b), x = rms_norm(s) * norm_w
    const float * a; const float * b; const float * norm_w;
    float * sum_out; float * x_out;   // mode 2: s and x are also written here when set (must not alias a / b)
    float eps;
};

// All-reduce folded into the last phase of a K-sharded matvec: what the kernel needs of an all-reduce context
// (sm100_collective.cu).  Every CTA stores the partial sums of its row tiles, each value in one 8-byte word with the step
// number as its tag, into its slot of every rank's receive area, then adds the slots in rank order, waiting (bounded) for
// each value's tag: the latency of one peer store, no fence, no flag (the scheme of NCCL's low-latency protocol).
constexpr int AR_MAX_RANKS = 8;
constexpr uint32_t AR_WAIT_LIMIT = 1u << 22;   // polls (each with a short sleep) before a rank gives up: ~1 s
struct ArFuse {
    uint2 * recv[AR_MAX_RANKS];       // every rank's receive area [2][world][capacity] of (value bits, step tag) (entry `rank` is the local one)
    uint32_t * step;                  // local: fused launches completed so far (the tag of the next one is this + 1)
    uint32_t * done;                  // local: CTAs of the running fused launch that have finished (the last one advances `step`)
    int * fault;                      // local: set when a wait ran out
    int rank, world, capacity;
    uint32_t wait_limit;              // polls before a wait gives up (AR_WAIT_LIMIT unless the context was told otherwise)
};
bool allreduce_fuse_args(void * ctx, ArFuse * out);   // false when ctx is null

int sm_count();          // SMs of the current device (cached per device)
int current_device();    // ordinal of the current device (0 when it cannot be read)

// One "a kernel with bounded waits was launched" mark per device: the kernel's fault word is a __device__ variable,
// i.e. one copy per device, and it is read back after a stream synchronisation only on devices that launched one.
constexpr int MAX_DEVICES = 64;
bool pdl_enabled();
void count_launch();
// What the library launched last on a stream, as far as the dispatcher of the Q4_K matvec cares: TAIL_Q4K_MATVEC after
// a single-tensor, single-column packed Q4_K matvec by matvec_q4k_imma, TAIL_Q4K_RING after one by matvec_q4k_ring
// (both set by the host functions), TAIL_OTHER after any other launch or copy of this library (launch() and the copy
// entries reset it).
enum { TAIL_OTHER = 0, TAIL_Q4K_MATVEC = 1, TAIL_Q4K_RING = 2 };
void stream_tail_set(cudaStream_t stream, int kind);
int stream_tail(cudaStream_t stream);
// launches of the calling thread without programmatic dependent launch while `on` (sm100_launch_serialized)
void thread_serialized(bool on);

// Launches `kernel` on `stream`; with programmatic dependent launch when enabled, so the kernel may
// start (and prefetch) while its predecessor on the stream drains.  Kernels launched through this
// must execute griddepcontrol.wait before they read anything a predecessor wrote or write anything.
template <typename... KArgs, typename... Args>
int launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (pdl_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) return cuda_fail(e, "kernel launch");
    stream_tail_set(stream, TAIL_OTHER);
    count_launch();
    return ST_OK;
}

// The same with a thread-block cluster of `cluster_x` CTAs along x (grid.x must be a multiple of it).
template <typename... KArgs, typename... Args>
int launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, unsigned cluster_x, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) return cuda_fail(e, "kernel launch (cluster)");
    stream_tail_set(stream, TAIL_OTHER);
    count_launch();
    return ST_OK;
}

// ---- activations as 16-bit integers (the integer tensor-core matvecs) ----
// A group of activations (16 or 32 of them) becomes integers in [-32512, 32512] with one f32 scale: x ~ s * q.
// The largest magnitude of the group is found on the BIT PATTERNS of |x| (for non-negative floats the integer
// order is the float order), because that order also ranks +inf and every NaN above all finite values, whereas
// fmaxf() drops NaNs: a group that holds a NaN or an infinity gets s = NaN and q = 0, so every output that
// reads the group becomes NaN, as the reference's f32 dot product would make it non-finite
// (src/core/ref/ops.cpp:968-980).  Groups below 1e-30 count as zero (their products are below 1e-28 of a weight).
__device__ __forceinline__ uint32_t act_abs_bits(const float4 & v) {
    const uint32_t a = __float_as_uint(v.x) & 0x7fffffffu, b = __float_as_uint(v.y) & 0x7fffffffu;
    const uint32_t c = __float_as_uint(v.z) & 0x7fffffffu, d = __float_as_uint(v.w) & 0x7fffffffu;
    return max(max(a, b), max(c, d));
}
// inv: multiplier that maps the group's values to the integer range (0 for an empty or poisoned group);
// s: the scale that maps the integers back
__device__ __forceinline__ void act_group_scale(uint32_t amax_bits, float & inv, float & s) {
    const float amax = __uint_as_float(amax_bits);
    const bool finite = amax_bits < 0x7f800000u;
    const bool some = finite && amax > 1e-30f;
    // the fast division is exact enough here (the integer range keeps 255 counts of head room) but returns 0 for a
    // divisor above 2^126: such groups are scaled down first
    inv = !some ? 0.0f : (amax > 1e30f ? __fdividef(32512.0f * 0x1p-40f, amax * 0x1p-40f) : __fdividef(32512.0f, amax));
    s = some ? amax * (1.0f / 32512.0f) : 0.0f;
    if (!finite) s = __uint_as_float(0x7fc00000u);
}

// One thread's share of an arg-max scan over x[0..n) by a CTA of `threads` threads: the largest value and its index, the
// lowest index on ties (every thread meets its elements in increasing index order; the caller's reduction compares indices).
// The loads go out in batches of eight 16-byte requests per thread: a scalar loop with the compare in it is bound by one L2
// round trip per element and thread (27 us for a 151 936-entry row from one CTA, against about 6 us this way).
__device__ __forceinline__ void argmax_scan(const float * x, int64_t n, int tid, int threads, float & best, int & bi) {
    best = -INFINITY;
    bi = 0x7fffffff;
    auto take = [&](float v, int64_t i) {
        if (v > best || bi == 0x7fffffff) { best = v; bi = (int) i; }
    };
    int64_t done = 0;
    if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        constexpr int U = 8;
        const int64_t n4 = n >> 2;
        const float4 * x4 = reinterpret_cast<const float4 *>(x);
        for (int64_t base = tid; base < n4; base += (int64_t) threads * U) {
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t i = base + (int64_t) u * threads;
                v[u] = i < n4 ? __ldcg(x4 + i) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t i = base + (int64_t) u * threads;
                if (i < n4) {
                    take(v[u].x, 4 * i);
                    take(v[u].y, 4 * i + 1);
                    take(v[u].z, 4 * i + 2);
                    take(v[u].w, 4 * i + 3);
                }
            }
        }
        done = n4 << 2;
    }
    for (int64_t i = done + tid; i < n; i += threads) take(x[i], i);
}

// device side of programmatic dependent launch
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

}  // namespace sm100
