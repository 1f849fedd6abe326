// One-shot all-reduce (sum) of a short f32 vector over the GPUs of one node, through peer-mapped memory.
//
// The tensor-parallel decode needs two all-reduces of the hidden vector (16 KiB) per layer.  At that size a
// collective is pure latency, so it is one kernel of one CTA per GPU instead of a library call: every rank stores
// its vector into its slot of EVERY rank's receive area (plain 8-byte stores over NVLink: a value and the step number
// as its tag in one word, so that neither a fence nor a flag is needed - the scheme of NCCL's low-latency protocol),
// then adds the slots in rank order (the same order everywhere: every rank gets the same bits), waiting - with a
// bound - for each value's tag.  No multicast, no loads from peer memory, no library kernel on peer pointers.
//
// Two receive areas alternate by step: a rank can only be one step ahead of the slowest one (it needs that rank's
// values to finish a step), and a rank sends its values for step s + 1 only after it has finished reading step s.
//
// This replaces the host-bounce copy the reference uses between devices (src/core/transport.cpp:53-146) on the
// tensor-parallel path; the reference itself has no collective.
#include "sm100_common.cuh"

#include <cstring>

namespace sm100 {

namespace {

constexpr int AR_THREADS = 1024;

struct ArArgs {
    uint2 * recv[AR_MAX_RANKS];       // every rank's receive area [2][world][capacity] of (value bits, step tag) (entry `rank` is the local one)
    uint32_t * counter;               // local: calls so far
    int * fault;                      // local: set when a wait ran out
    float * x;                        // in / out
    int n, capacity, rank, world;
    uint32_t wait_limit;              // polls before the wait for a peer gives up
};

__global__ void __launch_bounds__(AR_THREADS, 1) allreduce_kernel(ArArgs a) {
    pdl_wait();
    const int tid = threadIdx.x;
    const uint32_t step = __ldcg(a.counter) + 1u;   // every thread reads it; thread 0 advances it at the end
    const size_t buf = (size_t) (step & 1u) * a.world;
    // 1. my vector into my slot of every rank's receive area, every value in one 8-byte word with the step as its tag
    for (int i = tid; i < a.n; i += AR_THREADS) {
        const uint32_t bits = __float_as_uint(a.x[i]);
        for (int p = 0; p < a.world; ++p) {
            uint2 * dst = a.recv[p] + (buf + a.rank) * a.capacity + i;
            asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(bits), "r"(step) : "memory");
        }
    }
    pdl_launch_dependents();
    // 2. sum of the slots in rank order; a value is there when its tag equals this step (bounded wait)
    const uint2 * mine = a.recv[a.rank] + buf * a.capacity;
    uint32_t limit = a.wait_limit;   // a thread waits out the bound once at most: after a give-up it only looks
    for (int i = tid; i < a.n; i += AR_THREADS) {
        float acc = 0.f;
        for (int r = 0; r < a.world; ++r) {
            const uint2 * src = mine + (size_t) r * a.capacity + i;
            uint2 got;
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(got.x), "=r"(got.y) : "l"(src) : "memory");
            for (uint32_t spins = 0; got.y != step && spins < limit; ++spins) {
                if (spins > 32) __nanosleep(50);
                asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(got.x), "=r"(got.y) : "l"(src) : "memory");
            }
            if (got.y != step) {
                atomicExch(a.fault, 1 + r);
                limit = 0;
            }
            acc = r == 0 ? __uint_as_float(got.x) : __fadd_rn(acc, __uint_as_float(got.x));
        }
        a.x[i] = acc;
    }
    __syncthreads();
    if (tid == 0) *a.counter = step;
}

// Greedy token over a row-sharded vocabulary head: every rank's best (logit, global index) goes to every rank as two
// 8-byte words tagged with the call number (the scheme of the fused matvec exchange), and every rank picks the winner:
// highest logit, lowest index on ties - the rule of TOP_K with k = 1 (src/core/ref/ops.cpp:1189-1228) over the whole row.
struct AmArgs {
    uint2 * slots[AR_MAX_RANKS];   // every rank's candidate slots [2][world][2 words] (entry `rank` is the local one)
    uint32_t * step;               // local: calls completed so far
    int * fault;
    const float * x;               // this rank's logits (n of them, n may be 0)
    int64_t n, index_offset;       // global index of x[0]
    int32_t * out;                 // the winning global index
    int rank, world;
    uint32_t wait_limit;
};

__global__ void __launch_bounds__(1024) argmax_allreduce_kernel(AmArgs a) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float sv[32];
    __shared__ int si[32];
    float best;
    int bi;
    argmax_scan(a.x, a.n, (int) threadIdx.x, (int) blockDim.x, best, bi);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x >= 32) return;
    const int nw = blockDim.x >> 5;
    best = (int) threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
    bi = (int) threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    // every lane holds this rank's candidate; lane r hands it to rank r and then collects rank r's
    const uint32_t step = *a.step + 1u;
    const int lane = threadIdx.x;
    const uint32_t gidx = bi == 0x7fffffff ? 0x7fffffffu : (uint32_t) (a.index_offset + bi);
    if (lane < a.world) {
        uint2 * dst = a.slots[lane] + ((size_t) (step & 1u) * a.world + a.rank) * 2;
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(best)), "r"(step) : "memory");
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst + 1), "r"(gidx), "r"(step) : "memory");
    }
    float cv = -INFINITY;
    uint32_t ci = 0x7fffffffu;
    if (lane < a.world) {
        const uint2 * src = a.slots[a.rank] + ((size_t) (step & 1u) * a.world + lane) * 2;
        uint2 w0 = make_uint2(0u, 0u), w1 = make_uint2(0u, 0u);
        bool ok = false;
        for (uint32_t i = 0; i < a.wait_limit && !ok; ++i) {
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(w0.x), "=r"(w0.y) : "l"(src) : "memory");
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(w1.x), "=r"(w1.y) : "l"(src + 1) : "memory");
            ok = w0.y == step && w1.y == step;
            if (!ok && i > 32) __nanosleep(50);
        }
        if (!ok) atomicExch(a.fault, 200 + lane);
        else { cv = __uint_as_float(w0.x); ci = w1.x; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, cv, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, ci, o);
        if (ov > cv || (ov == cv && oi < ci)) { cv = ov; ci = oi; }
    }
    if (lane == 0) {
        a.out[0] = (int32_t) ci;
        *a.step = step;
    }
}

struct ArContext {
    ArArgs args;
    ArFuse fuse;
    AmArgs argmax;
    int device;
};

}  // namespace

bool allreduce_fuse_args(void * ctx, ArFuse * out) {
    if (ctx == nullptr) return false;
    *out = static_cast<ArContext *>(ctx)->fuse;
    return true;
}

}  // namespace sm100

using namespace sm100;

extern "C" {

size_t sm100_ipc_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

int sm100_ipc_export(void * device_ptr, void * handle_out) {
    if (device_ptr == nullptr || handle_out == nullptr) return fail(ST_INVALID, "ipc_export: null pointer");
    cudaIpcMemHandle_t h;
    SM100_CUDA(cudaIpcGetMemHandle(&h, device_ptr));
    memcpy(handle_out, &h, sizeof(h));
    return ST_OK;
}

int sm100_ipc_open(const void * handle, void ** device_ptr_out) {
    if (handle == nullptr || device_ptr_out == nullptr) return fail(ST_INVALID, "ipc_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    SM100_CUDA(cudaIpcOpenMemHandle(device_ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
    return ST_OK;
}

int sm100_ipc_close(void * device_ptr) {
    if (device_ptr == nullptr) return ST_OK;
    SM100_CUDA(cudaIpcCloseMemHandle(device_ptr));
    return ST_OK;
}

// area of one rank: [receive slots of sm100_allreduce_sum: 8 bytes per value][256 B unused][counter, fault 256 B]
//                   [receive slots of the fused matvec exchange: 8 bytes per value][its step counter and ticket 256 B]
//                   [candidate slots and call counter of the greedy merge 512 B]
size_t sm100_allreduce_area_bytes(int world, int capacity) {
    const size_t data = (size_t) 2 * world * capacity * sizeof(float);
    return 2 * data + 256 + 256 + 2 * data + 256 + 512 /* candidate slots of the greedy merge [2][8][2 words], its call counter */;
}

int sm100_allreduce_create(int rank, int world, int capacity, void * const * areas, sm100_allreduce_t * out) {
    if (out == nullptr || areas == nullptr) return fail(ST_INVALID, "allreduce_create: null pointer");
    if (world < 1 || world > AR_MAX_RANKS || rank < 0 || rank >= world) return fail(ST_INVALID, "allreduce_create: 1..8 ranks");
    if (capacity <= 0 || capacity % 4 != 0) return fail(ST_INVALID, "allreduce_create: the capacity must be a positive multiple of 4 floats");
    ArContext * c = new ArContext();
    SM100_CUDA(cudaGetDevice(&c->device));
    const size_t data = (size_t) 2 * world * capacity * sizeof(float);
    for (int p = 0; p < world; ++p) {
        if (areas[p] == nullptr) { delete c; return fail(ST_INVALID, "allreduce_create: area %d is null", p); }
        c->args.recv[p] = (uint2 *) areas[p];
    }
    c->args.counter = (uint32_t *) ((uint8_t *) areas[rank] + 2 * data + 256);
    c->args.fault = (int *) ((uint8_t *) areas[rank] + 2 * data + 256 + 64);
    const size_t fused = 2 * data + 512;
    for (int p = 0; p < world; ++p) c->fuse.recv[p] = (uint2 *) ((uint8_t *) areas[p] + fused);
    c->fuse.step = (uint32_t *) ((uint8_t *) areas[rank] + fused + 2 * data);
    c->fuse.done = c->fuse.step + 16;
    c->args.wait_limit = AR_WAIT_LIMIT;
    c->fuse.wait_limit = AR_WAIT_LIMIT;
    const size_t merge = fused + 2 * data + 256;
    for (int p = 0; p < world; ++p) c->argmax.slots[p] = (uint2 *) ((uint8_t *) areas[p] + merge);
    c->argmax.step = (uint32_t *) ((uint8_t *) areas[rank] + merge + 256);
    c->argmax.fault = c->args.fault;
    c->argmax.rank = rank;
    c->argmax.world = world;
    c->argmax.wait_limit = AR_WAIT_LIMIT;
    c->fuse.fault = c->args.fault;
    c->fuse.capacity = capacity;
    c->fuse.rank = rank;
    c->fuse.world = world;
    c->args.capacity = capacity;
    c->args.rank = rank;
    c->args.world = world;
    *out = c;
    return ST_OK;
}

int sm100_allreduce_sum(sm100_allreduce_t ctx, sm100_stream_t s, float * x, int n) {
    ArContext * c = (ArContext *) ctx;
    if (c == nullptr || x == nullptr) return fail(ST_INVALID, "allreduce_sum: null pointer");
    if (n <= 0 || n % 4 != 0 || n > c->args.capacity || ((uintptr_t) x & 15) != 0)
        return fail(ST_INVALID, "allreduce_sum: n must be a positive multiple of 4 within the capacity, x 16-byte aligned");
    ArArgs a = c->args;
    a.x = x;
    a.n = n;
    return launch(allreduce_kernel, dim3(1), dim3(AR_THREADS), 0, (cudaStream_t) s, a);
}

int sm100_argmax_allreduce(sm100_allreduce_t ctx, sm100_stream_t s, const float * x, int64_t n, int64_t index_offset, int32_t * out) {
    ArContext * c = (ArContext *) ctx;
    if (c == nullptr || out == nullptr || n < 0 || (n > 0 && x == nullptr) || index_offset < 0 || index_offset + n > 0x7ffffffe)
        return fail(ST_INVALID, "argmax_allreduce: null pointer or a shard outside the 31-bit index range");
    AmArgs a = c->argmax;
    a.x = x;
    a.n = n;
    a.index_offset = index_offset;
    a.out = out;
    return launch(argmax_allreduce_kernel, dim3(1), dim3(1024), 0, (cudaStream_t) s, a);
}

int sm100_allreduce_set_wait_limit(sm100_allreduce_t ctx, uint32_t polls) {
    ArContext * c = (ArContext *) ctx;
    if (c == nullptr || polls == 0) return fail(ST_INVALID, "allreduce_set_wait_limit: null context or zero polls");
    c->args.wait_limit = polls;
    c->fuse.wait_limit = polls;
    c->argmax.wait_limit = polls;
    return ST_OK;
}

int sm100_allreduce_fault(sm100_allreduce_t ctx, int * fault_out) {
    ArContext * c = (ArContext *) ctx;
    if (c == nullptr || fault_out == nullptr) return fail(ST_INVALID, "allreduce_fault: null pointer");
    SM100_CUDA(cudaMemcpy(fault_out, c->args.fault, sizeof(int), cudaMemcpyDeviceToHost));
    return ST_OK;
}

int sm100_allreduce_destroy(sm100_allreduce_t ctx) {
    delete (ArContext *) ctx;
    return ST_OK;
}

}  // extern "C"
