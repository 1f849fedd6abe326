// Devices, memory, streams, events and graph replay for libscrapgpu_sm100 (the part of the backend
// vtable that is not arithmetic: include/scrapgpu/backend.h:33-44 of the reference).
#include "sm100_common.cuh"

#include <atomic>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

namespace sm100 {

static thread_local std::string t_error;
static std::atomic<uint64_t> g_launches{0};
static std::atomic<int> g_pdl{1};

int fail(int status, const char * fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    t_error = buf;
    return status;
}

int cuda_fail(cudaError_t e, const char * what) {
    const int st = e == cudaErrorMemoryAllocation ? ST_OOM : ST_BACKEND;
    return fail(st, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

static thread_local int t_serialized = 0;

static thread_local int t_serialized_inner = 0;   // the library's own bracket, independent of the caller's
void thread_serialized(bool on) { t_serialized_inner = on ? 1 : 0; }

// kind of the last launch per stream (stream handle + 8 with the kind in the low bits; the legacy stream 0 can so be
// told from an empty slot); a handful of slots serves the few streams a process drives at a time, a lost entry only
// costs speed
static std::atomic<uintptr_t> g_tail[8];
void stream_tail_set(cudaStream_t stream, int kind) {
    const uintptr_t key = ((uintptr_t) stream + 8) & ~(uintptr_t) 7;
    for (auto & slot : g_tail) {
        if ((slot.load(std::memory_order_relaxed) & ~(uintptr_t) 7) != key) continue;
        slot.store(kind == TAIL_OTHER ? 0 : key | (uintptr_t) kind, std::memory_order_relaxed);
        return;
    }
    if (kind == TAIL_OTHER) return;
    for (auto & slot : g_tail) {
        uintptr_t empty = 0;
        if (slot.compare_exchange_strong(empty, key | (uintptr_t) kind, std::memory_order_relaxed)) return;
    }
    g_tail[(key >> 6) % 8].store(key | (uintptr_t) kind, std::memory_order_relaxed);
}
int stream_tail(cudaStream_t stream) {
    const uintptr_t key = ((uintptr_t) stream + 8) & ~(uintptr_t) 7;
    for (auto & slot : g_tail) {
        const uintptr_t v = slot.load(std::memory_order_relaxed);
        if ((v & ~(uintptr_t) 7) == key) return (int) (v & 7);
    }
    return TAIL_OTHER;
}
bool pdl_enabled() { return t_serialized == 0 && t_serialized_inner == 0 && g_pdl.load(std::memory_order_relaxed) != 0; }
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { (void) cudaGetLastError(); return 0; }
    return dev < 0 || dev >= MAX_DEVICES ? 0 : dev;
}

int sm_count() {
    static std::mutex mu;
    static std::vector<int> cache;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if ((int) cache.size() <= dev) cache.resize(dev + 1, 0);
    if (cache[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cache[dev] = n;
    }
    return cache[dev];
}

// Per-device scratch owned by the library, one buffer per slot (0 = attention partials, 1 = GEMM
// activations, 2 = quantized activation columns of the multi-column matvec), grown on demand.  A buffer that was
// handed out once is NEVER freed or moved: a CUDA graph captured earlier has its address baked into its kernel
// nodes and may be replayed at any time.  Growing therefore allocates a second, larger block (at least twice the
// old size, so the blocks left behind add up to less than the live one) and later calls use that; replays of older
// graphs keep working on the block they were captured with.  Calls that use the same slot must be ordered on one
// stream.  Allocation cannot happen while a stream is capturing: the first call of a shape (or sm100_scratch_reserve)
// has to come before the capture.
int device_scratch(int slot, size_t bytes, void ** out) {
    constexpr int SLOTS = 3;
    struct Entry { void * ptr[SLOTS] = {nullptr, nullptr, nullptr}; size_t size[SLOTS] = {0, 0, 0}; std::vector<void *> retired; };
    static std::mutex mu;
    static std::vector<Entry> table;
    if (slot < 0 || slot >= SLOTS) return fail(ST_INVALID, "device_scratch: bad slot");
    int dev = 0;
    SM100_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    if ((int) table.size() <= dev) table.resize(dev + 1);
    Entry & e = table[dev];
    if (e.size[slot] < bytes) {
        size_t want = bytes < (size_t) (8u << 20) ? (size_t) (8u << 20) : bytes;
        if (want < 2 * e.size[slot]) want = 2 * e.size[slot];
        void * fresh = nullptr;
        const cudaError_t me = cudaMalloc(&fresh, want);
        if (me == cudaErrorStreamCaptureUnsupported || me == cudaErrorStreamCaptureInvalidated) {
            (void) cudaGetLastError();
            return fail(ST_BACKEND, "the library's scratch buffer for this op does not exist yet (or is too small) and cannot be allocated while a "
                                    "stream is capturing: issue the same call once outside the capture first");
        }
        if (me != cudaSuccess) return cuda_fail(me, "cudaMalloc(scratch)");
        SM100_CUDA(cudaMemset(fresh, 0, want));   // the attention kernels keep counters in it that start at zero
        if (e.ptr[slot] != nullptr) e.retired.push_back(e.ptr[slot]);   // stays allocated: earlier graphs may still name it
        e.ptr[slot] = fresh;
        e.size[slot] = want;
    }
    *out = e.ptr[slot];
    return ST_OK;
}

int gemm_poll_fault();
int iq_poll_fault();

// Waits for the stream, then reads the fault words of the kernels with bounded waits on the STREAM's device (they are
// per-device variables; the current device may be another one in a process that drives several GPUs).
static int sync_and_poll(cudaStream_t st) {
    SM100_CUDA(cudaStreamSynchronize(st));
    int cur = 0, dev = 0;
    SM100_CUDA(cudaGetDevice(&cur));
    dev = cur;
    if (st != nullptr && cudaStreamGetDevice(st, &dev) != cudaSuccess) {
        (void) cudaGetLastError();
        dev = cur;
    }
    if (dev != cur) SM100_CUDA(cudaSetDevice(dev));
    int r = gemm_poll_fault();
    if (r == ST_OK) r = iq_poll_fault();
    if (dev != cur) (void) cudaSetDevice(cur);
    return r;
}

}  // namespace sm100

using namespace sm100;

extern "C" {

const char * sm100_last_error(void) { return t_error.c_str(); }

int sm100_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int sm100_device_info(int device, char * name, size_t name_size, uint64_t * total_memory, uint32_t * sms,
                      uint32_t * cc_major, uint32_t * cc_minor, uint64_t * shared_per_block) {
    cudaDeviceProp p;
    SM100_CUDA(cudaGetDeviceProperties(&p, device));
    if (name != nullptr && name_size > 0) {
        std::strncpy(name, p.name, name_size - 1);
        name[name_size - 1] = '\0';
    }
    if (total_memory) *total_memory = p.totalGlobalMem;
    if (sms) *sms = (uint32_t) p.multiProcessorCount;
    if (cc_major) *cc_major = (uint32_t) p.major;
    if (cc_minor) *cc_minor = (uint32_t) p.minor;
    if (shared_per_block) *shared_per_block = p.sharedMemPerBlockOptin;
    return ST_OK;
}

int sm100_set_device(int device) {
    SM100_CUDA(cudaSetDevice(device));
    return ST_OK;
}

int sm100_malloc(int device, size_t size, void ** out) {
    if (out == nullptr || size == 0) return fail(ST_INVALID, "sm100_malloc: out is null or size is 0");
    *out = nullptr;
    SM100_CUDA(cudaSetDevice(device));
    SM100_CUDA(cudaMalloc(out, size));  // cudaMalloc returns at least 256-byte aligned memory
    return ST_OK;
}

int sm100_free(int device, void * ptr) {
    if (ptr == nullptr) return ST_OK;
    SM100_CUDA(cudaSetDevice(device));
    SM100_CUDA(cudaFree(ptr));
    return ST_OK;
}

int sm100_host_alloc(size_t size, void ** out) {
    if (out == nullptr || size == 0) return fail(ST_INVALID, "sm100_host_alloc: out is null or size is 0");
    SM100_CUDA(cudaHostAlloc(out, size, cudaHostAllocPortable));
    return ST_OK;
}

int sm100_host_free(void * ptr) {
    if (ptr != nullptr) SM100_CUDA(cudaFreeHost(ptr));
    return ST_OK;
}

int sm100_stream_create(int device, sm100_stream_t * out) {
    if (out == nullptr) return fail(ST_INVALID, "sm100_stream_create: out is null");
    SM100_CUDA(cudaSetDevice(device));
    cudaStream_t s = nullptr;
    SM100_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *out = s;
    return ST_OK;
}

int sm100_stream_destroy(int device, sm100_stream_t stream) {
    if (stream == nullptr) return ST_OK;
    SM100_CUDA(cudaSetDevice(device));
    stream_tail_set((cudaStream_t) stream, TAIL_OTHER);   // a later stream may get the same handle
    SM100_CUDA(cudaStreamDestroy((cudaStream_t) stream));
    return ST_OK;
}

int sm100_stream_sync(sm100_stream_t stream) { return sync_and_poll((cudaStream_t) stream); }

int sm100_memcpy_h2d(sm100_stream_t s, void * dst, const void * src, size_t n, int blocking) {
    if (n == 0) return ST_OK;
    stream_tail_set((cudaStream_t) s, TAIL_OTHER);
    SM100_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, (cudaStream_t) s));
    if (blocking) SM100_CUDA(cudaStreamSynchronize((cudaStream_t) s));
    return ST_OK;
}

int sm100_memcpy_d2h(sm100_stream_t s, void * dst, const void * src, size_t n, int blocking) {
    if (n == 0) return ST_OK;
    stream_tail_set((cudaStream_t) s, TAIL_OTHER);
    SM100_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToHost, (cudaStream_t) s));
    // a blocking read makes results visible like a stream_sync does (include/scrapgpu/op.h:190-194), so a kernel that
    // gave up on a bounded wait is reported here too instead of handing out an incomplete result with status OK
    if (blocking) return sync_and_poll((cudaStream_t) s);
    return ST_OK;
}

int sm100_memcpy_d2d(sm100_stream_t s, void * dst, const void * src, size_t n, int blocking) {
    if (n == 0) return ST_OK;
    stream_tail_set((cudaStream_t) s, TAIL_OTHER);
    // overlapping ranges get memmove semantics through a stream-ordered temporary
    const char * a = (const char *) src;
    char * b = (char *) dst;
    if (a == b) return ST_OK;
    if ((b > a && b < a + n) || (a > b && a < b + n)) {
        void * tmp = nullptr;
        SM100_CUDA(cudaMallocAsync(&tmp, n, (cudaStream_t) s));
        cudaError_t e = cudaMemcpyAsync(tmp, src, n, cudaMemcpyDeviceToDevice, (cudaStream_t) s);
        if (e == cudaSuccess) e = cudaMemcpyAsync(dst, tmp, n, cudaMemcpyDeviceToDevice, (cudaStream_t) s);
        cudaFreeAsync(tmp, (cudaStream_t) s);
        if (e != cudaSuccess) return cuda_fail(e, "sm100_memcpy_d2d");
    } else {
        SM100_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToDevice, (cudaStream_t) s));
    }
    if (blocking) SM100_CUDA(cudaStreamSynchronize((cudaStream_t) s));
    return ST_OK;
}

int sm100_memset(sm100_stream_t s, void * dst, int byte, size_t n, int blocking) {
    if (n == 0) return ST_OK;
    stream_tail_set((cudaStream_t) s, TAIL_OTHER);
    SM100_CUDA(cudaMemsetAsync(dst, byte, n, (cudaStream_t) s));
    if (blocking) SM100_CUDA(cudaStreamSynchronize((cudaStream_t) s));
    return ST_OK;
}

int sm100_memcpy_peer(sm100_stream_t dst_stream, int dst_device, void * dst, sm100_stream_t src_stream, int src_device,
                      const void * src, size_t n) {
    if (n == 0) return ST_OK;
    // order: after everything enqueued on src_stream, before later work on dst_stream
    cudaEvent_t ready = nullptr;
    SM100_CUDA(cudaSetDevice(src_device));
    SM100_CUDA(cudaEventCreateWithFlags(&ready, cudaEventDisableTiming));
    cudaError_t e = cudaEventRecord(ready, (cudaStream_t) src_stream);
    if (e == cudaSuccess) e = cudaSetDevice(dst_device);
    if (e == cudaSuccess) e = cudaStreamWaitEvent((cudaStream_t) dst_stream, ready, 0);
    if (e == cudaSuccess) e = cudaMemcpyPeerAsync(dst, dst_device, src, src_device, n, (cudaStream_t) dst_stream);
    cudaEventDestroy(ready);
    if (e != cudaSuccess) return cuda_fail(e, "sm100_memcpy_peer");
    return ST_OK;
}

int sm100_peer_access(int device, int peer) {
    if (device == peer) return ST_OK;
    int can = 0;
    SM100_CUDA(cudaDeviceCanAccessPeer(&can, device, peer));
    if (!can) return fail(ST_UNSUPPORTED, "device %d cannot map the memory of device %d", device, peer);
    int cur = 0;
    SM100_CUDA(cudaGetDevice(&cur));
    SM100_CUDA(cudaSetDevice(device));
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
    (void) cudaSetDevice(cur);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void) cudaGetLastError();
        return ST_OK;
    }
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceEnablePeerAccess");
    return ST_OK;
}

int sm100_event_create(sm100_event_t * out) {
    if (out == nullptr) return fail(ST_INVALID, "sm100_event_create: out is null");
    cudaEvent_t e = nullptr;
    SM100_CUDA(cudaEventCreate(&e));
    *out = e;
    return ST_OK;
}

int sm100_event_destroy(sm100_event_t e) {
    if (e != nullptr) SM100_CUDA(cudaEventDestroy((cudaEvent_t) e));
    return ST_OK;
}

int sm100_event_record(sm100_event_t e, sm100_stream_t s) {
    SM100_CUDA(cudaEventRecord((cudaEvent_t) e, (cudaStream_t) s));
    return ST_OK;
}

int sm100_stream_wait_event(sm100_stream_t s, sm100_event_t e) {
    SM100_CUDA(cudaStreamWaitEvent((cudaStream_t) s, (cudaEvent_t) e, 0));
    return ST_OK;
}

int sm100_event_sync(sm100_event_t e) {
    SM100_CUDA(cudaEventSynchronize((cudaEvent_t) e));
    return ST_OK;
}

int sm100_event_elapsed_ms(sm100_event_t start, sm100_event_t stop, float * ms) {
    SM100_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t) start, (cudaEvent_t) stop));
    return ST_OK;
}

int sm100_graph_begin(sm100_stream_t s) {
    SM100_CUDA(cudaStreamBeginCapture((cudaStream_t) s, cudaStreamCaptureModeThreadLocal));
    return ST_OK;
}

int sm100_graph_end(sm100_stream_t s, sm100_graph_t * out) {
    if (out == nullptr) return fail(ST_INVALID, "sm100_graph_end: out is null");
    cudaGraph_t g = nullptr;
    SM100_CUDA(cudaStreamEndCapture((cudaStream_t) s, &g));
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
    *out = exec;
    return ST_OK;
}

int sm100_graph_launch(sm100_graph_t g, sm100_stream_t s) {
    stream_tail_set((cudaStream_t) s, TAIL_OTHER);
    SM100_CUDA(cudaGraphLaunch((cudaGraphExec_t) g, (cudaStream_t) s));
    return ST_OK;
}

int sm100_graph_destroy(sm100_graph_t g) {
    if (g != nullptr) SM100_CUDA(cudaGraphExecDestroy((cudaGraphExec_t) g));
    return ST_OK;
}

uint64_t sm100_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int sm100_scratch_reserve(int slot, size_t bytes) {
    void * p = nullptr;
    return device_scratch(slot, bytes, &p);
}

int sm100_set_pdl(int enabled) {
    g_pdl.store(enabled ? 1 : 0, std::memory_order_relaxed);
    return ST_OK;
}

int sm100_launch_serialized(int on) {
    t_serialized = on ? 1 : 0;
    return ST_OK;
}

}  // extern "C"
