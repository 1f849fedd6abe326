// MUL_MAT for callers whose activations and results live in HOST memory (the reference's usage through
// scrapgpu_tensor_upload -> op_execute -> scrapgpu_tensor_download, include/scrapgpu/tensor.h:45-53), as one call
// per product and without a host synchronisation in between.
//
// A pipe owns three in-order streams and a ring of `depth` slots (device x, device y, three events).  Call i takes
// slot i % depth:  copy stream   x host -> device           (after the slot's previous result has left)
//                  kernel stream sm100_mul_mat              (after the copy)
//                  result stream y device -> host           (after the kernel)
// so the copy of product i + 1 and the read-back of product i - 1 run beside the kernel of product i.  The host
// buffers must stay untouched until sm100_hostpipe_sync returns; pinned buffers (sm100_host_alloc) are needed for
// the copies to overlap.  Weights are device-resident, as after a tensor upload.
#include "sm100_common.cuh"
#include "scrapgpu_sm100.h"

#include <new>
#include <vector>

namespace sm100 {

namespace {

struct HostPipeSlot {
    float * x = nullptr;
    float * y = nullptr;
    cudaEvent_t in = nullptr, mm = nullptr, out = nullptr;
    bool used = false;
};

struct HostPipe {
    int device = 0;
    size_t x_bytes = 0, y_bytes = 0;
    cudaStream_t s_in = nullptr, s_mm = nullptr, s_out = nullptr;
    std::vector<HostPipeSlot> slots;
    size_t next = 0;
};

int pipe_free(HostPipe * p) {
    if (p == nullptr) return ST_OK;
    cudaSetDevice(p->device);
    for (HostPipeSlot & sl : p->slots) {
        if (sl.x != nullptr) cudaFree(sl.x);
        if (sl.y != nullptr) cudaFree(sl.y);
        if (sl.in != nullptr) cudaEventDestroy(sl.in);
        if (sl.mm != nullptr) cudaEventDestroy(sl.mm);
        if (sl.out != nullptr) cudaEventDestroy(sl.out);
    }
    if (p->s_in != nullptr) cudaStreamDestroy(p->s_in);
    if (p->s_mm != nullptr) cudaStreamDestroy(p->s_mm);
    if (p->s_out != nullptr) cudaStreamDestroy(p->s_out);
    delete p;
    return ST_OK;
}

int pipe_build(HostPipe * p, int depth) {
    SM100_CUDA(cudaSetDevice(p->device));
    SM100_CUDA(cudaStreamCreateWithFlags(&p->s_in, cudaStreamNonBlocking));
    SM100_CUDA(cudaStreamCreateWithFlags(&p->s_mm, cudaStreamNonBlocking));
    SM100_CUDA(cudaStreamCreateWithFlags(&p->s_out, cudaStreamNonBlocking));
    p->slots.resize((size_t) depth);
    for (HostPipeSlot & sl : p->slots) {
        SM100_CUDA(cudaMalloc((void **) &sl.x, p->x_bytes));
        SM100_CUDA(cudaMalloc((void **) &sl.y, p->y_bytes));
        SM100_CUDA(cudaEventCreateWithFlags(&sl.in, cudaEventDisableTiming));
        SM100_CUDA(cudaEventCreateWithFlags(&sl.mm, cudaEventDisableTiming));
        SM100_CUDA(cudaEventCreateWithFlags(&sl.out, cudaEventDisableTiming));
    }
    return ST_OK;
}

}  // namespace
}  // namespace sm100

using namespace sm100;

extern "C" int sm100_hostpipe_create(int device, int depth, size_t max_x_bytes, size_t max_y_bytes, sm100_hostpipe_t * out) {
    if (out == nullptr) return fail(ST_INVALID, "hostpipe_create: null result pointer");
    *out = nullptr;
    if (depth < 2 || depth > 4096) return fail(ST_INVALID, "hostpipe_create: depth %d outside 2..4096", depth);
    if (max_x_bytes == 0 || max_y_bytes == 0) return fail(ST_INVALID, "hostpipe_create: zero buffer size");
    HostPipe * p = new (std::nothrow) HostPipe();
    if (p == nullptr) return fail(ST_BACKEND, "hostpipe_create: out of host memory");
    p->device = device;
    p->x_bytes = (max_x_bytes + 255) / 256 * 256;
    p->y_bytes = (max_y_bytes + 255) / 256 * 256;
    const int st = pipe_build(p, depth);
    if (st != ST_OK) {
        pipe_free(p);
        return st;
    }
    *out = reinterpret_cast<sm100_hostpipe_t>(p);
    return ST_OK;
}

extern "C" int sm100_hostpipe_destroy(sm100_hostpipe_t pipe) { return pipe_free(reinterpret_cast<HostPipe *>(pipe)); }

extern "C" int sm100_hostpipe_stream(sm100_hostpipe_t pipe, int which, sm100_stream_t * out) {
    HostPipe * p = reinterpret_cast<HostPipe *>(pipe);
    if (p == nullptr || out == nullptr || which < 0 || which > 2) return fail(ST_INVALID, "hostpipe_stream: bad argument");
    *out = (sm100_stream_t) (which == 0 ? p->s_in : which == 1 ? p->s_mm : p->s_out);
    return ST_OK;
}

extern "C" int sm100_hostpipe_mul_mat(sm100_hostpipe_t pipe, int dtype, int layout, const void * w, int64_t w_row_stride, int64_t k, int64_t n,
                                      const float * host_x, int64_t m, float * host_y) {
    HostPipe * p = reinterpret_cast<HostPipe *>(pipe);
    if (p == nullptr || w == nullptr || host_x == nullptr || host_y == nullptr) return fail(ST_INVALID, "hostpipe_mul_mat: null pointer");
    if (k <= 0 || n <= 0 || m <= 0) return fail(ST_INVALID, "hostpipe_mul_mat: dimensions must be positive");
    const size_t xb = (size_t) k * (size_t) m * sizeof(float), yb = (size_t) n * (size_t) m * sizeof(float);
    if (xb > p->x_bytes || yb > p->y_bytes)
        return fail(ST_INVALID, "hostpipe_mul_mat: %zu / %zu bytes of activations / results exceed the pipe's %zu / %zu", xb, yb, p->x_bytes,
                    p->y_bytes);
    SM100_CUDA(cudaSetDevice(p->device));
    HostPipeSlot & sl = p->slots[p->next];
    p->next = (p->next + 1) % p->slots.size();
    // the slot's buffers are free once its previous result has been read back (which implies its kernel is done)
    if (sl.used) SM100_CUDA(cudaStreamWaitEvent(p->s_in, sl.out, 0));
    SM100_CUDA(cudaMemcpyAsync(sl.x, host_x, xb, cudaMemcpyHostToDevice, p->s_in));
    SM100_CUDA(cudaEventRecord(sl.in, p->s_in));
    SM100_CUDA(cudaStreamWaitEvent(p->s_mm, sl.in, 0));
    const int st = sm100_mul_mat((sm100_stream_t) p->s_mm, dtype, layout, w, w_row_stride, k, n, sl.x, k, m, sl.y, n);
    if (st != ST_OK) return st;
    SM100_CUDA(cudaEventRecord(sl.mm, p->s_mm));
    SM100_CUDA(cudaStreamWaitEvent(p->s_out, sl.mm, 0));
    SM100_CUDA(cudaMemcpyAsync(host_y, sl.y, yb, cudaMemcpyDeviceToHost, p->s_out));
    SM100_CUDA(cudaEventRecord(sl.out, p->s_out));
    sl.used = true;
    return ST_OK;
}

extern "C" int sm100_hostpipe_mul_mat_many(sm100_hostpipe_t pipe, int count, const sm100_hostpipe_item * items) {
    if (count < 0 || (count > 0 && items == nullptr)) return fail(ST_INVALID, "hostpipe_mul_mat_many: bad item list");
    for (int i = 0; i < count; ++i) {
        const sm100_hostpipe_item & it = items[i];
        const int st = sm100_hostpipe_mul_mat(pipe, it.dtype, it.layout, it.w, it.w_row_stride, it.k, it.n, it.host_x, it.m, it.host_y);
        if (st != ST_OK) return st;
    }
    return ST_OK;
}

extern "C" int sm100_hostpipe_sync(sm100_hostpipe_t pipe) {
    HostPipe * p = reinterpret_cast<HostPipe *>(pipe);
    if (p == nullptr) return fail(ST_INVALID, "hostpipe_sync: null pipe");
    SM100_CUDA(cudaSetDevice(p->device));
    SM100_CUDA(cudaStreamSynchronize(p->s_out));
    SM100_CUDA(cudaStreamSynchronize(p->s_in));
    // the kernel stream goes through the library's own synchronisation, which also reports a kernel's fault flag
    return sm100_stream_sync((sm100_stream_t) p->s_mm);
}
