// The `cuda_sm100` backend of ScrapGpuLibrary: host layer between the library's backend vtable
// (include/scrapgpu/backend.h:29-57 of the reference) and the CUDA compute library libscrapgpu_sm100.so
// (include/scrapgpu_sm100.h).  C++17, no CUDA headers: every device action goes through that C ABI.
//
// Contract followed (where the reference states it):
//   - every object handed out starts with a scrapgpu_object_header pointing at this backend's static vtable
//     (backend.h:22-27); foreign or NULL objects are answered with INVALID_ARGUMENT, never dereferenced further
//     (tests/cpu/cpu_tests.cpp:279-338)
//   - ops are enqueued on the stream's CUDA stream; results are visible after stream_sync or a blocking read
//     (include/scrapgpu/op.h:190-194); failures of enqueued work surface at the next stream_sync
//   - tensor_upload / tensor_download move natural bytes; a tensor whose layout tag is SCRAPGPU_LAYOUT_R32 is
//     packed / unpacked on the way (include/scrapgpu/tensor.h:45-53); here the tag selects the B200 plane layout
//   - UNSUPPORTED always carries a reason (reason out-parameter and last error)
//   - no exception crosses the C ABI
//   - plans deep-copy their descriptors and pin the buffers they reference: buffer_free is refused while a plan
//     lives (docs/API_CONTRACT.md:43)
// There is no CPU fallback: an op this backend does not implement is reported UNSUPPORTED.
#include "scrapgpu/cuda_sm100.h"

#include "scrapgpu_sm100.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <new>
#include <string>
#include <tuple>
#include <unordered_map>
#include <vector>

// Symbols of the ScrapGpuLibrary core.  They are weak so that the plugin also loads stand-alone (its vtable can be
// driven directly); inside a ScrapGpuLibrary process they resolve to the core's definitions.
#pragma weak scrapgpu_register_backend
#pragma weak scrapgpu_op_desc_validate
#pragma weak scrapgpu_set_last_error
#pragma weak scrapgpu_last_error
#pragma weak scrapgpu_get_device_count
#pragma weak scrapgpu_get_device

namespace {

constexpr int kQ4_0 = SCRAPGPU_DTYPE_Q4_0, kQ8_0 = SCRAPGPU_DTYPE_Q8_0, kQ4_K = SCRAPGPU_DTYPE_Q4_K, kQ6_K = SCRAPGPU_DTYPE_Q6_K;

// ---------------------------------------------------------------------------------------------------------
// objects
// ---------------------------------------------------------------------------------------------------------

struct Device {
    scrapgpu_object_header hdr;  // first member
    int ordinal = 0;
    std::string name, driver;
    uint64_t total_memory = 0, shared_per_block = 0;
    uint32_t sms = 0, cc_major = 0, cc_minor = 0;
    // (cos, sin) tables of ROPE, keyed by the parameters that determine them; built on the host with the
    // reference's recipe so that the rotation is bit-identical to the CPU backend
    std::mutex rope_mutex;
    std::map<std::tuple<int, uint32_t, uint32_t, uint32_t>, std::pair<void *, int32_t>> rope_tables;
};

struct Stream;

struct Buffer {
    scrapgpu_object_header hdr;
    Device * dev = nullptr;
    void * ptr = nullptr;
    size_t size = 0;
    // the last kernel that wrote into the buffer: the stream it ran on and that stream's launch number (see fresh())
    std::atomic<const Stream *> writer{nullptr};
    std::atomic<uint64_t> written{0};
};

struct Stream {
    scrapgpu_object_header hdr;
    Device * dev = nullptr;
    sm100_stream_t cuda = nullptr;
    uint64_t epoch = 0;     // ops enqueued so far
    uint64_t settled = 0;   // ops up to this number have completed before anything enqueued from now on starts
    // per-op-key timing table (SCRAPGPU_SM100_PROFILE=1), the counterpart of the OpenCL backend's GGML_CL11_PROFILE table
    // (src/backends/opencl11/executor.h:41-112): a pair of events around every op, read back at stream_sync
    struct ProfStat { std::string name; double ms = 0; size_t count = 0; double bytes = 0; };
    struct ProfPending { sm100_event_t start, stop; int key; };
    std::vector<ProfStat> prof_stats;
    std::vector<ProfPending> prof_pending;
    std::vector<sm100_event_t> prof_spare;
    scrapgpu_status sticky = SCRAPGPU_STATUS_OK;  // failure of enqueued work, reported at the next sync
    std::string sticky_message;
};

struct PlanNode {
    scrapgpu_op_desc desc;
    std::vector<scrapgpu_tensor_desc> inputs, outputs;
    std::vector<uint8_t> params;
    uint32_t use_count = 0;   // consumers of the node's result as the caller counted them (backend.h:10-14); 0 = not stated
    // the pointers inside desc refer to this object's own vectors: keep them right when the object is copied or moved
    void rebind() {
        desc.struct_size = sizeof(desc);
        desc.inputs = inputs.data();
        desc.input_count = inputs.size();
        desc.outputs = outputs.data();
        desc.output_count = outputs.size();
        desc.params = params.empty() ? nullptr : params.data();
        desc.params_size = params.size();
    }
    PlanNode() { desc = {}; }
    PlanNode(const PlanNode & o) : desc(o.desc), inputs(o.inputs), outputs(o.outputs), params(o.params), use_count(o.use_count) { rebind(); }
    PlanNode & operator=(const PlanNode & o) {
        if (this != &o) { desc = o.desc; inputs = o.inputs; outputs = o.outputs; params = o.params; use_count = o.use_count; rebind(); }
        return *this;
    }
};

// One sm100_mul_mat_fused launch standing for a normalisation or activation node and the MUL_MAT(s) that consume it
struct FusedCall {
    int prologue = 0;   // SM100_PROLOGUE_RMS_NORM or SM100_PROLOGUE_SWIGLU
    scrapgpu_tensor_desc a = {}, b = {}, norm_w = {}, sum_out = {}, x_out = {};
    bool has_b = false, has_sum = false, has_x = false;
    float eps = 0.0f;
    std::vector<scrapgpu_tensor_desc> w, y;
    // the two tensors are the gate and up projections of a GLU node that follows: its output comes out of the same launch
    // (sm100_mul_mat_glu), y[0] and y[1] are written as well
    bool has_glu = false;
    scrapgpu_tensor_desc glu_out = {};
};

// What plan_execute runs in place of a group of consecutive nodes of the caller's list
struct PlanStep {
    std::vector<size_t> nodes;   // the caller's nodes this step stands for, in order
    int lowered = -1;            // a public fused op (Plan::lowered) that replaces them, or -1
    int fused = -1;              // a FusedCall (Plan::fused) that replaces them, or -1
    bool declined = false;       // the replacement was answered UNSUPPORTED when first run: the caller's nodes run instead
};

struct Plan {
    scrapgpu_object_header hdr;
    Device * dev = nullptr;
    std::vector<PlanNode> nodes;       // deep copy of the caller's list
    std::vector<PlanNode> lowered;     // fused ops found at build time
    std::vector<FusedCall> fused;
    std::vector<PlanStep> steps;
    std::vector<Buffer *> pinned;
    // replay: the steps are recorded once into a CUDA graph (the second execution; the first one runs them one by one
    // and lets the library create whatever scratch and tables they need), later executions launch the graph
    uint64_t executions = 0;
    sm100_graph_t graph = nullptr;
    bool graph_refused = false;
    size_t launches_per_execution = 0;
};

extern const scrapgpu_backend_vtable g_vtable;

std::mutex g_registry_mutex;
std::vector<std::unique_ptr<Device>> g_devices;
bool g_devices_probed = false;

std::mutex g_pin_mutex;
std::unordered_map<Buffer *, size_t> g_pins;  // live plans referencing each buffer

thread_local std::string t_local_error;  // used when the core is not loaded

// ---------------------------------------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------------------------------------

void set_error(const char * message) {
    if (scrapgpu_set_last_error != nullptr) scrapgpu_set_last_error(message);
    else t_local_error = message;
}

scrapgpu_status invalid(const char * message) {
    set_error(message);
    return SCRAPGPU_STATUS_INVALID_ARGUMENT;
}

scrapgpu_status unsupported(const char * message, const char ** reason = nullptr) {
    if (reason != nullptr) *reason = message;
    set_error(message);
    return SCRAPGPU_STATUS_UNSUPPORTED;
}

scrapgpu_status bad(const char * message, const char ** reason) {
    if (reason != nullptr) *reason = message;
    set_error(message);
    return SCRAPGPU_STATUS_INVALID_ARGUMENT;
}

// status of a libscrapgpu_sm100 call -> status of the vtable call (the codes are shared; the message is copied)
scrapgpu_status from_sm100(int st) {
    if (st == 0) return SCRAPGPU_STATUS_OK;
    const char * m = sm100_last_error();
    set_error(m != nullptr && *m != '\0' ? m : "cuda_sm100: device call failed");
    return st >= 1 && st <= 5 ? static_cast<scrapgpu_status>(st) : SCRAPGPU_STATUS_BACKEND_ERROR;
}

template <typename F>
scrapgpu_status guard(F && fn) noexcept {
    try {
        return fn();
    } catch (const std::bad_alloc &) {
        try { set_error("out of host memory"); } catch (...) {}
        return SCRAPGPU_STATUS_OUT_OF_MEMORY;
    } catch (...) {
        try { set_error("the cuda_sm100 backend threw an exception"); } catch (...) {}
        return SCRAPGPU_STATUS_BACKEND_ERROR;
    }
}

// ---------------------------------------------------------------------------------------------------------
// object checks
// ---------------------------------------------------------------------------------------------------------

template <typename T, typename H>
T * own(H * handle) {
    auto * o = reinterpret_cast<T *>(handle);
    return o != nullptr && o->hdr.backend == &g_vtable ? o : nullptr;
}

Device * as_device(scrapgpu_device_t * d) {
    Device * dev = own<Device>(d);
    if (dev == nullptr) return nullptr;
    for (const auto & known : g_devices) if (known.get() == dev) return dev;
    return nullptr;
}
Buffer * as_buffer(scrapgpu_buffer_t * b) { return own<Buffer>(b); }
Stream * as_stream(scrapgpu_stream_t * s) { return own<Stream>(s); }
Plan * as_plan(scrapgpu_plan_t * p) { return own<Plan>(p); }

// ---------------------------------------------------------------------------------------------------------
// descriptor math (the public definitions of include/scrapgpu/tensor.h; the core's sgt:: helpers are internal)
// ---------------------------------------------------------------------------------------------------------

size_t type_size(int dtype) {
    switch (dtype) {
        case SCRAPGPU_DTYPE_F32: case SCRAPGPU_DTYPE_I32: return 4;
        case SCRAPGPU_DTYPE_F16: case SCRAPGPU_DTYPE_I16: case SCRAPGPU_DTYPE_BF16: return 2;
        case SCRAPGPU_DTYPE_I64: return 8;
        case kQ4_0: return 18;
        case kQ8_0: return 34;
        case kQ4_K: return 144;
        case kQ6_K: return 210;
        default: return 0;
    }
}

size_t block_size(int dtype) {
    switch (dtype) {
        case kQ4_0: case kQ8_0: return 32;
        case kQ4_K: case kQ6_K: return 256;
        default: return type_size(dtype) != 0 ? 1 : 0;
    }
}

bool is_quant(int dtype) { return block_size(dtype) > 1; }

scrapgpu_tensor_desc load_desc(const scrapgpu_tensor_desc & in) {
    scrapgpu_tensor_desc out = {};
    if (in.struct_size >= sizeof(size_t)) {
        std::memcpy(&out, &in, std::min(in.struct_size, sizeof(out)));
        out.struct_size = sizeof(out);
    }
    return out;
}

int64_t ne(const scrapgpu_tensor_desc & t, int i) { return t.ne[i] > 0 ? t.ne[i] : 1; }

uint64_t sat_mul(uint64_t a, uint64_t b) { return a != 0 && b > UINT64_MAX / a ? UINT64_MAX : a * b; }
uint64_t sat_add(uint64_t a, uint64_t b) { return b > UINT64_MAX - a ? UINT64_MAX : a + b; }

// bytes from the tensor's first byte to one past its last (0 for an empty or unknown tensor)
uint64_t span_bytes(const scrapgpu_tensor_desc & t) {
    const size_t bs = block_size(t.dtype), ts = type_size(t.dtype);
    if (bs == 0 || ts == 0) return 0;
    for (int i = 0; i < 4; ++i) if (t.ne[i] <= 0) return 0;
    uint64_t n = bs == 1 ? ts : sat_mul((uint64_t) t.ne[0], t.nb[0]) / bs;
    for (int i = bs == 1 ? 0 : 1; i < 4; ++i) n = sat_add(n, sat_mul((uint64_t) (t.ne[i] - 1), t.nb[i]));
    return n;
}

bool span_ok(const scrapgpu_tensor_desc & t) {
    const uint64_t half = UINT64_MAX / 2;
    if (t.offset > half) return false;
    uint64_t span = t.offset;
    for (int i = 0; i < 4; ++i) {
        const uint64_t count = (uint64_t) (ne(t, i) - 1);
        if (t.nb[i] != 0 && count > (half - span) / t.nb[i]) return false;
        span += count * t.nb[i];
        if (span > half) return false;
    }
    return true;
}

// ggml contiguity: dims of size 1 (and nb[0] of a single-block row) are unconstrained
bool contiguous(const scrapgpu_tensor_desc & t) {
    const size_t bs = block_size(t.dtype), ts = type_size(t.dtype);
    if (bs == 0 || ts == 0) return false;
    uint64_t next = ts;
    if (t.ne[0] != (int64_t) bs && t.nb[0] != next) return false;
    next *= (uint64_t) (t.ne[0] / (int64_t) bs);
    for (int i = 1; i < 4; ++i) {
        if (t.ne[i] != 1 && t.nb[i] != next) return false;
        next = sat_mul(next, (uint64_t) t.ne[i]);
    }
    return next != UINT64_MAX;
}

bool same_shape(const scrapgpu_tensor_desc & a, const scrapgpu_tensor_desc & b) {
    for (int i = 0; i < 4; ++i) if (ne(a, i) != ne(b, i)) return false;
    return true;
}

bool elements(const scrapgpu_tensor_desc & t, int64_t & out) {
    int64_t n = 1;
    for (int i = 0; i < 4; ++i) {
        const int64_t d = ne(t, i);
        if (n > std::numeric_limits<int64_t>::max() / d) return false;
        n *= d;
    }
    out = n;
    return true;
}

template <typename T>
T load_params(const scrapgpu_op_desc * desc) {
    T p = {};
    if (desc->params != nullptr) std::memcpy(&p, desc->params, std::min(desc->params_size, sizeof(T)));
    return p;
}

template <typename E>
uint32_t enum_bits(const E & e) {
    uint32_t v = 0;
    std::memcpy(&v, &e, std::min(sizeof(e), sizeof(v)));
    return v;
}

// ---------------------------------------------------------------------------------------------------------
// op_supported: descriptor-only checks; the shape rules are the reference's (src/backends/cpu/api.cpp:394-830,
// src/core/ref/ops.cpp), the dtype / layout coverage is this backend's
// ---------------------------------------------------------------------------------------------------------

bool f32(const scrapgpu_tensor_desc & t) { return t.dtype == SCRAPGPU_DTYPE_F32; }

scrapgpu_status check_tensor_meta(const scrapgpu_tensor_desc & raw, bool weight_slot, const char ** reason) {
    const scrapgpu_tensor_desc t = load_desc(raw);
    if (type_size(t.dtype) == 0) return unsupported("unknown tensor dtype", reason);
    for (int i = 0; i < 4; ++i) if (t.ne[i] <= 0) return bad("non-positive tensor dim", reason);
    if (!span_ok(t)) return unsupported("tensor strides or offset overflow the address space", reason);
    if (t.layout != SCRAPGPU_LAYOUT_NATURAL) {
        if (t.layout != SCRAPGPU_LAYOUT_R32) return unsupported("unknown tensor layout", reason);
        if (!weight_slot || !is_quant(t.dtype)) return unsupported("only quantized weight tensors can use the backend-packed layout", reason);
        if (!contiguous(t) || ne(t, 2) * ne(t, 3) != 1) return unsupported("a backend-packed tensor must be a whole contiguous 2-D tensor (no views)", reason);
        if (t.ne[0] % (int64_t) block_size(t.dtype) != 0) return unsupported("quantized row length must be a multiple of the block size", reason);
        if (t.offset % 32 != 0) return unsupported("a backend-packed tensor must start on a 32-byte boundary of its buffer", reason);
    }
    return SCRAPGPU_STATUS_OK;
}

scrapgpu_status require_rows(const scrapgpu_tensor_desc & t, const char * what, const char ** reason) {
    if (t.nb[0] != type_size(t.dtype)) return unsupported(what, reason);
    if (is_quant(t.dtype) && t.ne[0] % (int64_t) block_size(t.dtype) != 0) return unsupported("quantized row length must be a multiple of the block size", reason);
    return SCRAPGPU_STATUS_OK;
}

bool mm_weight(int dtype) {
    return dtype == SCRAPGPU_DTYPE_F32 || dtype == SCRAPGPU_DTYPE_F16 || is_quant(dtype);
}

scrapgpu_status mul_mat_shapes(const scrapgpu_tensor_desc & w, const scrapgpu_tensor_desc & x, const scrapgpu_tensor_desc & d, int allow_broadcast,
                               const char ** reason) {
    if (!f32(x) || !f32(d)) return unsupported("MUL_MAT expects an F32 src1 and destination", reason);
    if (!mm_weight(w.dtype)) return unsupported("MUL_MAT weights must be F32, F16, Q4_0, Q8_0, Q4_K or Q6_K on cuda_sm100", reason);
    scrapgpu_status st = require_rows(w, "MUL_MAT needs contiguous rows of src0 (nb0 == element size)", reason);
    if (st != SCRAPGPU_STATUS_OK) return st;
    if (x.nb[0] != 4 || d.nb[0] != 4) return unsupported("MUL_MAT needs contiguous rows of src1 and dst (nb0 == element size)", reason);
    if (ne(w, 0) != ne(x, 0)) return bad("MUL_MAT: the inner dimensions of src0 and src1 differ", reason);
    if (ne(x, 2) % ne(w, 2) != 0 || ne(x, 3) % ne(w, 3) != 0) return bad("MUL_MAT: src1 dims 2 and 3 must be multiples of the src0 dims", reason);
    if (allow_broadcast == 0 && (ne(x, 2) != ne(w, 2) || ne(x, 3) != ne(w, 3))) return unsupported("MUL_MAT: broadcasting over dims 2/3 is not allowed", reason);
    if (ne(d, 0) != ne(w, 1) || ne(d, 1) != ne(x, 1) || ne(d, 2) != ne(x, 2) || ne(d, 3) != ne(x, 3)) return bad("MUL_MAT: dst must be [ne01, ne11, ne12, ne13]", reason);
    if (is_quant(w.dtype) && ((x.offset % 16) != 0 || (x.nb[1] % 16) != 0 || (x.nb[2] % 16) != 0 || (x.nb[3] % 16) != 0))
        return unsupported("MUL_MAT over quantized weights needs 16-byte aligned activation columns", reason);
    if (w.layout == SCRAPGPU_LAYOUT_NATURAL && is_quant(w.dtype) && ((w.offset % 2) != 0 || (w.nb[1] % 2) != 0))
        return unsupported("natural quantized weights must be 2-byte aligned", reason);
    return SCRAPGPU_STATUS_OK;
}

scrapgpu_status supports(const scrapgpu_op_desc * desc, const char ** reason) {
    const char * local = nullptr;
    if (reason == nullptr) reason = &local;
    *reason = nullptr;
    if (desc == nullptr || desc->struct_size < sizeof(scrapgpu_op_desc)) return bad("op descriptor is too small", reason);
    if (desc->input_count > 32 || desc->output_count > 32 || (desc->input_count != 0 && desc->inputs == nullptr) ||
        (desc->output_count != 0 && desc->outputs == nullptr))
        return bad("invalid tensor descriptor arrays", reason);
    for (size_t i = 0; i < desc->input_count; ++i)
        if (desc->inputs[i].struct_size < sizeof(scrapgpu_tensor_desc)) return bad("input tensor descriptor is too small", reason);
    for (size_t i = 0; i < desc->output_count; ++i)
        if (desc->outputs[i].struct_size < sizeof(scrapgpu_tensor_desc)) return bad("output tensor descriptor is too small", reason);
    if (scrapgpu_op_desc_validate != nullptr) {
        const scrapgpu_status valid = scrapgpu_op_desc_validate(desc);
        if (valid != SCRAPGPU_STATUS_OK) {
            *reason = scrapgpu_last_error != nullptr ? scrapgpu_last_error() : "op descriptor failed validation";
            return valid;
        }
    }
    switch (desc->op) {
        case SCRAPGPU_OP_NONE: case SCRAPGPU_OP_RESHAPE: case SCRAPGPU_OP_VIEW: case SCRAPGPU_OP_PERMUTE: case SCRAPGPU_OP_TRANSPOSE:
            return SCRAPGPU_STATUS_OK;
        default: break;
    }
    if (desc->input_count < 1 || desc->output_count < 1) return bad("op needs at least one input and one output", reason);
    const bool multi = desc->op == SCRAPGPU_OP_MUL_MAT_MULTI;
    for (size_t i = 0; i < desc->input_count; ++i) {
        const bool weight_slot = (desc->op == SCRAPGPU_OP_MUL_MAT && i == 0) || (desc->op == SCRAPGPU_OP_GET_ROWS && i == 0) || (multi && i + 1 < desc->input_count);
        const scrapgpu_status st = check_tensor_meta(desc->inputs[i], weight_slot, reason);
        if (st != SCRAPGPU_STATUS_OK) return st;
    }
    for (size_t i = 0; i < desc->output_count; ++i) {
        const scrapgpu_status st = check_tensor_meta(desc->outputs[i], false, reason);
        if (st != SCRAPGPU_STATUS_OK) return st;
    }

    const auto s0 = load_desc(desc->inputs[0]);
    const auto s1 = desc->input_count > 1 ? load_desc(desc->inputs[1]) : scrapgpu_tensor_desc{};
    const auto s2 = desc->input_count > 2 ? load_desc(desc->inputs[2]) : scrapgpu_tensor_desc{};
    const auto dd = load_desc(desc->outputs[0]);

    switch (desc->op) {
        case SCRAPGPU_OP_ADD: case SCRAPGPU_OP_SUB: case SCRAPGPU_OP_MUL: case SCRAPGPU_OP_DIV:
            if (desc->input_count != 2) return bad("binary ops take two inputs", reason);
            if (!f32(s0) || !f32(s1) || !f32(dd)) return unsupported("binary ops need F32 tensors", reason);
            if (!same_shape(s0, dd)) return bad("binary op: src0 must have the shape of dst", reason);
            for (int i = 0; i < 4; ++i) if (ne(s1, i) > ne(dd, i)) return bad("binary op: src1 cannot be larger than dst", reason);
            return SCRAPGPU_STATUS_OK;

        case SCRAPGPU_OP_SCALE: case SCRAPGPU_OP_CLAMP: case SCRAPGPU_OP_SQR: case SCRAPGPU_OP_SQRT: case SCRAPGPU_OP_UNARY:
            if (!f32(s0) || !f32(dd)) return unsupported("unary-like ops expect F32 tensors", reason);
            if (!same_shape(s0, dd)) return bad("unary-like op: src0 must have the shape of dst", reason);
            if (desc->op == SCRAPGPU_OP_UNARY && enum_bits(load_params<scrapgpu_unary_params>(desc).kind) > (uint32_t) SCRAPGPU_UNARY_TANH)
                return unsupported("unary kind is not implemented", reason);
            return SCRAPGPU_STATUS_OK;

        case SCRAPGPU_OP_GLU: {
            const auto p = load_params<scrapgpu_glu_params>(desc);
            const bool split = desc->input_count == 2;
            if (split != (p.split_inputs != 0)) return bad("GLU: split_inputs does not match the number of inputs", reason);
            if (!f32(s0) || !f32(dd) || (split && !f32(s1))) return unsupported("GLU expects F32 tensors", reason);
            if (enum_bits(p.kind) > (uint32_t) SCRAPGPU_GLU_REGLU) return unsupported("unknown GLU kind", reason);
            if (split) return same_shape(s0, dd) && same_shape(s1, dd) ? SCRAPGPU_STATUS_OK : bad("GLU with split inputs needs src0, src1 and dst of the same shape", reason);
            for (int i = 1; i < 4; ++i) if (ne(s0, i) != ne(dd, i)) return bad("GLU: src0 and dst differ outside of dim 0", reason);
            return ne(s0, 0) == 2 * ne(dd, 0) ? SCRAPGPU_STATUS_OK : bad("GLU: src0 dim 0 must be twice the dst dim 0", reason);
        }

        case SCRAPGPU_OP_RMS_NORM:
            if (!f32(s0) || !f32(dd)) return unsupported("RMS_NORM expects F32 tensors", reason);
            return same_shape(s0, dd) ? SCRAPGPU_STATUS_OK : bad("RMS_NORM: src0 must have the shape of dst", reason);

        case SCRAPGPU_OP_RMS_NORM_MUL:
            if (desc->input_count != 2) return bad("RMS_NORM_MUL takes 2 inputs and 1 output", reason);
            if (!f32(s0) || !f32(s1) || !f32(dd)) return unsupported("RMS_NORM_MUL expects F32 tensors", reason);
            if (s1.nb[0] != 4) return unsupported("RMS_NORM_MUL needs a contiguous weight row", reason);
            return same_shape(s0, dd) && ne(s1, 0) == ne(s0, 0) ? SCRAPGPU_STATUS_OK : bad("RMS_NORM_MUL: dst must match src0 and the weight must be a row vector", reason);

        case SCRAPGPU_OP_ADD_RMS_NORM_MUL: {
            if (desc->input_count != 3 || desc->output_count != 2) return bad("ADD_RMS_NORM_MUL takes 3 inputs and 2 outputs", reason);
            const auto o1 = load_desc(desc->outputs[1]);
            if (!f32(s0) || !f32(s1) || !f32(s2) || !f32(dd) || !f32(o1)) return unsupported("ADD_RMS_NORM_MUL expects F32 tensors", reason);
            if (s2.nb[0] != 4) return unsupported("ADD_RMS_NORM_MUL needs a contiguous weight row", reason);
            return same_shape(s0, s1) && same_shape(s0, dd) && same_shape(s0, o1) && ne(s2, 0) == ne(s0, 0)
                       ? SCRAPGPU_STATUS_OK : bad("ADD_RMS_NORM_MUL: a, b, the outputs and the weight row must have matching shapes", reason);
        }

        case SCRAPGPU_OP_ROPE: {
            const auto p = load_params<scrapgpu_rope_params>(desc);
            if (enum_bits(p.mode) > (uint32_t) SCRAPGPU_ROPE_MODE_NEOX) return unsupported("unknown ROPE mode", reason);
            if (desc->input_count < 2) return bad("ROPE needs the positions tensor as inputs[1]", reason);
            if ((!f32(s0) && s0.dtype != SCRAPGPU_DTYPE_F16) || dd.dtype != s0.dtype) return unsupported("ROPE expects F32 or F16 tensors of the same dtype", reason);
            if (s1.dtype != SCRAPGPU_DTYPE_I32) return unsupported("ROPE positions must be I32", reason);
            if (p.n_offs != nullptr) return unsupported("ROPE n_offs is not supported", reason);
            if (p.freq_factors != nullptr && desc->input_count != 3) return unsupported("ROPE params->freq_factors must be NULL or describe inputs[2]", reason);
            if (p.ext_factor != 0.0f) return unsupported("ROPE with yarn extrapolation (ext_factor != 0) is not implemented on cuda_sm100", reason);
            if (!same_shape(s0, dd)) return bad("ROPE: src0 must have the shape of dst", reason);
            if (s0.nb[0] != type_size(s0.dtype) || dd.nb[0] != type_size(dd.dtype)) return unsupported("ROPE needs contiguous rows (nb0 == element size)", reason);
            if (p.n_dims <= 0 || p.n_dims % 2 != 0 || p.n_dims > s0.ne[0] || s0.ne[0] % 2 != 0) return bad("ROPE: n_dims must be a positive even number not above ne0 (ne0 even)", reason);
            if (ne(s1, 0) < ne(dd, 2)) return bad("ROPE: not enough positions for the sequence dimension", reason);
            if (s1.nb[0] != 4) return unsupported("ROPE positions must be contiguous", reason);
            if (desc->input_count == 3 && (s2.dtype != SCRAPGPU_DTYPE_F32 || ne(s2, 0) < p.n_dims / 2 || s2.nb[0] != 4))
                return bad("ROPE: freq factors must be contiguous F32 with at least n_dims/2 entries", reason);
            return SCRAPGPU_STATUS_OK;
        }

        case SCRAPGPU_OP_SOFT_MAX: {
            const auto p = load_params<scrapgpu_soft_max_params>(desc);
            if (!f32(s0) || !f32(dd)) return unsupported("SOFT_MAX expects F32 tensors", reason);
            if (!same_shape(s0, dd)) return bad("SOFT_MAX: src0 must have the shape of dst", reason);
            if (p.mask != nullptr && desc->input_count != 2) return unsupported("SOFT_MAX params->mask must be NULL or describe inputs[1]", reason);
            if (desc->input_count == 2 && ((!f32(s1) && s1.dtype != SCRAPGPU_DTYPE_F16) || ne(s1, 0) != ne(s0, 0) || ne(s1, 1) < ne(s0, 1)))
                return bad("SOFT_MAX mask must be F32/F16, as long as a row and cover the rows of src0", reason);
            return SCRAPGPU_STATUS_OK;
        }

        case SCRAPGPU_OP_GET_ROWS: {
            if (desc->input_count != 2) return bad("GET_ROWS takes two inputs", reason);
            if (s1.dtype != SCRAPGPU_DTYPE_I32 || !f32(dd)) return unsupported("GET_ROWS expects I32 indices and an F32 destination", reason);
            if (s0.dtype != SCRAPGPU_DTYPE_F32 && s0.dtype != SCRAPGPU_DTYPE_F16 && !is_quant(s0.dtype)) return unsupported("GET_ROWS dtype is not implemented", reason);
            const scrapgpu_status st = require_rows(s0, "GET_ROWS needs contiguous rows (nb0 == element size)", reason);
            if (st != SCRAPGPU_STATUS_OK) return st;
            if (s1.nb[0] != 4 || dd.nb[0] != 4) return unsupported("GET_ROWS needs contiguous indices and destination rows", reason);
            return ne(s1, 3) == 1 && ne(s1, 1) <= ne(s0, 2) && ne(s1, 2) <= ne(s0, 3) && ne(dd, 0) == ne(s0, 0) && ne(dd, 1) == ne(s1, 0) &&
                           ne(dd, 2) == ne(s1, 1) && ne(dd, 3) == ne(s1, 2)
                       ? SCRAPGPU_STATUS_OK : bad("GET_ROWS: dst must be [ne00, ids] over the slices of src0", reason);
        }

        case SCRAPGPU_OP_SET_ROWS:
        case SCRAPGPU_OP_SET_ROWS_PAIR: {
            // SET_ROWS_PAIR = two SET_ROWS in one op: inputs [src0_a, ids_a, src0_b, ids_b], outputs [dst_a, dst_b]
            // (include/scrapgpu/op.h:45, src/core/op.cpp:208-210, src/backends/opencl11/api.cpp:454-458)
            const bool pair = enum_bits(desc->op) == (uint32_t) SCRAPGPU_OP_SET_ROWS_PAIR;
            if (!pair && desc->input_count != 2) return bad("SET_ROWS takes two inputs", reason);
            if (pair && (desc->input_count != 4 || desc->output_count != 2)) return bad("SET_ROWS_PAIR takes four inputs and two outputs", reason);
            const auto okdt = [](const scrapgpu_tensor_desc & t) { return t.dtype == SCRAPGPU_DTYPE_F32 || t.dtype == SCRAPGPU_DTYPE_F16; };
            const auto one = [&](const scrapgpu_tensor_desc & src, const scrapgpu_tensor_desc & ids, const scrapgpu_tensor_desc & dst) -> scrapgpu_status {
                if (!okdt(src) || !okdt(dst)) return unsupported("SET_ROWS expects F32/F16 values and destination", reason);
                if (ids.dtype != SCRAPGPU_DTYPE_I32 && ids.dtype != SCRAPGPU_DTYPE_I64) return unsupported("SET_ROWS indices must be I32 or I64", reason);
                const scrapgpu_status st = require_rows(src, "SET_ROWS needs contiguous rows (nb0 == element size)", reason);
                if (st != SCRAPGPU_STATUS_OK) return st;
                return ne(src, 0) == ne(dst, 0) && ne(src, 2) == ne(dst, 2) && ne(src, 3) == ne(dst, 3) && ne(dst, 1) >= 1 && ne(ids, 0) >= ne(src, 1) &&
                               ne(src, 2) % ne(ids, 1) == 0 && ne(src, 3) % ne(ids, 2) == 0
                           ? SCRAPGPU_STATUS_OK : bad("SET_ROWS: dst must match src0 except along dim 1 and the index tensor must cover its rows", reason);
            };
            const scrapgpu_status first = one(s0, s1, dd);
            if (first != SCRAPGPU_STATUS_OK || !pair) return first;
            const auto s3 = load_desc(desc->inputs[3]);
            const auto o1 = load_desc(desc->outputs[1]);
            if (s0.dtype != s2.dtype || dd.dtype != o1.dtype) return unsupported("SET_ROWS_PAIR needs two SET_ROWS with the same dtypes", reason);
            return one(s2, s3, o1);
        }

        case SCRAPGPU_OP_CPY: case SCRAPGPU_OP_DUP: case SCRAPGPU_OP_CONT: {
            const auto okdt = [](const scrapgpu_tensor_desc & t) { return t.dtype == SCRAPGPU_DTYPE_F32 || t.dtype == SCRAPGPU_DTYPE_F16 || t.dtype == SCRAPGPU_DTYPE_BF16; };
            if (!okdt(s0) || !okdt(dd)) return unsupported("CPY/DUP/CONT support F32, F16 and BF16 only", reason);
            int64_t ns = 0, nd = 0;
            if (!elements(s0, ns) || !elements(dd, nd) || ns != nd) return bad("CPY/DUP/CONT: src0 and dst must have the same number of elements", reason);
            return SCRAPGPU_STATUS_OK;
        }

        case SCRAPGPU_OP_MUL_MAT: {
            if (desc->input_count != 2) return bad("MUL_MAT takes two inputs", reason);
            const auto p = load_params<scrapgpu_mul_mat_params>(desc);
            return mul_mat_shapes(s0, s1, dd, p.allow_broadcast, reason);
        }

        case SCRAPGPU_OP_MUL_MAT_MULTI: {
            // inputs [w_0 .. w_{n-1}, x], outputs [d_0 .. d_{n-1}], one F32 activation column shared by all
            const size_t n = desc->output_count;
            if (n < 2 || n > 3 || desc->input_count != n + 1) return bad("MUL_MAT_MULTI takes n+1 inputs and n outputs (2 <= n <= 3)", reason);
            const auto x = load_desc(desc->inputs[n]);
            if (ne(x, 1) != 1 || ne(x, 2) != 1 || ne(x, 3) != 1) return unsupported("MUL_MAT_MULTI shares a single activation column", reason);
            for (size_t i = 0; i < n; ++i) {
                const scrapgpu_status st = mul_mat_shapes(load_desc(desc->inputs[i]), x, load_desc(desc->outputs[i]), 0, reason);
                if (st != SCRAPGPU_STATUS_OK) return st;
            }
            return SCRAPGPU_STATUS_OK;
        }

        case SCRAPGPU_OP_CONT_MUL_MAT: {
            // inputs [a, x], output [dst]: `a` is the transposed view a CONT would have copied (dim 1 contiguous), x one
            // F32 column per (i2, i3) (src/backends/opencl11/api.cpp:260-300 states the OpenCL backend's conditions)
            if (desc->input_count != 2) return bad("CONT_MUL_MAT takes two inputs", reason);
            if ((s0.dtype != SCRAPGPU_DTYPE_F16 && !f32(s0)) || !f32(s1) || !f32(dd)) return unsupported("CONT_MUL_MAT needs an F16 or F32 view, an F32 vector and an F32 dst", reason);
            if (s0.nb[1] != type_size(s0.dtype)) return unsupported("CONT_MUL_MAT src0 must be a transposed view (dim 1 contiguous)", reason);
            if (ne(s1, 1) != 1 || s1.nb[0] != 4 || dd.nb[0] != 4 || ne(s0, 0) != ne(s1, 0) || ne(s1, 2) % ne(s0, 2) != 0 || ne(s1, 3) % ne(s0, 3) != 0)
                return unsupported("CONT_MUL_MAT needs a single F32 column x with x.ne[0] == a.ne[0] and x.ne[2], x.ne[3] multiples of a's", reason);
            if (ne(dd, 0) != ne(s0, 1) || ne(dd, 1) != 1 || ne(dd, 2) != ne(s1, 2) || ne(dd, 3) != ne(s1, 3)) return bad("CONT_MUL_MAT dst must be [a.ne1, 1, x.ne2, x.ne3]", reason);
            if (ne(s1, 2) * ne(s1, 3) > 65535) return unsupported("CONT_MUL_MAT: too many (dim 2, dim 3) slices", reason);
            return SCRAPGPU_STATUS_OK;
        }

        case SCRAPGPU_OP_ARGSORT:
            return unsupported("ARGSORT is not implemented on cuda_sm100 (TOP_K with k = 1 is)", reason);
        case SCRAPGPU_OP_TOP_K: {
            const auto p = load_params<scrapgpu_argsort_params>(desc);
            if (!f32(s0) || dd.dtype != SCRAPGPU_DTYPE_I32) return unsupported("TOP_K expects F32 keys and I32 indices", reason);
            if (ne(dd, 1) != ne(s0, 1) || ne(dd, 2) != ne(s0, 2) || ne(dd, 3) != ne(s0, 3)) return bad("TOP_K: dst must have the rows of src0", reason);
            if (p.top_k != 0 && (int64_t) p.top_k != ne(dd, 0)) return bad("TOP_K: params top_k does not match dst ne0", reason);
            if (ne(dd, 0) != 1) return unsupported("TOP_K is implemented for k = 1 (greedy arg-max) on cuda_sm100", reason);
            return SCRAPGPU_STATUS_OK;
        }

        default:
            return unsupported("op is not implemented by the cuda_sm100 backend", reason);
    }
}

// ---------------------------------------------------------------------------------------------------------
// tensor resolution and aliasing
// ---------------------------------------------------------------------------------------------------------

struct Ref {
    Buffer * buf = nullptr;
    scrapgpu_tensor_desc d = {};
    char * base() const { return static_cast<char *>(buf->ptr) + d.offset; }
};

scrapgpu_status resolve(Stream * s, const scrapgpu_tensor_desc & raw, Ref & out) {
    const scrapgpu_tensor_desc td = load_desc(raw);
    Buffer * b = as_buffer(td.buffer);
    if (b == nullptr) return invalid("tensor desc has no cuda_sm100 buffer");
    if (b->dev != s->dev) return invalid("tensor buffer and stream belong to different devices");
    const uint64_t nbytes = span_bytes(td);
    if (td.offset > (uint64_t) b->size || nbytes > (uint64_t) b->size - td.offset) return invalid("tensor exceeds its buffer");
    out.buf = b;
    out.d = td;
    return SCRAPGPU_STATUS_OK;
}

bool overlap(const Ref & a, const Ref & b) {
    if (a.buf != b.buf) return false;
    const uint64_t a0 = a.d.offset, a1 = a0 + span_bytes(a.d), b0 = b.d.offset, b1 = b0 + span_bytes(b.d);
    return a0 < b1 && b0 < a1;
}

bool same_view(const Ref & a, const Ref & b) {
    if (a.buf != b.buf || a.d.offset != b.d.offset || a.d.dtype != b.d.dtype) return false;
    for (int i = 0; i < 4; ++i) if (a.d.ne[i] != b.d.ne[i] || a.d.nb[i] != b.d.nb[i]) return false;
    return true;
}

// in-place is sound only where a thread reads an element before it writes the same element
bool in_place_ok(scrapgpu_op op) {
    switch (op) {
        case SCRAPGPU_OP_ADD: case SCRAPGPU_OP_SUB: case SCRAPGPU_OP_MUL: case SCRAPGPU_OP_DIV: case SCRAPGPU_OP_GLU:
        case SCRAPGPU_OP_SCALE: case SCRAPGPU_OP_CLAMP: case SCRAPGPU_OP_SQR: case SCRAPGPU_OP_SQRT: case SCRAPGPU_OP_UNARY:
        case SCRAPGPU_OP_RMS_NORM: case SCRAPGPU_OP_SOFT_MAX: case SCRAPGPU_OP_RMS_NORM_MUL: case SCRAPGPU_OP_ADD_RMS_NORM_MUL:
        case SCRAPGPU_OP_CPY: case SCRAPGPU_OP_DUP: case SCRAPGPU_OP_CONT:
            return true;
        default:
            return false;
    }
}

scrapgpu_status check_aliasing(scrapgpu_op op, const std::vector<Ref> & in, const std::vector<Ref> & out) {
    for (size_t i = 0; i < out.size(); ++i)
        for (size_t j = i + 1; j < out.size(); ++j)
            if (overlap(out[i], out[j])) return invalid("op outputs overlap each other");
    for (size_t i = 0; i < out.size(); ++i) {
        for (size_t j = 0; j < in.size(); ++j) {
            if (!overlap(out[i], in[j])) continue;
            if (!in_place_ok(op)) return invalid("the output overlaps an input and this op is not in-place safe");
            if (!same_view(out[i], in[j])) return invalid("a partially overlapping output/input view is not in-place safe");
            if ((op == SCRAPGPU_OP_RMS_NORM_MUL && j == 1) || (op == SCRAPGPU_OP_ADD_RMS_NORM_MUL && j == 2)) return invalid("normalization outputs must not alias the weight input");
            // a GLU over fused halves reads two elements per output: in place would overwrite a later input
            if (op == SCRAPGPU_OP_GLU && in.size() == 1) return invalid("GLU over fused halves cannot run in place");
        }
    }
    return SCRAPGPU_STATUS_OK;
}

sm100_view view_of(const Ref & r) {
    sm100_view v;
    v.data = r.base();
    for (int i = 0; i < 4; ++i) {
        v.ne[i] = ne(r.d, i);
        v.nb[i] = (int64_t) r.d.nb[i];
    }
    return v;
}

// ---------------------------------------------------------------------------------------------------------
// ROPE tables
// ---------------------------------------------------------------------------------------------------------

uint32_t float_bits(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return u;
}

// (cos, sin) for positions [0, n) and pairs [0, n_dims/2): theta = position * theta_scale^j by sequential f32
// multiplies, theta_scale = powf(base, -2/n_dims), libm cosf/sinf, times attn_factor (src/core/ref/ops.cpp:559-601).
// volatile keeps the compiler from contracting or reassociating the products.
scrapgpu_status rope_table(Device * dev, Stream * s, int n_dims, float base, float freq_scale, float attn_factor, const float ** out, int32_t * count) {
    static const int32_t kPositions = [] {
        const char * v = std::getenv("SCRAPGPU_SM100_ROPE_TABLE");
        const long n = v != nullptr ? std::atol(v) : 4096;
        return (int32_t) (n < 0 ? 0 : n > (1 << 20) ? (1 << 20) : n);
    }();
    *out = nullptr;
    *count = 0;
    if (kPositions == 0) return SCRAPGPU_STATUS_OK;
    const auto key = std::make_tuple(n_dims, float_bits(base), float_bits(freq_scale), float_bits(attn_factor));
    std::lock_guard<std::mutex> lock(dev->rope_mutex);
    auto it = dev->rope_tables.find(key);
    if (it == dev->rope_tables.end()) {
        const int half = n_dims / 2;
        std::vector<float> host((size_t) kPositions * half * 2);
        const float theta_scale = std::pow(base, -2.0f / (float) n_dims);
        for (int32_t p = 0; p < kPositions; ++p) {
            volatile float theta = (float) p;
            for (int j = 0; j < half; ++j) {
                const float th = freq_scale * (theta / 1.0f);
                host[((size_t) p * half + j) * 2 + 0] = std::cos(th) * attn_factor;
                host[((size_t) p * half + j) * 2 + 1] = std::sin(th) * attn_factor;
                theta = theta * theta_scale;
            }
        }
        void * devp = nullptr;
        scrapgpu_status st = from_sm100(sm100_malloc(dev->ordinal, host.size() * sizeof(float), &devp));
        if (st != SCRAPGPU_STATUS_OK) return st;
        st = from_sm100(sm100_memcpy_h2d(s->cuda, devp, host.data(), host.size() * sizeof(float), 1));
        if (st != SCRAPGPU_STATUS_OK) {
            sm100_free(dev->ordinal, devp);
            return st;
        }
        it = dev->rope_tables.emplace(key, std::make_pair(devp, kPositions)).first;
    }
    *out = static_cast<const float *>(it->second.first);
    *count = it->second.second;
    return SCRAPGPU_STATUS_OK;
}

// ---------------------------------------------------------------------------------------------------------
// op dispatch
// ---------------------------------------------------------------------------------------------------------

bool dense_rows(const scrapgpu_tensor_desc & t) {
    // rows follow each other without gaps across all outer dims
    uint64_t next = t.nb[0] * (uint64_t) t.ne[0];
    if (t.nb[0] != type_size(t.dtype)) return false;
    for (int i = 1; i < 4; ++i) {
        if (t.ne[i] != 1 && t.nb[i] != next) return false;
        next *= (uint64_t) t.ne[i];
    }
    return true;
}

scrapgpu_status run_mul_mat(Stream * s, const Ref & w, const Ref & x, const Ref & d) {
    const int64_t k = ne(w.d, 0), n = ne(w.d, 1), m = ne(x.d, 1);
    const int64_t r2 = ne(x.d, 2) / ne(w.d, 2), r3 = ne(x.d, 3) / ne(w.d, 3);
    const int layout = w.d.layout == SCRAPGPU_LAYOUT_R32 ? 1 : 0;
    for (int64_t i3 = 0; i3 < ne(x.d, 3); ++i3) {
        for (int64_t i2 = 0; i2 < ne(x.d, 2); ++i2) {
            const char * wp = w.base() + (i2 / r2) * w.d.nb[2] + (i3 / r3) * w.d.nb[3];
            const float * xp = reinterpret_cast<const float *>(x.base() + i2 * x.d.nb[2] + i3 * x.d.nb[3]);
            float * yp = reinterpret_cast<float *>(d.base() + i2 * d.d.nb[2] + i3 * d.d.nb[3]);
            const scrapgpu_status st = from_sm100(sm100_mul_mat(s->cuda, w.d.dtype, layout, wp, layout ? 0 : (int64_t) w.d.nb[1], k, n, xp,
                                                                (int64_t) (x.d.nb[1] / 4), m, yp, (int64_t) (d.d.nb[1] / 4)));
            if (st != SCRAPGPU_STATUS_OK) return st;
        }
    }
    return SCRAPGPU_STATUS_OK;
}

// ---- profile table ----
bool profiling() {
    static const bool on = [] { const char * e = std::getenv("SCRAPGPU_SM100_PROFILE"); return e != nullptr && std::atoi(e) != 0; }();
    return on;
}

const char * dtype_name(int dt) {
    switch (dt) {
        case SCRAPGPU_DTYPE_F32: return "f32";
        case SCRAPGPU_DTYPE_F16: return "f16";
        case SCRAPGPU_DTYPE_I32: return "i32";
        case SCRAPGPU_DTYPE_I64: return "i64";
        case SCRAPGPU_DTYPE_I16: return "i16";
        case SCRAPGPU_DTYPE_BF16: return "bf16";
        case SCRAPGPU_DTYPE_Q4_0: return "q4_0";
        case SCRAPGPU_DTYPE_Q8_0: return "q8_0";
        case SCRAPGPU_DTYPE_Q4_K: return "q4_K";
        case SCRAPGPU_DTYPE_Q6_K: return "q6_K";
        default: return "?";
    }
}

const char * op_name(int op);

// the key of an op in the table: the op, for MUL_MAT the weight type, matvec or matrix form and the column count, for
// the row and copy ops the two types (the keys of adapters/ggml/ggml-cl11.cpp:1033-1049)
std::string prof_key_name(const scrapgpu_op_desc * desc) {
    std::string key = op_name(desc->op);
    if (desc->input_count == 0 || desc->inputs == nullptr) return key;
    const scrapgpu_tensor_desc a = load_desc(desc->inputs[0]);
    if (desc->op == SCRAPGPU_OP_MUL_MAT && desc->input_count >= 2) {
        const int64_t cols = ne(load_desc(desc->inputs[1]), 1);
        key += std::string(" ") + dtype_name(a.dtype) + (a.layout == SCRAPGPU_LAYOUT_R32 ? " packed" : "") + (cols <= 8 ? " mv" : " mm") + " n=" + std::to_string(cols);
    } else if (desc->op == SCRAPGPU_OP_MUL_MAT_MULTI) {
        key += std::string(" ") + dtype_name(a.dtype) + " x" + std::to_string(desc->output_count);
    } else if ((desc->op == SCRAPGPU_OP_GET_ROWS || desc->op == SCRAPGPU_OP_CPY || desc->op == SCRAPGPU_OP_SET_ROWS) && desc->output_count >= 1) {
        key += std::string(" ") + dtype_name(a.dtype) + "->" + dtype_name(load_desc(desc->outputs[0]).dtype);
    }
    static const bool shapes = std::getenv("SCRAPGPU_SM100_PROFILE_SHAPES") != nullptr;
    if (shapes) {
        char buf[96];
        std::snprintf(buf, sizeof(buf), " src0[%lld,%lld,%lld,%lld]", (long long) ne(a, 0), (long long) ne(a, 1), (long long) ne(a, 2), (long long) ne(a, 3));
        key += buf;
    }
    return key;
}

double weight_bytes(const scrapgpu_tensor_desc & w) {
    return (double) (ne(w, 0) / (int64_t) block_size(w.dtype)) * (double) type_size(w.dtype) * (double) (ne(w, 1) * ne(w, 2) * ne(w, 3));
}

// Brackets the launches of one op with two events while the table is on; the launches inside are fully serialized so
// that the pair times this op alone (with programmatic dependent launch neighbouring kernels overlap).
struct ProfScope {
    Stream * s = nullptr;
    sm100_event_t start = nullptr;
    int key = -1;
    ProfScope(Stream * stream, const std::string & name, double bytes) {
        if (!profiling()) return;
        s = stream;
        for (size_t i = 0; i < s->prof_stats.size() && key < 0; ++i) if (s->prof_stats[i].name == name) key = (int) i;
        if (key < 0) {
            s->prof_stats.emplace_back();
            s->prof_stats.back().name = name;
            key = (int) s->prof_stats.size() - 1;
        }
        s->prof_stats[(size_t) key].count++;
        s->prof_stats[(size_t) key].bytes += bytes;
        start = event();
        if (start != nullptr) sm100_event_record(start, s->cuda);
        sm100_launch_serialized(1);
    }
    ~ProfScope() {
        if (s == nullptr) return;
        sm100_launch_serialized(0);
        sm100_event_t stop = start != nullptr ? event() : nullptr;
        if (stop == nullptr) {
            if (start != nullptr) s->prof_spare.push_back(start);
            return;
        }
        sm100_event_record(stop, s->cuda);
        try {
            s->prof_pending.push_back({start, stop, key});
        } catch (...) {   // out of memory for the bookkeeping: this op goes untimed
            sm100_event_destroy(start);
            sm100_event_destroy(stop);
        }
    }
    sm100_event_t event() {
        if (!s->prof_spare.empty()) {
            sm100_event_t e = s->prof_spare.back();
            s->prof_spare.pop_back();
            return e;
        }
        sm100_event_t e = nullptr;
        return sm100_event_create(&e) == 0 ? e : nullptr;
    }
};

// after a successful stream synchronisation: the finished pairs go into the table
void prof_collect(Stream * s) {
    for (const Stream::ProfPending & p : s->prof_pending) {
        float ms = 0.0f;
        if (sm100_event_elapsed_ms(p.start, p.stop, &ms) == 0 && p.key >= 0 && (size_t) p.key < s->prof_stats.size()) s->prof_stats[(size_t) p.key].ms += ms;
        s->prof_spare.push_back(p.start);
        s->prof_spare.push_back(p.stop);
    }
    s->prof_pending.clear();
}

// the table as text, slowest key first (the layout of cl11_prof_print, src/backends/opencl11/executor.h:87-106)
std::string prof_report(Stream * s) {
    std::vector<const Stream::ProfStat *> v;
    double total = 0;
    for (const Stream::ProfStat & st : s->prof_stats) {
        v.push_back(&st);
        total += st.ms;
    }
    std::sort(v.begin(), v.end(), [](const Stream::ProfStat * a, const Stream::ProfStat * b) { return a->ms > b->ms; });
    char line[256];
    std::snprintf(line, sizeof(line), "cuda_sm100 profile of %s: total kernel time %.3f ms\n", s->dev->name.c_str(), total);
    std::string out = line;
    for (const Stream::ProfStat * st : v) {
        char gbs[64] = "";
        if (st->bytes > 0 && st->ms > 0) std::snprintf(gbs, sizeof(gbs), "  weights %.2f GB/s", st->bytes / (st->ms * 1e6));
        std::snprintf(line, sizeof(line), "  %-44s %6zu calls %10.3f ms %8.1f us/call %5.1f%%%s\n", st->name.c_str(), st->count, st->ms,
                      st->ms * 1e3 / (double) std::max<size_t>(1, st->count), 100.0 * st->ms / std::max(1e-9, total), gbs);
        out += line;
    }
    return out;
}

// The matvec and GEMM kernels request their weights before they wait for the kernels ahead of them on the stream
// (sm100_launch_serialized in scrapgpu_sm100.h).  That is sound for weights that sit in memory since an upload, not for
// a left operand some kernel has written since the stream last settled (the K cache of the core's attention
// composition, a CPY into a weight): such a MUL_MAT is launched fully serialized.
bool fresh(const Stream * s, const scrapgpu_tensor_desc & raw) {
    const Buffer * b = as_buffer(load_desc(raw).buffer);
    return b != nullptr && b->writer.load(std::memory_order_relaxed) == s && b->written.load(std::memory_order_relaxed) > s->settled;
}
void wrote(Stream * s, const scrapgpu_tensor_desc & raw) {
    Buffer * b = as_buffer(load_desc(raw).buffer);
    if (b == nullptr) return;
    b->writer.store(s, std::memory_order_relaxed);
    b->written.store(s->epoch, std::memory_order_relaxed);
}
struct Serialized {
    bool on;
    explicit Serialized(bool o) : on(o) { if (on) sm100_launch_serialized(1); }
    ~Serialized() { if (on) sm100_launch_serialized(0); }
};

scrapgpu_status execute_op(Stream * s, const scrapgpu_op_desc * desc);

scrapgpu_status execute(Stream * s, const scrapgpu_op_desc * desc) {
    bool serial = false;
    if (desc != nullptr && desc->inputs != nullptr) {
        const size_t weights = desc->op == SCRAPGPU_OP_MUL_MAT || desc->op == SCRAPGPU_OP_CONT_MUL_MAT ? 1
                               : desc->op == SCRAPGPU_OP_MUL_MAT_MULTI ? desc->output_count : 0;
        for (size_t i = 0; i < weights && i < desc->input_count; ++i) serial = serial || fresh(s, desc->inputs[i]);
    }
    scrapgpu_status st;
    if (profiling() && desc != nullptr) {
        const bool mm = (desc->op == SCRAPGPU_OP_MUL_MAT || desc->op == SCRAPGPU_OP_MUL_MAT_MULTI) && desc->inputs != nullptr;
        double bytes = 0;
        for (size_t i = 0; mm && i < (desc->op == SCRAPGPU_OP_MUL_MAT ? 1 : desc->output_count) && i < desc->input_count; ++i) bytes += weight_bytes(load_desc(desc->inputs[i]));
        ProfScope prof(s, prof_key_name(desc), bytes);
        st = execute_op(s, desc);
    } else {
        Serialized scope(serial);
        st = execute_op(s, desc);
    }
    if (st == SCRAPGPU_STATUS_OK && desc->outputs != nullptr) {
        ++s->epoch;
        for (size_t i = 0; i < desc->output_count; ++i) wrote(s, desc->outputs[i]);
    }
    return st;
}

scrapgpu_status execute_op(Stream * s, const scrapgpu_op_desc * desc) {
    const char * why = nullptr;
    scrapgpu_status st = supports(desc, &why);
    if (st != SCRAPGPU_STATUS_OK) return st;
    switch (desc->op) {
        case SCRAPGPU_OP_NONE: case SCRAPGPU_OP_RESHAPE: case SCRAPGPU_OP_VIEW: case SCRAPGPU_OP_PERMUTE: case SCRAPGPU_OP_TRANSPOSE:
            return SCRAPGPU_STATUS_OK;  // metadata only
        default: break;
    }
    std::vector<Ref> in(desc->input_count), out(desc->output_count);
    for (size_t i = 0; i < desc->input_count; ++i) {
        st = resolve(s, desc->inputs[i], in[i]);
        if (st != SCRAPGPU_STATUS_OK) return st;
    }
    for (size_t i = 0; i < desc->output_count; ++i) {
        st = resolve(s, desc->outputs[i], out[i]);
        if (st != SCRAPGPU_STATUS_OK) return st;
    }
    st = check_aliasing(desc->op, in, out);
    if (st != SCRAPGPU_STATUS_OK) return st;
    st = from_sm100(sm100_set_device(s->dev->ordinal));
    if (st != SCRAPGPU_STATUS_OK) return st;

    switch (desc->op) {
        case SCRAPGPU_OP_ADD: case SCRAPGPU_OP_SUB: case SCRAPGPU_OP_MUL: case SCRAPGPU_OP_DIV: {
            int64_t n = 0;
            if (desc->op == SCRAPGPU_OP_ADD && same_shape(in[0].d, in[1].d) && dense_rows(in[0].d) && dense_rows(in[1].d) && dense_rows(out[0].d) &&
                elements(out[0].d, n))
                return from_sm100(sm100_add(s->cuda, (const float *) in[0].base(), (const float *) in[1].base(), (float *) out[0].base(), n));
            const sm100_view a = view_of(in[0]), b = view_of(in[1]), y = view_of(out[0]);
            return from_sm100(sm100_binary(s->cuda, (int) desc->op - (int) SCRAPGPU_OP_ADD, &a, &b, &y));
        }
        case SCRAPGPU_OP_SCALE: case SCRAPGPU_OP_CLAMP: case SCRAPGPU_OP_SQR: case SCRAPGPU_OP_SQRT: case SCRAPGPU_OP_UNARY: {
            const sm100_view x = view_of(in[0]), y = view_of(out[0]);
            int code = 0;
            float p0 = 0.f, p1 = 0.f;
            if (desc->op == SCRAPGPU_OP_SCALE) { const auto p = load_params<scrapgpu_scale_params>(desc); code = 0; p0 = p.scale; p1 = p.bias; }
            else if (desc->op == SCRAPGPU_OP_CLAMP) { const auto p = load_params<scrapgpu_clamp_params>(desc); code = 1; p0 = p.min_value; p1 = p.max_value; }
            else if (desc->op == SCRAPGPU_OP_SQR) code = 2;
            else if (desc->op == SCRAPGPU_OP_SQRT) code = 3;
            else code = 10 + (int) enum_bits(load_params<scrapgpu_unary_params>(desc).kind);
            return from_sm100(sm100_unary(s->cuda, code, p0, p1, &x, &y));
        }
        case SCRAPGPU_OP_GLU: {
            const auto p = load_params<scrapgpu_glu_params>(desc);
            const sm100_view x = view_of(in[0]), y = view_of(out[0]);
            if (desc->input_count == 2) {
                int64_t n = 0;
                if (p.kind == SCRAPGPU_GLU_SWIGLU && dense_rows(in[0].d) && dense_rows(in[1].d) && dense_rows(out[0].d) && elements(out[0].d, n))
                    return from_sm100(sm100_swiglu(s->cuda, (const float *) in[0].base(), (const float *) in[1].base(), (float *) out[0].base(), n));
                const sm100_view g = view_of(in[1]);
                return from_sm100(sm100_glu(s->cuda, (int) p.kind, &x, &g, 0, &y));
            }
            return from_sm100(sm100_glu(s->cuda, (int) p.kind, &x, nullptr, p.swapped != 0, &y));
        }
        case SCRAPGPU_OP_RMS_NORM: case SCRAPGPU_OP_RMS_NORM_MUL: {
            const auto p = load_params<scrapgpu_rms_norm_params>(desc);
            const float * w = desc->op == SCRAPGPU_OP_RMS_NORM_MUL ? (const float *) in[1].base() : nullptr;
            const sm100_view x = view_of(in[0]), y = view_of(out[0]);
            return from_sm100(sm100_rms_norm_view(s->cuda, &x, nullptr, w, nullptr, &y, p.eps));
        }
        case SCRAPGPU_OP_ADD_RMS_NORM_MUL: {
            const auto p = load_params<scrapgpu_rms_norm_params>(desc);
            const sm100_view a = view_of(in[0]), b = view_of(in[1]), sum = view_of(out[0]), y = view_of(out[1]);
            return from_sm100(sm100_rms_norm_view(s->cuda, &a, &b, (const float *) in[2].base(), &sum, &y, p.eps));
        }
        case SCRAPGPU_OP_ROPE: {
            const auto p = load_params<scrapgpu_rope_params>(desc);
            const float * table = nullptr;
            int32_t count = 0;
            const float * ff = desc->input_count > 2 ? (const float *) in[2].base() : nullptr;
            if (ff == nullptr) {
                st = rope_table(s->dev, s, p.n_dims, p.freq_base, p.freq_scale, p.attn_factor, &table, &count);
                if (st != SCRAPGPU_STATUS_OK) return st;
            }
            const sm100_view x = view_of(in[0]), y = view_of(out[0]);
            return from_sm100(sm100_rope_view_dt(s->cuda, in[0].d.dtype, &x, (const int32_t *) in[1].base(), table, 0, count, ff, &y, p.n_dims,
                                                 p.mode == SCRAPGPU_ROPE_MODE_NEOX, p.freq_base, p.freq_scale, p.attn_factor));
        }
        case SCRAPGPU_OP_SOFT_MAX: {
            const auto p = load_params<scrapgpu_soft_max_params>(desc);
            const sm100_view x = view_of(in[0]), y = view_of(out[0]);
            if (desc->input_count == 2) {
                const sm100_view m = view_of(in[1]);
                return from_sm100(sm100_soft_max_view(s->cuda, &x, &m, in[1].d.dtype == SCRAPGPU_DTYPE_F16, &y, p.scale));
            }
            return from_sm100(sm100_soft_max_view(s->cuda, &x, nullptr, 0, &y, p.scale));
        }
        case SCRAPGPU_OP_GET_ROWS: {
            const Ref & t = in[0];
            const Ref & ids = in[1];
            const int layout = t.d.layout == SCRAPGPU_LAYOUT_R32 ? 1 : 0;
            for (int64_t i12 = 0; i12 < ne(ids.d, 2); ++i12) {
                for (int64_t i11 = 0; i11 < ne(ids.d, 1); ++i11) {
                    const char * tp = t.base() + i11 * t.d.nb[2] + i12 * t.d.nb[3];
                    const int32_t * ip = (const int32_t *) (ids.base() + i11 * ids.d.nb[1] + i12 * ids.d.nb[2]);
                    float * dp = (float *) (out[0].base() + i11 * out[0].d.nb[2] + i12 * out[0].d.nb[3]);
                    st = from_sm100(sm100_get_rows(s->cuda, t.d.dtype, layout, tp, layout ? 0 : (int64_t) t.d.nb[1], ne(t.d, 0), ne(t.d, 1), ip, ne(ids.d, 0), dp,
                                                   (int64_t) (out[0].d.nb[1] / 4)));
                    if (st != SCRAPGPU_STATUS_OK) return st;
                }
            }
            return SCRAPGPU_STATUS_OK;
        }
        case SCRAPGPU_OP_SET_ROWS: {
            const sm100_view src = view_of(in[0]), ids = view_of(in[1]), dst = view_of(out[0]);
            return from_sm100(sm100_set_rows_view(s->cuda, &src, in[0].d.dtype, &ids, in[1].d.dtype == SCRAPGPU_DTYPE_I64, &dst, out[0].d.dtype));
        }
        case SCRAPGPU_OP_SET_ROWS_PAIR: {
            for (int i = 0; i < 2; ++i) {
                const sm100_view src = view_of(in[2 * i]), ids = view_of(in[2 * i + 1]), dst = view_of(out[i]);
                const scrapgpu_status st = from_sm100(
                    sm100_set_rows_view(s->cuda, &src, in[2 * i].d.dtype, &ids, in[2 * i + 1].d.dtype == SCRAPGPU_DTYPE_I64, &dst, out[i].d.dtype));
                if (st != SCRAPGPU_STATUS_OK) return st;
            }
            return SCRAPGPU_STATUS_OK;
        }
        case SCRAPGPU_OP_CPY: case SCRAPGPU_OP_DUP: case SCRAPGPU_OP_CONT: {
            const sm100_view src = view_of(in[0]), dst = view_of(out[0]);
            return from_sm100(sm100_cpy(s->cuda, &src, in[0].d.dtype, &dst, out[0].d.dtype));
        }
        case SCRAPGPU_OP_MUL_MAT:
            return run_mul_mat(s, in[0], in[1], out[0]);
        case SCRAPGPU_OP_MUL_MAT_MULTI: {
            const size_t n = desc->output_count;
            bool fusable = true;
            int dtypes[3], layouts[3];
            const void * ws[3];
            int64_t ns[3];
            float * ys[3];
            for (size_t i = 0; i < n; ++i) {
                const Ref & w = in[i];
                dtypes[i] = w.d.dtype;
                layouts[i] = w.d.layout == SCRAPGPU_LAYOUT_R32 ? 1 : 0;
                ws[i] = w.base();
                ns[i] = ne(w.d, 1);
                ys[i] = (float *) out[i].base();
                fusable = fusable && (layouts[i] == 1 || w.d.nb[1] == (uint64_t) (ne(w.d, 0) / (int64_t) block_size(w.d.dtype)) * type_size(w.d.dtype)) && ne(w.d, 2) * ne(w.d, 3) == 1;
            }
            if (fusable) return from_sm100(sm100_mul_mat_multi(s->cuda, (int) n, dtypes, layouts, ws, ne(in[n].d, 0), ns, (const float *) in[n].base(), ys));
            for (size_t i = 0; i < n; ++i) {
                st = run_mul_mat(s, in[i], in[n], out[i]);
                if (st != SCRAPGPU_STATUS_OK) return st;
            }
            return SCRAPGPU_STATUS_OK;
        }
        case SCRAPGPU_OP_CONT_MUL_MAT: {
            const sm100_view a = view_of(in[0]), x = view_of(in[1]), y = view_of(out[0]);
            return from_sm100(sm100_cont_mul_mat(s->cuda, &a, in[0].d.dtype, &x, &y));
        }
        case SCRAPGPU_OP_TOP_K: {
            const sm100_view x = view_of(in[0]), o = view_of(out[0]);
            return from_sm100(sm100_top1_view(s->cuda, &x, &o));
        }
        default:
            return unsupported("op is not implemented by the cuda_sm100 backend");
    }
}

// failures of enqueued work are remembered on the stream and reported at the next sync as well
scrapgpu_status enqueue_result(Stream * s, scrapgpu_status st) {
    if (st == SCRAPGPU_STATUS_BACKEND_ERROR || st == SCRAPGPU_STATUS_DEVICE_LOST) {
        s->sticky = st;
        const char * m = sm100_last_error();
        s->sticky_message = m != nullptr ? m : "";
    }
    return st;
}

// ---------------------------------------------------------------------------------------------------------
// vtable: devices
// ---------------------------------------------------------------------------------------------------------

void probe_devices() {
    if (g_devices_probed) return;
    g_devices_probed = true;
    const int n = sm100_device_count();
    for (int i = 0; i < n; ++i) {
        char name[128] = {};
        uint64_t mem = 0, shared = 0;
        uint32_t sms = 0, major = 0, minor = 0;
        if (sm100_device_info(i, name, sizeof(name), &mem, &sms, &major, &minor, &shared) != 0) continue;
        if (major != 10) continue;  // kernels are built for sm_100a only
        auto d = std::make_unique<Device>();
        d->hdr.backend = &g_vtable;
        d->ordinal = i;
        d->name = name;
        d->total_memory = mem;
        d->shared_per_block = shared;
        d->sms = sms;
        d->cc_major = major;
        d->cc_minor = minor;
        g_devices.push_back(std::move(d));
    }
}

size_t v_get_device_count(void *) {
    std::lock_guard<std::mutex> lock(g_registry_mutex);
    probe_devices();
    return g_devices.size();
}

scrapgpu_status v_get_device(void *, size_t index, scrapgpu_device_t ** out_device) {
    return guard([&]() -> scrapgpu_status {
        if (out_device == nullptr) return invalid("out_device is null");
        std::lock_guard<std::mutex> lock(g_registry_mutex);
        probe_devices();
        if (index >= g_devices.size()) return invalid("device index out of range");
        *out_device = reinterpret_cast<scrapgpu_device_t *>(g_devices[index].get());
        return SCRAPGPU_STATUS_OK;
    });
}

scrapgpu_status v_device_get_info(scrapgpu_device_t * device, scrapgpu_device_info * info) {
    return guard([&]() -> scrapgpu_status {
        Device * d = as_device(device);
        if (d == nullptr) return invalid("not a cuda_sm100 device");
        if (info == nullptr || info->struct_size < sizeof(size_t)) return invalid("device info struct is too small");
        static const std::string used = "CUDA runtime, kernels built for sm_100a";
        scrapgpu_device_info full = {};
        full.struct_size = sizeof(full);
        full.name = d->name.c_str();
        full.vendor = "NVIDIA";
        full.platform_name = "CUDA";
        full.driver_version = "";
        full.backend_name = "cuda_sm100";
        full.reported_api_version = d->cc_minor == 0 ? "compute capability 10.0" : "compute capability 10.x";
        full.used_api_version = used.c_str();
        full.generation = SCRAPGPU_DEVICE_GENERATION_UNKNOWN;
        full.generation_reason = "NVIDIA Blackwell (sm_100a); newer than the generations the enum names";
        full.total_memory_bytes = d->total_memory;
        full.max_allocation_reported_bytes = d->total_memory;
        full.max_allocation_used_bytes = d->total_memory;
        full.max_work_group_size = 1024;
        full.local_memory_bytes = d->shared_per_block;
        full.compute_units = d->sms;
        full.warp_or_wave_width = 32;
        full.quirks = 0;
        full.probed_quirks = 0;
        full.tuning_profile_name = "b200";
        full.tuning_overrides = "";
        const size_t caller = info->struct_size;
        std::memcpy(info, &full, std::min(caller, sizeof(full)));
        info->struct_size = caller;
        return SCRAPGPU_STATUS_OK;
    });
}

// ---------------------------------------------------------------------------------------------------------
// vtable: buffers
// ---------------------------------------------------------------------------------------------------------

scrapgpu_status v_buffer_alloc(scrapgpu_device_t * device, size_t size, scrapgpu_buffer_t ** out_buffer) {
    return guard([&]() -> scrapgpu_status {
        Device * d = as_device(device);
        if (d == nullptr || out_buffer == nullptr) return invalid("device or out_buffer is null");
        *out_buffer = nullptr;
        auto b = std::make_unique<Buffer>();
        b->hdr.backend = &g_vtable;
        b->dev = d;
        b->size = size;
        const scrapgpu_status st = from_sm100(sm100_malloc(d->ordinal, size == 0 ? 1 : size, &b->ptr));  // cudaMalloc: >= 256-byte aligned
        if (st != SCRAPGPU_STATUS_OK) return st;
        *out_buffer = reinterpret_cast<scrapgpu_buffer_t *>(b.release());
        return SCRAPGPU_STATUS_OK;
    });
}

scrapgpu_status v_buffer_free(scrapgpu_buffer_t * buffer) {
    return guard([&]() -> scrapgpu_status {
        Buffer * b = as_buffer(buffer);
        if (b == nullptr) return invalid("not a cuda_sm100 buffer");
        {
            std::lock_guard<std::mutex> lock(g_pin_mutex);
            if (g_pins.find(b) != g_pins.end()) return invalid("buffer is still referenced by a live plan");
        }
        const scrapgpu_status st = from_sm100(sm100_free(b->dev->ordinal, b->ptr));
        b->hdr.backend = nullptr;
        delete b;
        return st;
    });
}

struct Io {
    Stream * s;
    Buffer * b;
};

scrapgpu_status io_check(scrapgpu_stream_t * stream, scrapgpu_buffer_t * buffer, uint64_t offset, size_t size, const char * what, Io & io) {
    io.s = as_stream(stream);
    io.b = as_buffer(buffer);
    if (io.s == nullptr || io.b == nullptr) return invalid("stream or buffer is not a cuda_sm100 object");
    if (io.b->dev != io.s->dev) return invalid("buffer and stream belong to different devices");
    if (size != 0 && (offset > (uint64_t) io.b->size || size > io.b->size - (size_t) offset)) return invalid(what);
    io.s->settled = io.s->epoch;   // a copy or fill on the stream runs after all kernels before it and before all after it
    return from_sm100(sm100_set_device(io.s->dev->ordinal));
}

scrapgpu_status v_buffer_write(scrapgpu_stream_t * stream, scrapgpu_buffer_t * buffer, uint64_t offset, const void * data, size_t size, int blocking) {
    return guard([&]() -> scrapgpu_status {
        Io io;
        const scrapgpu_status st = io_check(stream, buffer, offset, size, "write exceeds the buffer", io);
        if (st != SCRAPGPU_STATUS_OK || size == 0) return st;
        if (data == nullptr) return invalid("data is null");
        // blocking = 0 enqueues the copy (in stream order) and returns.  From page-locked host memory the copy engine
        // reads `data` later, so the caller keeps it untouched until the next stream_sync, as with a non-blocking
        // clEnqueueWriteBuffer of the OpenCL backend; a pageable source is staged by the CUDA runtime before the call
        // returns, so it may be reused at once.
        return enqueue_result(io.s, from_sm100(sm100_memcpy_h2d(io.s->cuda, static_cast<char *>(io.b->ptr) + offset, data, size, blocking != 0)));
    });
}

scrapgpu_status v_buffer_read(scrapgpu_stream_t * stream, scrapgpu_buffer_t * buffer, uint64_t offset, void * data, size_t size, int blocking) {
    return guard([&]() -> scrapgpu_status {
        Io io;
        const scrapgpu_status st = io_check(stream, buffer, offset, size, "read exceeds the buffer", io);
        if (st != SCRAPGPU_STATUS_OK || size == 0) return st;
        if (data == nullptr) return invalid("data is null");
        // blocking = 0: `data` holds the bytes after the next stream_sync (page-locked destination; the CUDA runtime
        // completes a copy into pageable memory before it returns)
        return enqueue_result(io.s, from_sm100(sm100_memcpy_d2h(io.s->cuda, data, static_cast<char *>(io.b->ptr) + offset, size, blocking != 0)));
    });
}

scrapgpu_status v_buffer_copy(scrapgpu_stream_t * stream, scrapgpu_buffer_t * dst, uint64_t dst_offset, scrapgpu_buffer_t * src, uint64_t src_offset, size_t size,
                              int blocking) {
    return guard([&]() -> scrapgpu_status {
        Io a, b;
        scrapgpu_status st = io_check(stream, dst, dst_offset, size, "copy exceeds a buffer", a);
        if (st != SCRAPGPU_STATUS_OK) return st;
        st = io_check(stream, src, src_offset, size, "copy exceeds a buffer", b);
        if (st != SCRAPGPU_STATUS_OK || size == 0) return st;
        return enqueue_result(a.s, from_sm100(sm100_memcpy_d2d(a.s->cuda, static_cast<char *>(a.b->ptr) + dst_offset, static_cast<char *>(b.b->ptr) + src_offset, size,
                                                              blocking)));
    });
}

scrapgpu_status v_buffer_fill(scrapgpu_stream_t * stream, scrapgpu_buffer_t * buffer, uint64_t offset, size_t size, uint8_t byte, int blocking) {
    return guard([&]() -> scrapgpu_status {
        Io io;
        const scrapgpu_status st = io_check(stream, buffer, offset, size, "fill exceeds the buffer", io);
        if (st != SCRAPGPU_STATUS_OK || size == 0) return st;
        return enqueue_result(io.s, from_sm100(sm100_memset(io.s->cuda, static_cast<char *>(io.b->ptr) + offset, byte, size, blocking)));
    });
}

// ---------------------------------------------------------------------------------------------------------
// vtable: streams
// ---------------------------------------------------------------------------------------------------------

scrapgpu_status v_stream_create(scrapgpu_device_t * device, scrapgpu_stream_t ** out_stream) {
    return guard([&]() -> scrapgpu_status {
        Device * d = as_device(device);
        if (d == nullptr || out_stream == nullptr) return invalid("device or out_stream is null");
        *out_stream = nullptr;
        auto s = std::make_unique<Stream>();
        s->hdr.backend = &g_vtable;
        s->dev = d;
        const scrapgpu_status st = from_sm100(sm100_stream_create(d->ordinal, &s->cuda));
        if (st != SCRAPGPU_STATUS_OK) return st;
        *out_stream = reinterpret_cast<scrapgpu_stream_t *>(s.release());
        return SCRAPGPU_STATUS_OK;
    });
}

scrapgpu_status v_stream_free(scrapgpu_stream_t * stream) {
    return guard([&]() -> scrapgpu_status {
        Stream * s = as_stream(stream);
        if (s == nullptr) return invalid("not a cuda_sm100 stream");
        if (sm100_stream_sync(s->cuda) == 0) prof_collect(s);
        if (!s->prof_stats.empty()) std::fputs(prof_report(s).c_str(), stderr);
        for (const Stream::ProfPending & p : s->prof_pending) { sm100_event_destroy(p.start); sm100_event_destroy(p.stop); }
        for (sm100_event_t e : s->prof_spare) sm100_event_destroy(e);
        const scrapgpu_status st = from_sm100(sm100_stream_destroy(s->dev->ordinal, s->cuda));
        s->hdr.backend = nullptr;
        delete s;
        return st;
    });
}

scrapgpu_status v_stream_sync(scrapgpu_stream_t * stream) {
    return guard([&]() -> scrapgpu_status {
        Stream * s = as_stream(stream);
        if (s == nullptr) return invalid("not a cuda_sm100 stream");
        const scrapgpu_status st = from_sm100(sm100_stream_sync(s->cuda));
        if (st != SCRAPGPU_STATUS_OK) return st;
        s->settled = s->epoch;
        prof_collect(s);
        if (s->sticky != SCRAPGPU_STATUS_OK) {
            const scrapgpu_status sticky = s->sticky;
            set_error(s->sticky_message.empty() ? "an operation enqueued on this stream failed" : s->sticky_message.c_str());
            s->sticky = SCRAPGPU_STATUS_OK;
            return sticky;
        }
        return SCRAPGPU_STATUS_OK;
    });
}

scrapgpu_device_t * v_stream_device(scrapgpu_stream_t * stream) {
    Stream * s = as_stream(stream);
    return s == nullptr ? nullptr : reinterpret_cast<scrapgpu_device_t *>(s->dev);
}

// ---------------------------------------------------------------------------------------------------------
// vtable: tensor transfers
// ---------------------------------------------------------------------------------------------------------

scrapgpu_status transfer(scrapgpu_stream_t * stream, const scrapgpu_tensor_desc * raw, void * host, size_t size, bool to_device) {
    Stream * s = as_stream(stream);
    if (s == nullptr || raw == nullptr) return invalid("stream or tensor desc is null");
    if (raw->struct_size < offsetof(scrapgpu_tensor_desc, offset) + sizeof(raw->offset)) return invalid("tensor desc is too small");
    const scrapgpu_tensor_desc td = load_desc(*raw);
    Buffer * b = as_buffer(td.buffer);
    if (b == nullptr) return invalid("tensor desc has no cuda_sm100 buffer");
    if (b->dev != s->dev) return invalid("tensor buffer and stream belong to different devices");
    if (td.offset > (uint64_t) b->size || size > b->size - (size_t) td.offset) return invalid("transfer exceeds the buffer");
    if (size > span_bytes(td)) return invalid("transfer size exceeds the tensor");
    if (size == 0) return SCRAPGPU_STATUS_OK;
    if (host == nullptr) return invalid("host pointer is null");
    if (!contiguous(td)) return unsupported("tensor is not contiguous; use buffer_read / buffer_write for raw strided transfers");
    scrapgpu_status st = from_sm100(sm100_set_device(s->dev->ordinal));
    if (st != SCRAPGPU_STATUS_OK) return st;
    char * dev_ptr = static_cast<char *>(b->ptr) + td.offset;
    if (td.layout == SCRAPGPU_LAYOUT_NATURAL) {
        return enqueue_result(s, from_sm100(to_device ? sm100_memcpy_h2d(s->cuda, dev_ptr, host, size, 1) : sm100_memcpy_d2h(s->cuda, host, dev_ptr, size, 1)));
    }
    if (td.layout != SCRAPGPU_LAYOUT_R32) return unsupported("unknown tensor layout");
    // backend-packed: the host side is natural bytes, the device side the plane layout (whole blocks only)
    if (!is_quant(td.dtype)) return unsupported("only quantized tensors have a backend-packed layout");
    if (ne(td, 2) * ne(td, 3) != 1) return unsupported("a backend-packed tensor must be 2-D");
    if (td.offset % 32 != 0) return unsupported("a backend-packed tensor must start on a 32-byte boundary of its buffer");
    const size_t bb = type_size(td.dtype);
    if (size % bb != 0) return unsupported("a transfer of a backend-packed tensor must cover whole blocks");
    if (span_bytes(td) > (uint64_t) b->size - td.offset) return invalid("tensor exceeds its buffer");
    void * staging = nullptr;
    st = from_sm100(sm100_malloc(s->dev->ordinal, size, &staging));
    if (st != SCRAPGPU_STATUS_OK) return st;
    const int64_t blocks = (int64_t) (size / bb);
    if (to_device) {
        st = from_sm100(sm100_memcpy_h2d(s->cuda, staging, host, size, 0));
        if (st == SCRAPGPU_STATUS_OK) st = from_sm100(sm100_pack_device_range(s->cuda, td.dtype, td.ne[0], td.ne[1], 0, blocks, staging, dev_ptr, 1));
        if (st == SCRAPGPU_STATUS_OK) st = from_sm100(sm100_stream_sync(s->cuda));
    } else {
        st = from_sm100(sm100_pack_device_range(s->cuda, td.dtype, td.ne[0], td.ne[1], 0, blocks, staging, dev_ptr, 0));
        if (st == SCRAPGPU_STATUS_OK) st = from_sm100(sm100_memcpy_d2h(s->cuda, host, staging, size, 1));
    }
    sm100_free(s->dev->ordinal, staging);
    return enqueue_result(s, st);
}

scrapgpu_status v_tensor_upload(scrapgpu_stream_t * stream, const scrapgpu_tensor_desc * desc, const void * host, size_t size) {
    return guard([&]() -> scrapgpu_status { return transfer(stream, desc, const_cast<void *>(host), size, true); });
}

scrapgpu_status v_tensor_download(scrapgpu_stream_t * stream, const scrapgpu_tensor_desc * desc, void * host, size_t size) {
    return guard([&]() -> scrapgpu_status { return transfer(stream, desc, host, size, false); });
}

// ---------------------------------------------------------------------------------------------------------
// vtable: ops and plans
// ---------------------------------------------------------------------------------------------------------

scrapgpu_status v_op_supported(scrapgpu_device_t * device, const scrapgpu_op_desc * desc, const char ** reason) {
    if (as_device(device) == nullptr) {
        if (reason != nullptr) *reason = "not a cuda_sm100 device";
        return invalid("not a cuda_sm100 device");
    }
    return guard([&]() -> scrapgpu_status { return supports(desc, reason); });
}

scrapgpu_status v_op_execute(scrapgpu_stream_t * stream, const scrapgpu_op_desc * desc) {
    return guard([&]() -> scrapgpu_status {
        Stream * s = as_stream(stream);
        if (s == nullptr) return invalid("not a cuda_sm100 stream");
        if (desc == nullptr) return invalid("op desc is null");
        return enqueue_result(s, execute(s, desc));
    });
}

const char * op_name(int op) {
    switch (op) {
        case SCRAPGPU_OP_ADD: return "ADD";
        case SCRAPGPU_OP_MUL: return "MUL";
        case SCRAPGPU_OP_GLU: return "GLU";
        case SCRAPGPU_OP_RMS_NORM: return "RMS_NORM";
        case SCRAPGPU_OP_ROPE: return "ROPE";
        case SCRAPGPU_OP_SOFT_MAX: return "SOFT_MAX";
        case SCRAPGPU_OP_GET_ROWS: return "GET_ROWS";
        case SCRAPGPU_OP_SET_ROWS: return "SET_ROWS";
        case SCRAPGPU_OP_CPY: return "CPY";
        case SCRAPGPU_OP_MUL_MAT: return "MUL_MAT";
        case SCRAPGPU_OP_TOP_K: return "TOP_K";
        case SCRAPGPU_OP_RMS_NORM_MUL: return "RMS_NORM_MUL";
        case SCRAPGPU_OP_ADD_RMS_NORM_MUL: return "ADD_RMS_NORM_MUL";
        case SCRAPGPU_OP_MUL_MAT_MULTI: return "MUL_MAT_MULTI";
        case SCRAPGPU_OP_SET_ROWS_PAIR: return "SET_ROWS_PAIR";
        case SCRAPGPU_OP_CONT_MUL_MAT: return "CONT_MUL_MAT";
        default: return "OP";
    }
}

// ---------------------------------------------------------------------------------------------------------
// plans: "selection happens once at plan build, launches are cheap afterwards" (docs/API_CONTRACT.md:79-92 of the
// reference).  plan_build copies the caller's nodes, then looks at neighbouring nodes the way the reference's ggml
// adapter does per graph (adapters/ggml/ggml-cl11.cpp:904-1031): RMS_NORM + MUL, ADD + RMS_NORM + MUL, MUL_MATs that
// share src1, pairs of SET_ROWS become the public fused ops (include/scrapgpu/op.h:43-46); on top of that a
// normalisation or a split SwiGLU whose row feeds packed Q4_K MUL_MATs goes into the matvec launch itself
// (sm100_mul_mat_fused).  An intermediate result is left unwritten only when the caller's output_use_count
// (include/scrapgpu/backend.h:10-14) says that the next node is its single consumer.  plan_execute runs the steps
// one by one the first time and replays a captured CUDA graph from the third time on.
// ---------------------------------------------------------------------------------------------------------

bool same_tensor(const scrapgpu_tensor_desc & a, const scrapgpu_tensor_desc & b) {
    if (a.buffer != b.buffer || a.offset != b.offset || a.dtype != b.dtype || a.layout != b.layout) return false;
    for (int i = 0; i < 4; ++i) if (ne(a, i) != ne(b, i) || (ne(a, i) > 1 && a.nb[i] != b.nb[i])) return false;
    return a.nb[0] == b.nb[0];
}

bool single_row(const scrapgpu_tensor_desc & t) { return f32(t) && t.nb[0] == 4 && ne(t, 1) * ne(t, 2) * ne(t, 3) == 1; }

bool descs_overlap(const scrapgpu_tensor_desc & a, const scrapgpu_tensor_desc & b) {
    if (a.buffer != b.buffer) return false;
    const uint64_t a0 = a.offset, a1 = a0 + span_bytes(a), b0 = b.offset, b1 = b0 + span_bytes(b);
    return a0 < b1 && b0 < a1;
}

PlanNode make_node(scrapgpu_op op, std::vector<scrapgpu_tensor_desc> in, std::vector<scrapgpu_tensor_desc> out, const void * params, size_t params_size,
                   uint32_t use_count) {
    PlanNode n;
    n.desc.op = op;
    n.inputs = std::move(in);
    n.outputs = std::move(out);
    if (params != nullptr && params_size > 0) n.params.assign(static_cast<const uint8_t *>(params), static_cast<const uint8_t *>(params) + params_size);
    n.use_count = use_count;
    n.rebind();
    return n;
}

bool packed_q4k_weight(const scrapgpu_tensor_desc & w) {
    return w.dtype == kQ4_K && w.layout == SCRAPGPU_LAYOUT_R32 && ne(w, 2) * ne(w, 3) == 1 && ne(w, 1) % 16 == 0 && ne(w, 0) % 256 == 0;
}

// an item of the working list while lowering: a node (the caller's or a fused one) and the caller's nodes it covers
struct LowerItem {
    PlanNode node;
    std::vector<size_t> covers;
    bool synthetic = false;     // built here (the caller's nodes stay available as the fallback)
    bool y_count_known = false; // use_count is the consumer count of the row a following MUL_MAT would read
};

void lower_plan(Plan & plan) {
    std::vector<LowerItem> items;
    for (size_t i = 0; i < plan.nodes.size(); ++i) {
        LowerItem it;
        it.node = plan.nodes[i];
        it.covers = {i};
        const auto op = plan.nodes[i].desc.op;
        it.y_count_known = op == SCRAPGPU_OP_RMS_NORM_MUL || op == SCRAPGPU_OP_MUL || op == SCRAPGPU_OP_GLU || op == SCRAPGPU_OP_RMS_NORM;
        items.push_back(std::move(it));
    }
    auto accepted = [](PlanNode & n) {
        const char * why = nullptr;
        return supports(&n.desc, &why) == SCRAPGPU_STATUS_OK;
    };
    auto merge = [&](size_t at, size_t count, PlanNode node, bool y_known) {
        LowerItem m;
        m.node = std::move(node);
        for (size_t k = 0; k < count; ++k) m.covers.insert(m.covers.end(), items[at + k].covers.begin(), items[at + k].covers.end());
        m.synthetic = true;
        m.y_count_known = y_known;
        items.erase(items.begin() + (long) at, items.begin() + (long) (at + count));
        items.insert(items.begin() + (long) at, std::move(m));
    };

    // 1. RMS_NORM -> MUL by a weight row  =>  RMS_NORM_MUL (the normalised, unweighted row is not written: one consumer only)
    for (size_t i = 0; i + 1 < items.size(); ++i) {
        const PlanNode & a = items[i].node, & b = items[i + 1].node;
        if (a.desc.op != SCRAPGPU_OP_RMS_NORM || b.desc.op != SCRAPGPU_OP_MUL || a.use_count != 1 || b.inputs.size() != 2) continue;
        const scrapgpu_tensor_desc & t = a.outputs[0];
        int wi = -1;
        if (same_tensor(b.inputs[0], t)) wi = 1;
        else if (same_tensor(b.inputs[1], t) && same_shape(b.inputs[1], b.outputs[0])) wi = 0;
        if (wi < 0) continue;
        const scrapgpu_tensor_desc & w = b.inputs[wi];
        if (!f32(w) || w.nb[0] != 4 || ne(w, 0) != ne(t, 0) || ne(w, 1) * ne(w, 2) * ne(w, 3) != 1) continue;
        PlanNode n = make_node(SCRAPGPU_OP_RMS_NORM_MUL, {a.inputs[0], w}, {b.outputs[0]}, a.desc.params, a.desc.params_size, b.use_count);
        if (!accepted(n)) continue;
        merge(i, 2, std::move(n), true);
    }
    // 2. ADD -> RMS_NORM_MUL on one row  =>  ADD_RMS_NORM_MUL (the sum is still written: it is the new residual)
    for (size_t i = 0; i + 1 < items.size(); ++i) {
        const PlanNode & a = items[i].node, & b = items[i + 1].node;
        if (a.desc.op != SCRAPGPU_OP_ADD || b.desc.op != SCRAPGPU_OP_RMS_NORM_MUL || a.inputs.size() != 2) continue;
        if (!same_tensor(b.inputs[0], a.outputs[0]) || !single_row(a.outputs[0]) || !same_shape(a.inputs[0], a.inputs[1])) continue;
        PlanNode n = make_node(SCRAPGPU_OP_ADD_RMS_NORM_MUL, {a.inputs[0], a.inputs[1], b.inputs[1]}, {a.outputs[0], b.outputs[0]}, b.desc.params,
                               b.desc.params_size, b.use_count);
        if (!accepted(n)) continue;
        merge(i, 2, std::move(n), items[i + 1].y_count_known);
    }
    // 3. neighbouring MUL_MATs over the same single activation column  =>  MUL_MAT_MULTI (2 or 3 of them)
    for (size_t i = 0; i + 1 < items.size(); ++i) {
        if (items[i].node.desc.op != SCRAPGPU_OP_MUL_MAT) continue;
        const scrapgpu_tensor_desc & x = items[i].node.inputs[1];
        if (ne(x, 1) * ne(x, 2) * ne(x, 3) != 1) continue;
        size_t run = 1;
        while (run < 3 && i + run < items.size() && items[i + run].node.desc.op == SCRAPGPU_OP_MUL_MAT && same_tensor(items[i + run].node.inputs[1], x)) ++run;
        if (run < 2) continue;
        // no member may write what a later member reads (they run as one launch)
        bool independent = true;
        for (size_t k = 0; k < run && independent; ++k)
            for (size_t m = 0; m < run; ++m)
                if (descs_overlap(items[i + k].node.outputs[0], x) || (m != k && descs_overlap(items[i + k].node.outputs[0], items[i + m].node.inputs[0]))) independent = false;
        if (!independent) continue;
        std::vector<scrapgpu_tensor_desc> in, out;
        for (size_t k = 0; k < run; ++k) { in.push_back(items[i + k].node.inputs[0]); out.push_back(items[i + k].node.outputs[0]); }
        in.push_back(x);
        PlanNode n = make_node(SCRAPGPU_OP_MUL_MAT_MULTI, std::move(in), std::move(out), nullptr, 0, 0);
        if (!accepted(n)) continue;
        merge(i, run, std::move(n), false);
    }
    // 4. two neighbouring SET_ROWS (the K and the V row of a token)  =>  SET_ROWS_PAIR
    for (size_t i = 0; i + 1 < items.size(); ++i) {
        const PlanNode & a = items[i].node, & b = items[i + 1].node;
        if (a.desc.op != SCRAPGPU_OP_SET_ROWS || b.desc.op != SCRAPGPU_OP_SET_ROWS) continue;
        if (descs_overlap(a.outputs[0], b.inputs[0]) || descs_overlap(a.outputs[0], b.inputs[1]) || descs_overlap(a.outputs[0], b.outputs[0])) continue;
        PlanNode n = make_node(SCRAPGPU_OP_SET_ROWS_PAIR, {a.inputs[0], a.inputs[1], b.inputs[0], b.inputs[1]}, {a.outputs[0], b.outputs[0]}, a.desc.params,
                               a.desc.params_size, 0);
        if (!accepted(n)) continue;
        merge(i, 2, std::move(n), false);
    }

    // 5. steps: a normalisation / split SwiGLU followed by the packed Q4_K MUL_MAT(s) that read its row goes into one launch
    for (size_t i = 0; i < items.size(); ++i) {
        PlanStep step;
        step.nodes = items[i].covers;
        const PlanNode & a = items[i].node;
        bool fused_away = false, glu_joined = false;
        if (i + 1 < items.size()) {
            const PlanNode & b = items[i + 1].node;
            const bool mm = b.desc.op == SCRAPGPU_OP_MUL_MAT || b.desc.op == SCRAPGPU_OP_MUL_MAT_MULTI;
            const size_t nw = mm ? b.outputs.size() : 0;
            const scrapgpu_tensor_desc * x = mm ? &b.inputs[nw] : nullptr;
            bool weights_ok = mm;
            for (size_t k = 0; k < nw && weights_ok; ++k) weights_ok = packed_q4k_weight(b.inputs[k]) && dense_rows(b.outputs[k]);
            FusedCall f;
            bool ok = false;
            if (weights_ok && (a.desc.op == SCRAPGPU_OP_RMS_NORM_MUL || a.desc.op == SCRAPGPU_OP_ADD_RMS_NORM_MUL)) {
                const bool add = a.desc.op == SCRAPGPU_OP_ADD_RMS_NORM_MUL;
                const scrapgpu_tensor_desc & y = a.outputs[add ? 1 : 0];
                if (same_tensor(*x, y) && single_row(y) && ne(y, 0) <= 8192 && single_row(a.inputs[0])) {
                    f.prologue = SM100_PROLOGUE_RMS_NORM;
                    f.a = a.inputs[0];
                    f.has_b = add;
                    if (add) f.b = a.inputs[1];
                    f.norm_w = a.inputs[add ? 2 : 1];
                    f.has_sum = add;
                    if (add) f.sum_out = a.outputs[0];
                    f.eps = load_params<scrapgpu_rms_norm_params>(&a.desc).eps;
                    // the normalised row itself is written unless the caller said that these MUL_MATs are its only reader
                    f.has_x = !(items[i].y_count_known && a.use_count == (uint32_t) nw);
                    f.x_out = y;
                    ok = !descs_overlap(y, f.a) && (!add || (!descs_overlap(y, f.b) && !descs_overlap(f.sum_out, f.a) && !descs_overlap(f.sum_out, f.b)));
                }
            } else if (weights_ok && nw == 1 && a.desc.op == SCRAPGPU_OP_GLU && a.inputs.size() == 2 && a.use_count == 1) {
                const auto gp = load_params<scrapgpu_glu_params>(&a.desc);
                if (gp.kind == SCRAPGPU_GLU_SWIGLU && same_tensor(*x, a.outputs[0]) && single_row(a.outputs[0]) && single_row(a.inputs[0]) && single_row(a.inputs[1])) {
                    f.prologue = SM100_PROLOGUE_SWIGLU;
                    f.a = a.inputs[0];
                    f.b = a.inputs[1];
                    f.has_b = true;
                    ok = true;
                }
            }
            if (ok) {
                for (size_t k = 0; k < nw; ++k) {
                    f.w.push_back(b.inputs[k]);
                    f.y.push_back(b.outputs[k]);
                    if (descs_overlap(b.outputs[k], f.a) || (f.has_b && descs_overlap(b.outputs[k], f.b))) ok = false;
                }
            }
            // ... and a split SwiGLU over exactly these two projections joins the launch as its epilogue
            if (ok && f.prologue == SM100_PROLOGUE_RMS_NORM && nw == 2 && i + 2 < items.size()) {
                const PlanNode & gn = items[i + 2].node;
                if (gn.desc.op == SCRAPGPU_OP_GLU && gn.inputs.size() == 2 && load_params<scrapgpu_glu_params>(&gn.desc).kind == SCRAPGPU_GLU_SWIGLU) {
                    const scrapgpu_tensor_desc & act = gn.outputs[0];
                    bool clear = same_tensor(gn.inputs[0], b.outputs[0]) && same_tensor(gn.inputs[1], b.outputs[1]) && single_row(act) &&
                                 ne(b.inputs[0], 1) == ne(b.inputs[1], 1) && !descs_overlap(act, f.a) && !descs_overlap(act, b.outputs[0]) &&
                                 !descs_overlap(act, b.outputs[1]);
                    if (f.has_b) clear = clear && !descs_overlap(act, f.b);
                    if (f.has_sum) clear = clear && !descs_overlap(act, f.sum_out);
                    if (f.has_x) clear = clear && !descs_overlap(act, f.x_out);
                    if (clear) {
                        f.has_glu = true;
                        f.glu_out = act;
                    }
                }
            }
            if (ok) {
                step.nodes.insert(step.nodes.end(), items[i + 1].covers.begin(), items[i + 1].covers.end());
                if (f.has_glu) {
                    step.nodes.insert(step.nodes.end(), items[i + 2].covers.begin(), items[i + 2].covers.end());
                    glu_joined = true;
                }
                step.fused = (int) plan.fused.size();
                plan.fused.push_back(std::move(f));
                fused_away = true;
            }
        }
        if (!fused_away && items[i].synthetic) {
            step.lowered = (int) plan.lowered.size();
            plan.lowered.push_back(items[i].node);
        }
        plan.steps.push_back(std::move(step));
        if (fused_away) i += glu_joined ? 2 : 1;
    }
}

scrapgpu_status run_fused(Stream * s, const FusedCall & f) {
    Ref a, b, nw, so, xo;
    scrapgpu_status st = resolve(s, f.a, a);
    if (st == SCRAPGPU_STATUS_OK && f.has_b) st = resolve(s, f.b, b);
    if (st == SCRAPGPU_STATUS_OK && f.prologue == SM100_PROLOGUE_RMS_NORM) st = resolve(s, f.norm_w, nw);
    if (st == SCRAPGPU_STATUS_OK && f.has_sum) st = resolve(s, f.sum_out, so);
    if (st == SCRAPGPU_STATUS_OK && f.has_x) st = resolve(s, f.x_out, xo);
    if (st != SCRAPGPU_STATUS_OK) return st;
    const size_t n = f.w.size();
    int dtypes[3], layouts[3];
    const void * ws[3];
    int64_t ns[3];
    float * ys[3];
    for (size_t i = 0; i < n; ++i) {
        Ref w, y;
        if ((st = resolve(s, f.w[i], w)) != SCRAPGPU_STATUS_OK || (st = resolve(s, f.y[i], y)) != SCRAPGPU_STATUS_OK) return st;
        dtypes[i] = w.d.dtype;
        layouts[i] = 1;
        ws[i] = w.base();
        ns[i] = ne(w.d, 1);
        ys[i] = (float *) y.base();
    }
    if ((st = from_sm100(sm100_set_device(s->dev->ordinal))) != SCRAPGPU_STATUS_OK) return st;
    bool serial = false;
    for (size_t i = 0; i < n; ++i) serial = serial || fresh(s, f.w[i]);
    std::unique_ptr<ProfScope> prof;
    if (profiling()) {
        double bytes = 0;
        for (size_t i = 0; i < n; ++i) bytes += weight_bytes(load_desc(f.w[i]));
        prof.reset(new ProfScope(s, std::string(f.prologue == SM100_PROLOGUE_RMS_NORM ? "RMS_NORM_MUL" : "GLU") + " + MUL_MAT " + dtype_name(dtypes[0]) + " packed mv x" + std::to_string(n), bytes));
    }
    Ref go;
    if (f.has_glu && (st = resolve(s, f.glu_out, go)) != SCRAPGPU_STATUS_OK) return st;
    if (f.has_glu) {
        Serialized scope(serial);
        st = from_sm100(sm100_mul_mat_glu(s->cuda, f.prologue, (const float *) a.base(), f.has_b ? (const float *) b.base() : nullptr, (const float *) nw.base(), f.eps,
                                          f.has_sum ? (float *) so.base() : nullptr, f.has_x ? (float *) xo.base() : nullptr, dtypes[0], 1, ws[0], ws[1],
                                          ne(f.a, 0), ns[0], ys[0], ys[1], (float *) go.base()));
    } else {
        Serialized scope(serial);
        st = from_sm100(sm100_mul_mat_fused(s->cuda, f.prologue, (const float *) a.base(), f.has_b ? (const float *) b.base() : nullptr,
                                            f.prologue == SM100_PROLOGUE_RMS_NORM ? (const float *) nw.base() : nullptr, f.eps,
                                            f.has_sum ? (float *) so.base() : nullptr, f.has_x ? (float *) xo.base() : nullptr, (int) n, dtypes, layouts,
                                            ws, ne(f.a, 0), ns, ys));
    }
    prof.reset();
    if (st == SCRAPGPU_STATUS_OK) {
        ++s->epoch;
        for (size_t i = 0; i < n; ++i) wrote(s, f.y[i]);
        if (f.has_sum) wrote(s, f.sum_out);
        if (f.has_x) wrote(s, f.x_out);
        if (f.has_glu) wrote(s, f.glu_out);
    }
    return st;
}

// runs the plan's steps in order on the stream (directly, or into a capture)
scrapgpu_status run_steps(Stream * s, Plan * plan) {
    for (PlanStep & step : plan->steps) {
        scrapgpu_status st = SCRAPGPU_STATUS_UNSUPPORTED;
        if (!step.declined && step.fused >= 0) st = run_fused(s, plan->fused[(size_t) step.fused]);
        else if (!step.declined && step.lowered >= 0) st = execute(s, &plan->lowered[(size_t) step.lowered].desc);
        if ((step.fused >= 0 || step.lowered >= 0) && !step.declined) {
            if (st == SCRAPGPU_STATUS_OK) continue;
            // refused before anything was launched (a shape the fused kernel does not serve, an aliasing the fused form
            // cannot honour): the caller's own nodes, each of which was accepted at build time, run from now on
            if (st != SCRAPGPU_STATUS_UNSUPPORTED && st != SCRAPGPU_STATUS_INVALID_ARGUMENT) return enqueue_result(s, st);
            step.declined = true;
        }
        for (size_t i : step.nodes) {
            st = enqueue_result(s, execute(s, &plan->nodes[i].desc));
            if (st != SCRAPGPU_STATUS_OK) return st;
        }
    }
    return SCRAPGPU_STATUS_OK;
}

scrapgpu_status v_plan_build(scrapgpu_device_t * device, const scrapgpu_plan_desc * desc, scrapgpu_plan_t ** out_plan) {
    return guard([&]() -> scrapgpu_status {
        Device * d = as_device(device);
        if (d == nullptr || desc == nullptr || out_plan == nullptr || desc->struct_size < offsetof(scrapgpu_plan_desc, node_count) + sizeof(desc->node_count) ||
            desc->node_count > 4096 || (desc->node_count > 0 && desc->nodes == nullptr))
            return invalid("device, plan desc or node list is invalid");
        *out_plan = nullptr;
        auto plan = std::make_unique<Plan>();
        plan->hdr.backend = &g_vtable;
        plan->dev = d;
        plan->nodes.resize(desc->node_count);
        for (size_t i = 0; i < desc->node_count; ++i) {
            const scrapgpu_plan_node & src = desc->nodes[i];
            if (src.struct_size < offsetof(scrapgpu_plan_node, op) + sizeof(src.op)) return invalid("plan node is too small");
            const char * why = nullptr;
            const scrapgpu_status st = supports(&src.op, &why);  // a plan fails to build rather than midway through execution
            if (st != SCRAPGPU_STATUS_OK) {
                char buf[256];
                std::snprintf(buf, sizeof(buf), "plan node %zu (%s): %s", i, op_name((int) src.op.op), why != nullptr ? why : "not supported");
                set_error(buf);
                return st;
            }
            PlanNode & n = plan->nodes[i];
            n.desc = src.op;
            for (size_t j = 0; j < src.op.input_count; ++j) n.inputs.push_back(load_desc(src.op.inputs[j]));
            for (size_t j = 0; j < src.op.output_count; ++j) n.outputs.push_back(load_desc(src.op.outputs[j]));
            if (src.op.params != nullptr && src.op.params_size > 0) {
                const uint8_t * p = static_cast<const uint8_t *>(src.op.params);
                n.params.assign(p, p + src.op.params_size);
            }
            n.use_count = src.struct_size >= offsetof(scrapgpu_plan_node, output_use_count) + sizeof(src.output_use_count) ? src.output_use_count : 0;
            n.rebind();
            // descriptor pointers inside the params must point at the plan's own copies
            if (src.op.op == SCRAPGPU_OP_ROPE && n.params.size() >= sizeof(scrapgpu_rope_params)) {
                auto * p = reinterpret_cast<scrapgpu_rope_params *>(n.params.data());
                p->freq_factors = p->freq_factors != nullptr && n.inputs.size() > 2 ? &n.inputs[2] : nullptr;
                p->n_offs = p->n_offs != nullptr && n.inputs.size() > 3 ? &n.inputs[3] : nullptr;
            }
            if (src.op.op == SCRAPGPU_OP_SOFT_MAX && n.params.size() >= sizeof(scrapgpu_soft_max_params)) {
                auto * p = reinterpret_cast<scrapgpu_soft_max_params *>(n.params.data());
                p->mask = p->mask != nullptr && n.inputs.size() > 1 ? &n.inputs[1] : nullptr;
            }
            for (const auto & t : n.inputs) if (Buffer * rb = as_buffer(t.buffer)) plan->pinned.push_back(rb);
            for (const auto & t : n.outputs) if (Buffer * rb = as_buffer(t.buffer)) plan->pinned.push_back(rb);
        }
        static const bool fuse = [] { const char * e = std::getenv("SCRAPGPU_SM100_PLAN_FUSION"); return e == nullptr || std::atoi(e) != 0; }();
        if (fuse) {
            lower_plan(*plan);
        } else {
            for (size_t i = 0; i < plan->nodes.size(); ++i) {
                PlanStep st;
                st.nodes = {i};
                plan->steps.push_back(std::move(st));
            }
        }
        {
            std::lock_guard<std::mutex> lock(g_pin_mutex);
            for (Buffer * rb : plan->pinned) ++g_pins[rb];
        }
        *out_plan = reinterpret_cast<scrapgpu_plan_t *>(plan.release());
        return SCRAPGPU_STATUS_OK;
    });
}

scrapgpu_status v_plan_execute(scrapgpu_stream_t * stream, scrapgpu_plan_t * plan_) {
    return guard([&]() -> scrapgpu_status {
        Stream * s = as_stream(stream);
        Plan * plan = as_plan(plan_);
        if (s == nullptr || plan == nullptr) return invalid("stream or plan is not a cuda_sm100 object");
        if (plan->dev != s->dev) return invalid("plan and stream belong to different devices");
        static const bool graphs = [] { const char * e = std::getenv("SCRAPGPU_SM100_PLAN_GRAPH"); return e == nullptr || std::atoi(e) != 0; }();
        const uint64_t run = plan->executions++;
        scrapgpu_status st = from_sm100(sm100_set_device(s->dev->ordinal));
        if (st != SCRAPGPU_STATUS_OK) return st;
        if (plan->graph != nullptr) {
            // a graph launch starts after everything enqueued before it and ends before anything enqueued after it
            st = enqueue_result(s, from_sm100(sm100_graph_launch(plan->graph, s->cuda)));
            s->settled = ++s->epoch;
            return st;
        }
        // first execution: step by step (scratch buffers, ROPE tables and fused-or-not decisions settle here);
        // second: the same steps recorded into a graph, which is then launched; a plan of one launch gains nothing
        if (!graphs || profiling() || plan->graph_refused || run == 0 || plan->launches_per_execution < 2) {
            const uint64_t before = sm100_launch_count();
            st = run_steps(s, plan);
            plan->launches_per_execution = (size_t) (sm100_launch_count() - before);
            return st;
        }
        st = from_sm100(sm100_graph_begin(s->cuda));
        if (st != SCRAPGPU_STATUS_OK) {   // e.g. the caller is capturing this stream itself: just enqueue
            plan->graph_refused = true;
            return run_steps(s, plan);
        }
        const scrapgpu_status recorded = run_steps(s, plan);
        sm100_graph_t g = nullptr;
        const scrapgpu_status ended = from_sm100(sm100_graph_end(s->cuda, &g));
        if (recorded != SCRAPGPU_STATUS_OK || ended != SCRAPGPU_STATUS_OK) {
            if (g != nullptr) sm100_graph_destroy(g);
            plan->graph_refused = true;   // nothing was executed by the failed recording: run the steps directly
            s->sticky = SCRAPGPU_STATUS_OK;
            return run_steps(s, plan);
        }
        plan->graph = g;
        st = enqueue_result(s, from_sm100(sm100_graph_launch(plan->graph, s->cuda)));
        s->settled = ++s->epoch;
        return st;
    });
}

scrapgpu_status v_plan_free(scrapgpu_plan_t * plan_) {
    return guard([&]() -> scrapgpu_status {
        Plan * plan = as_plan(plan_);
        if (plan == nullptr) return invalid("not a cuda_sm100 plan");
        {
            std::lock_guard<std::mutex> lock(g_pin_mutex);
            for (Buffer * rb : plan->pinned) {
                auto it = g_pins.find(rb);
                if (it != g_pins.end() && --it->second == 0) g_pins.erase(it);
            }
        }
        if (plan->graph != nullptr) sm100_graph_destroy(plan->graph);
        plan->hdr.backend = nullptr;
        delete plan;
        return SCRAPGPU_STATUS_OK;
    });
}

const scrapgpu_backend_vtable g_vtable = {
    /* struct_size      */ sizeof(scrapgpu_backend_vtable),
    /* name             */ "cuda_sm100",
    /* userdata         */ nullptr,
    /* get_device_count */ v_get_device_count,
    /* get_device       */ v_get_device,
    /* device_get_info  */ v_device_get_info,
    /* buffer_alloc     */ v_buffer_alloc,
    /* buffer_free      */ v_buffer_free,
    /* buffer_write     */ v_buffer_write,
    /* buffer_read      */ v_buffer_read,
    /* buffer_copy      */ v_buffer_copy,
    /* buffer_fill      */ v_buffer_fill,
    /* stream_sync      */ v_stream_sync,
    /* op_supported     */ v_op_supported,
    /* plan_build       */ v_plan_build,
    /* plan_execute     */ v_plan_execute,
    /* plan_free        */ v_plan_free,
    /* stream_create    */ v_stream_create,
    /* stream_free      */ v_stream_free,
    /* tensor_upload    */ v_tensor_upload,
    /* tensor_download  */ v_tensor_download,
    /* op_execute       */ v_op_execute,
    /* stream_device    */ v_stream_device,
};

// ---------------------------------------------------------------------------------------------------------
// fused attention entry
// ---------------------------------------------------------------------------------------------------------

bool strict_contiguous(const scrapgpu_tensor_desc & t) {
    uint64_t next = 4;
    for (int i = 0; i < 4; ++i) {
        if (t.nb[i] != next) return false;
        next *= (uint64_t) ne(t, i);
    }
    return true;
}

scrapgpu_status attention(scrapgpu_device_t * device, scrapgpu_stream_t * stream, const scrapgpu_attention_params * params, const scrapgpu_tensor_desc * position) {
    Device * d = as_device(device);
    Stream * s = as_stream(stream);
    if (d == nullptr || s == nullptr) return invalid("device or stream is not a cuda_sm100 object");
    if (s->dev != d) return invalid("stream and device differ");
    if (params == nullptr || params->struct_size < sizeof(scrapgpu_attention_params)) return invalid("attention params are missing or too small");
    if (params->query == nullptr || params->key == nullptr || params->value == nullptr || params->output == nullptr) return invalid("attention needs query, key, value and output");
    if (!std::isfinite(params->scale)) return invalid("attention scale must be finite");
    Ref q, k, v, o, m, pos;
    scrapgpu_status st;
    if ((st = resolve(s, *params->query, q)) != SCRAPGPU_STATUS_OK) return st;
    if ((st = resolve(s, *params->key, k)) != SCRAPGPU_STATUS_OK) return st;
    if ((st = resolve(s, *params->value, v)) != SCRAPGPU_STATUS_OK) return st;
    if ((st = resolve(s, *params->output, o)) != SCRAPGPU_STATUS_OK) return st;
    const bool has_mask = params->mask != nullptr;
    if (has_mask && (st = resolve(s, *params->mask, m)) != SCRAPGPU_STATUS_OK) return st;
    if (position != nullptr) {
        if ((st = resolve(s, *position, pos)) != SCRAPGPU_STATUS_OK) return st;
        if (pos.d.dtype != SCRAPGPU_DTYPE_I32) return unsupported("the attention position tensor must be I32");
    }
    for (const Ref * r : {&q, &k, &v, &o}) {
        if (!f32(r->d) || r->d.layout != SCRAPGPU_LAYOUT_NATURAL) return unsupported("attention tensors must be F32 in the natural layout");
        if (!strict_contiguous(r->d)) return unsupported("attention tensors must be contiguous");
    }
    const int64_t D = ne(q.d, 0), Q = ne(q.d, 1), Hq = ne(q.d, 2), B = ne(q.d, 3);
    const int64_t Kn = ne(k.d, 1), Hkv = ne(k.d, 2), Dv = ne(v.d, 0);
    if (ne(k.d, 0) != D || ne(k.d, 3) != B || ne(v.d, 1) != Kn || ne(v.d, 2) != Hkv || ne(v.d, 3) != B) return invalid("attention: key/value shapes do not match the query");
    if (ne(o.d, 0) != Dv || ne(o.d, 1) != Q || ne(o.d, 2) != Hq || ne(o.d, 3) != B) return invalid("attention: output must be [Dv, Q, Hq, B]");
    if (Hkv <= 0 || Hq % Hkv != 0) return invalid("attention: Hq must be divisible by Hkv");
    int64_t mask_heads = 1, mask_batches = 1;
    if (has_mask) {
        if (!f32(m.d) || !strict_contiguous(m.d)) return unsupported("the attention mask must be contiguous F32");
        if (ne(m.d, 0) != Kn || ne(m.d, 1) != Q || (ne(m.d, 2) != 1 && ne(m.d, 2) != Hq) || (ne(m.d, 3) != 1 && ne(m.d, 3) != B)) return invalid("attention: mask must be [K, Q, 1 or Hq, 1 or B]");
        mask_heads = ne(m.d, 2);
        mask_batches = ne(m.d, 3);
    }
    for (const Ref * r : {&q, &k, &v}) if (overlap(o, *r)) return invalid("attention output overlaps an input");
    if ((st = from_sm100(sm100_set_device(d->ordinal))) != SCRAPGPU_STATUS_OK) return st;
    const uint64_t off = params->query_position_offset > (uint64_t) std::numeric_limits<int64_t>::max() / 2 ? (uint64_t) std::numeric_limits<int64_t>::max() / 2
                                                                                                             : params->query_position_offset;
    for (int64_t b = 0; b < B; ++b) {
        const float * mp = has_mask ? (const float *) (m.base() + (mask_batches == 1 ? 0 : b) * m.d.nb[3]) : nullptr;
        st = from_sm100(sm100_attention(s->cuda, (const float *) (q.base() + b * q.d.nb[3]), (const float *) (k.base() + b * k.d.nb[3]),
                                        (const float *) (v.base() + b * v.d.nb[3]), mp, mask_heads, (float *) (o.base() + b * o.d.nb[3]), D, Dv, Q, Kn, Hq, Hkv,
                                        params->causal != 0, (int64_t) off, position != nullptr ? (const int32_t *) pos.base() : nullptr, params->scale));
        if (st != SCRAPGPU_STATUS_OK) return enqueue_result(s, st);
    }
    return SCRAPGPU_STATUS_OK;
}


// ---------------------------------------------------------------------------------------------------------
// multi-GPU transport and the tensor-parallel device group
// ---------------------------------------------------------------------------------------------------------

struct Group {
    std::vector<Device *> devices;
    std::vector<void *> areas;              // receive area of every device (sm100_allreduce_area_bytes each)
    std::vector<sm100_allreduce_t> ranks;   // the all-reduce context of every device
    size_t capacity = 0;
};

std::mutex g_group_mutex;
std::vector<Group *> g_groups;

Group * as_group(scrapgpu_cuda_sm100_group_t * g) {
    std::lock_guard<std::mutex> lock(g_group_mutex);
    for (Group * known : g_groups) if ((void *) known == (void *) g) return known;
    return nullptr;
}

void destroy_group(Group * g) {
    for (size_t i = 0; i < g->ranks.size(); ++i) if (g->ranks[i] != nullptr) sm100_allreduce_destroy(g->ranks[i]);
    for (size_t i = 0; i < g->areas.size(); ++i) if (g->areas[i] != nullptr) sm100_free(g->devices[i]->ordinal, g->areas[i]);
    delete g;
}

scrapgpu_status tensor_copy(scrapgpu_stream_t * src_stream, const scrapgpu_tensor_desc * src, scrapgpu_stream_t * dst_stream, const scrapgpu_tensor_desc * dst) {
    Stream * ss = as_stream(src_stream);
    Stream * ds = as_stream(dst_stream);
    if (ss == nullptr || ds == nullptr || src == nullptr || dst == nullptr) return invalid("src_stream, dst_stream, src or dst is null or not a cuda_sm100 object");
    if (src->struct_size < sizeof(scrapgpu_tensor_desc) || dst->struct_size < sizeof(scrapgpu_tensor_desc)) return invalid("tensor desc is too small");
    const scrapgpu_tensor_desc s = load_desc(*src), d = load_desc(*dst);
    if (type_size(s.dtype) == 0) return unsupported("unknown tensor dtype");
    if (s.dtype != d.dtype) return unsupported("src and dst dtypes differ");
    for (int i = 0; i < 4; ++i) {
        if (s.ne[i] != d.ne[i]) return unsupported("src and dst shapes differ");
        if (s.ne[i] < 0) return invalid("negative tensor dim");
    }
    if (s.layout == SCRAPGPU_LAYOUT_R32 || d.layout == SCRAPGPU_LAYOUT_R32)
        return unsupported("backend-packed tensors are not allowed: move them through the host with tensor_download / tensor_upload");
    if (!contiguous(s) || !contiguous(d)) return unsupported("tensor is not contiguous; use buffer_read / buffer_write for raw strided transfers");
    Ref rs, rd;
    scrapgpu_status st = resolve(ss, s, rs);
    if (st == SCRAPGPU_STATUS_OK) st = resolve(ds, d, rd);
    if (st != SCRAPGPU_STATUS_OK) return st;
    const uint64_t bytes = span_bytes(s);
    if (bytes == 0) return SCRAPGPU_STATUS_OK;
    if (ss->dev == ds->dev && overlap(rs, rd)) return invalid("src and dst overlap");
    return enqueue_result(ds, from_sm100(sm100_memcpy_peer(ds->cuda, ds->dev->ordinal, rd.base(), ss->cuda, ss->dev->ordinal, rs.base(), (size_t) bytes)));
}

scrapgpu_status shard(const scrapgpu_tensor_desc * full_, int split_dim, size_t rank, size_t world, scrapgpu_tensor_desc * out) {
    if (full_ == nullptr || out == nullptr || full_->struct_size < sizeof(scrapgpu_tensor_desc)) return invalid("tensor desc is null or too small");
    if (world == 0 || rank >= world) return invalid("rank must be below world");
    const scrapgpu_tensor_desc full = load_desc(*full_);
    const size_t bs = block_size(full.dtype), ts = type_size(full.dtype);
    if (bs == 0) return unsupported("unknown tensor dtype");
    if (full.layout != SCRAPGPU_LAYOUT_NATURAL) return unsupported("shards are cut from the natural layout (pack the shard, not the full tensor)");
    if (ne(full, 2) * ne(full, 3) != 1) return unsupported("a 2-D weight tensor is expected");
    if (full.nb[0] != ts) return unsupported("rows must be contiguous");
    scrapgpu_tensor_desc v = full;
    if (split_dim == 1) {
        const int64_t n = ne(full, 1), per = (n + (int64_t) world - 1) / (int64_t) world;
        const int64_t lo = std::min<int64_t>(n, (int64_t) rank * per), cnt = std::max<int64_t>(0, std::min<int64_t>(n, lo + per) - lo);
        v.ne[1] = cnt;
        v.offset = full.offset + (uint64_t) lo * full.nb[1];
    } else if (split_dim == 0) {
        const int64_t k = ne(full, 0);
        if (k % (int64_t) world != 0 || (k / (int64_t) world) % (int64_t) bs != 0) return unsupported("K / world must be a whole number of quantization blocks");
        const int64_t kl = k / (int64_t) world;
        v.ne[0] = kl;
        v.offset = full.offset + (uint64_t) rank * (uint64_t) (kl / (int64_t) bs) * ts;
    } else {
        return invalid("split_dim must be 0 (K) or 1 (rows)");
    }
    *out = v;
    return SCRAPGPU_STATUS_OK;
}

scrapgpu_status upload_view(scrapgpu_stream_t * stream, const scrapgpu_tensor_desc * dst_, const void * host_base, const scrapgpu_tensor_desc * view_) {
    Stream * s = as_stream(stream);
    if (s == nullptr || dst_ == nullptr || view_ == nullptr || host_base == nullptr) return invalid("stream, dst, host_base or src_view is null");
    if (dst_->struct_size < sizeof(scrapgpu_tensor_desc) || view_->struct_size < sizeof(scrapgpu_tensor_desc)) return invalid("tensor desc is too small");
    const scrapgpu_tensor_desc d = load_desc(*dst_), v = load_desc(*view_);
    const size_t bs = block_size(v.dtype), ts = type_size(v.dtype);
    if (bs == 0 || v.dtype != d.dtype) return unsupported("dtypes differ or are unknown");
    for (int i = 0; i < 4; ++i) if (ne(v, i) != ne(d, i)) return unsupported("src view and dst shapes differ");
    if (v.nb[0] != ts || ne(v, 0) % (int64_t) bs != 0 || ne(v, 2) * ne(v, 3) != 1) return unsupported("the view must be 2-D with contiguous rows of whole blocks");
    const size_t row = (size_t) (ne(v, 0) / (int64_t) bs) * ts;
    const size_t rows = (size_t) ne(v, 1);
    std::vector<uint8_t> staging(row * rows);
    const uint8_t * base = static_cast<const uint8_t *>(host_base) + v.offset;
    for (size_t r = 0; r < rows; ++r) std::memcpy(staging.data() + r * row, base + r * v.nb[1], row);
    return transfer(stream, &d, staging.data(), staging.size(), true);
}

}  // namespace

extern "C" {

SCRAPGPU_API const scrapgpu_backend_vtable * scrapgpu_cuda_sm100_vtable(void) { return &g_vtable; }

SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_register(void) {
    return guard([&]() -> scrapgpu_status {
        if (scrapgpu_register_backend == nullptr) return unsupported("the ScrapGpuLibrary core is not loaded: scrapgpu_register_backend is unresolved");
        static std::mutex reg_mutex;
        std::lock_guard<std::mutex> lock(reg_mutex);
        {
            std::lock_guard<std::mutex> lock2(g_registry_mutex);
            probe_devices();
        }
        static bool registered = false;
        if (registered) return SCRAPGPU_STATUS_OK;
        const scrapgpu_status st = scrapgpu_register_backend(&g_vtable);
        registered = st == SCRAPGPU_STATUS_OK;
        return st;
    });
}

SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_attention(scrapgpu_device_t * device, scrapgpu_stream_t * stream, const scrapgpu_attention_params * params) {
    return guard([&]() -> scrapgpu_status { return attention(device, stream, params, nullptr); });
}

SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_attention_at(scrapgpu_device_t * device, scrapgpu_stream_t * stream, const scrapgpu_attention_params * params,
                                                             const scrapgpu_tensor_desc * position) {
    return guard([&]() -> scrapgpu_status {
        if (position == nullptr) return invalid("position tensor is null");
        return attention(device, stream, params, position);
    });
}

SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_tensor_copy(scrapgpu_stream_t * src_stream, const scrapgpu_tensor_desc * src, scrapgpu_stream_t * dst_stream,
                                                            const scrapgpu_tensor_desc * dst) {
    return guard([&]() -> scrapgpu_status { return tensor_copy(src_stream, src, dst_stream, dst); });
}

SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_shard(const scrapgpu_tensor_desc * full, int split_dim, size_t rank, size_t world, scrapgpu_tensor_desc * out_view) {
    return guard([&]() -> scrapgpu_status { return shard(full, split_dim, rank, world, out_view); });
}

SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_upload_view(scrapgpu_stream_t * stream, const scrapgpu_tensor_desc * dst, const void * host_base,
                                                            const scrapgpu_tensor_desc * src_view) {
    return guard([&]() -> scrapgpu_status { return upload_view(stream, dst, host_base, src_view); });
}

SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_group_create(scrapgpu_device_t * const * devices, size_t count, size_t max_elements,
                                                             scrapgpu_cuda_sm100_group_t ** out_group) {
    return guard([&]() -> scrapgpu_status {
        if (devices == nullptr || out_group == nullptr) return invalid("devices or out_group is null");
        *out_group = nullptr;
        if (count < 1 || count > 8) return unsupported("a group has 1 to 8 devices");
        if (max_elements == 0 || max_elements % 4 != 0 || max_elements > (size_t) 1 << 24) return invalid("max_elements must be a positive multiple of 4 (at most 2^24)");
        auto g = std::make_unique<Group>();
        for (size_t i = 0; i < count; ++i) {
            Device * d = as_device(devices[i]);
            if (d == nullptr) return invalid("not a cuda_sm100 device");
            for (Device * seen : g->devices) if (seen == d) return invalid("a device appears twice in the group");
            g->devices.push_back(d);
        }
        g->capacity = max_elements;
        scrapgpu_status st = SCRAPGPU_STATUS_OK;
        for (size_t i = 0; i < count && st == SCRAPGPU_STATUS_OK; ++i)
            for (size_t j = 0; j < count && st == SCRAPGPU_STATUS_OK; ++j)
                if (i != j) st = from_sm100(sm100_peer_access(g->devices[i]->ordinal, g->devices[j]->ordinal));
        const size_t area_bytes = sm100_allreduce_area_bytes((int) count, (int) max_elements);
        g->areas.assign(count, nullptr);
        g->ranks.assign(count, nullptr);
        for (size_t i = 0; i < count && st == SCRAPGPU_STATUS_OK; ++i) {
            st = from_sm100(sm100_malloc(g->devices[i]->ordinal, area_bytes, &g->areas[i]));
            if (st == SCRAPGPU_STATUS_OK) st = from_sm100(sm100_memset(nullptr, g->areas[i], 0, area_bytes, 1));
        }
        for (size_t i = 0; i < count && st == SCRAPGPU_STATUS_OK; ++i) {
            st = from_sm100(sm100_set_device(g->devices[i]->ordinal));
            if (st == SCRAPGPU_STATUS_OK) st = from_sm100(sm100_allreduce_create((int) i, (int) count, (int) max_elements, g->areas.data(), &g->ranks[i]));
        }
        if (st != SCRAPGPU_STATUS_OK) {
            destroy_group(g.release());
            return st;
        }
        Group * raw = g.release();
        {
            std::lock_guard<std::mutex> lock(g_group_mutex);
            g_groups.push_back(raw);
        }
        *out_group = reinterpret_cast<scrapgpu_cuda_sm100_group_t *>(raw);
        return SCRAPGPU_STATUS_OK;
    });
}

SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_group_free(scrapgpu_cuda_sm100_group_t * group) {
    return guard([&]() -> scrapgpu_status {
        Group * g = as_group(group);
        if (g == nullptr) return invalid("not a cuda_sm100 device group");
        {
            std::lock_guard<std::mutex> lock(g_group_mutex);
            g_groups.erase(std::find(g_groups.begin(), g_groups.end(), g));
        }
        destroy_group(g);
        return SCRAPGPU_STATUS_OK;
    });
}

SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_group_all_reduce(scrapgpu_cuda_sm100_group_t * group, scrapgpu_stream_t * const * streams,
                                                                 const scrapgpu_tensor_desc * tensors) {
    return guard([&]() -> scrapgpu_status {
        Group * g = as_group(group);
        if (g == nullptr || streams == nullptr || tensors == nullptr) return invalid("group, streams or tensors is null");
        const size_t n = g->devices.size();
        std::vector<Ref> refs(n);
        std::vector<Stream *> ss(n);
        int64_t count = 0;
        for (size_t i = 0; i < n; ++i) {
            ss[i] = as_stream(streams[i]);
            if (ss[i] == nullptr || ss[i]->dev != g->devices[i]) return invalid("streams[i] must be a stream of the group's device i");
            if (tensors[i].struct_size < sizeof(scrapgpu_tensor_desc)) return invalid("tensor desc is too small");
            const scrapgpu_status st = resolve(ss[i], tensors[i], refs[i]);
            if (st != SCRAPGPU_STATUS_OK) return st;
            int64_t elems = 0;
            if (!f32(refs[i].d) || !contiguous(refs[i].d) || !elements(refs[i].d, elems)) return unsupported("all-reduce tensors must be contiguous F32");
            if (i == 0) count = elems;
            if (elems != count) return invalid("all-reduce tensors must have the same length on every device");
            if (((uintptr_t) refs[i].base() & 15) != 0) return unsupported("all-reduce tensors must be 16-byte aligned");
        }
        if (count <= 0 || count % 4 != 0 || (size_t) count > g->capacity) return invalid("the tensor length must be a positive multiple of 4 within the group's max_elements");
        if (n == 1) return SCRAPGPU_STATUS_OK;   // the sum over one device is the tensor itself
        for (size_t i = 0; i < n; ++i) {
            scrapgpu_status st = from_sm100(sm100_set_device(g->devices[i]->ordinal));
            if (st == SCRAPGPU_STATUS_OK) st = from_sm100(sm100_allreduce_sum(g->ranks[i], ss[i]->cuda, (float *) refs[i].base(), (int) count));
            if (st != SCRAPGPU_STATUS_OK) return enqueue_result(ss[i], st);
        }
        return SCRAPGPU_STATUS_OK;
    });
}

SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_group_mul_mat_all_reduce(scrapgpu_cuda_sm100_group_t * group, scrapgpu_stream_t * const * streams,
                                                                         const scrapgpu_tensor_desc * weights, const scrapgpu_tensor_desc * inputs,
                                                                         const scrapgpu_tensor_desc * outputs) {
    return guard([&]() -> scrapgpu_status {
        Group * g = as_group(group);
        if (g == nullptr || streams == nullptr || weights == nullptr || inputs == nullptr || outputs == nullptr) return invalid("group, streams or tensors is null");
        const size_t n = g->devices.size();
        std::vector<Ref> w(n), x(n), y(n);
        std::vector<Stream *> ss(n);
        int64_t rows = 0;
        for (size_t i = 0; i < n; ++i) {
            ss[i] = as_stream(streams[i]);
            if (ss[i] == nullptr || ss[i]->dev != g->devices[i]) return invalid("streams[i] must be a stream of the group's device i");
            scrapgpu_status st = resolve(ss[i], weights[i], w[i]);
            if (st == SCRAPGPU_STATUS_OK) st = resolve(ss[i], inputs[i], x[i]);
            if (st == SCRAPGPU_STATUS_OK) st = resolve(ss[i], outputs[i], y[i]);
            if (st != SCRAPGPU_STATUS_OK) return st;
            int64_t xe = 0, ye = 0;
            if (!f32(x[i].d) || !contiguous(x[i].d) || !elements(x[i].d, xe) || !f32(y[i].d) || !contiguous(y[i].d) || !elements(y[i].d, ye))
                return unsupported("the activation and result vectors must be contiguous F32");
            if (ne(w[i].d, 2) * ne(w[i].d, 3) != 1 || !is_quant(w[i].d.dtype)) return unsupported("the K shards must be 2-D quantized weight tensors");
            if (xe != ne(w[i].d, 0) || ye != ne(w[i].d, 1)) return invalid("shapes: x has K_i elements, y has N, W_i is [K_i, N]");
            if (i == 0) rows = ye;
            if (ye != rows) return invalid("every device's shard must have the same number of rows");
            if (w[i].d.layout != SCRAPGPU_LAYOUT_R32 && w[i].d.nb[1] != (uint64_t) (ne(w[i].d, 0) / (int64_t) block_size(w[i].d.dtype)) * type_size(w[i].d.dtype))
                return unsupported("natural-layout shards must have contiguous rows");
        }
        if (rows <= 0 || rows % 4 != 0 || (size_t) rows > g->capacity) return invalid("N must be a positive multiple of 4 within the group's max_elements");
        for (size_t i = 0; i < n; ++i) {
            scrapgpu_status st = from_sm100(sm100_set_device(g->devices[i]->ordinal));
            if (st != SCRAPGPU_STATUS_OK) return st;
            Serialized scope(fresh(ss[i], weights[i]));
            if (n == 1) {
                st = from_sm100(sm100_mul_mat(ss[i]->cuda, w[i].d.dtype, w[i].d.layout == SCRAPGPU_LAYOUT_R32 ? 1 : 0, w[i].base(), 0, ne(w[i].d, 0), rows,
                                              (const float *) x[i].base(), ne(w[i].d, 0), 1, (float *) y[i].base(), rows));
            } else {
                st = from_sm100(sm100_mul_mat_allreduce(g->ranks[i], ss[i]->cuda, 0, (const float *) x[i].base(), nullptr, w[i].d.dtype,
                                                        w[i].d.layout == SCRAPGPU_LAYOUT_R32 ? 1 : 0, w[i].base(), ne(w[i].d, 0), rows, (float *) y[i].base()));
            }
            if (st != SCRAPGPU_STATUS_OK) return enqueue_result(ss[i], st);
            ++ss[i]->epoch;
            wrote(ss[i], outputs[i]);
        }
        return SCRAPGPU_STATUS_OK;
    });
}

SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_group_status(scrapgpu_cuda_sm100_group_t * group) {
    return guard([&]() -> scrapgpu_status {
        Group * g = as_group(group);
        if (g == nullptr) return invalid("not a cuda_sm100 device group");
        for (size_t i = 0; i < g->ranks.size(); ++i) {
            int fault = 0;
            scrapgpu_status st = from_sm100(sm100_set_device(g->devices[i]->ordinal));
            if (st == SCRAPGPU_STATUS_OK) st = from_sm100(sm100_allreduce_fault(g->ranks[i], &fault));
            if (st != SCRAPGPU_STATUS_OK) return st;
            if (fault != 0) {
                set_error("a device of the group gave up waiting for a peer during an all-reduce; the reduced tensors are incomplete");
                return SCRAPGPU_STATUS_BACKEND_ERROR;
            }
        }
        return SCRAPGPU_STATUS_OK;
    });
}

SCRAPGPU_API uint64_t scrapgpu_cuda_sm100_launch_count(void) { return sm100_launch_count(); }

SCRAPGPU_API size_t scrapgpu_cuda_sm100_profile_report(scrapgpu_stream_t * stream, char * out, size_t capacity) {
    Stream * s = as_stream(stream);
    if (s == nullptr || s->prof_stats.empty()) {
        if (out != nullptr && capacity > 0) out[0] = 0;
        return 0;
    }
    std::string text;
    try {
        text = prof_report(s);
    } catch (...) {
        return 0;
    }
    if (out != nullptr && capacity > 0) {
        const size_t n = std::min(capacity - 1, text.size());
        std::memcpy(out, text.data(), n);
        out[n] = 0;
    }
    return text.size() + 1;
}

}  // extern "C"
