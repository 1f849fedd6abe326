"""ctypes mirror of the ScrapGpuLibrary public C ABI (version 0.4).

These are the structures a caller of the reference library fills in; the `cuda_sm100` backend plugin
receives exactly these through its vtable.  Field order and types follow the reference headers:

  scrapgpu_tensor_desc        include/scrapgpu/tensor.h:29-37
  scrapgpu_op_desc            include/scrapgpu/op.h:176-185
  parameter structs           include/scrapgpu/op.h:76-174
  scrapgpu_device_info        include/scrapgpu/device.h:30-52
  scrapgpu_backend_vtable     include/scrapgpu/backend.h:29-57
  scrapgpu_attention_params   include/scrapgpu/attention.h:31-44

Nothing here computes anything: it is the binding layer used by the tests and the benchmark to drive
the plugin the way a C caller would.
"""
from __future__ import annotations

import ctypes as C

# ---- enums ---------------------------------------------------------------------------------------
# scrapgpu_dtype (tensor.h:10-22)
F32, F16, I32, I64, I16, BF16 = 0, 1, 2, 3, 4, 5
Q4_0, Q8_0, Q4_K, Q6_K = 16, 17, 32, 33
DTYPE_NAMES = {F32: "f32", F16: "f16", I32: "i32", I64: "i64", I16: "i16", BF16: "bf16",
               Q4_0: "q4_0", Q8_0: "q8_0", Q4_K: "q4_k", Q6_K: "q6_k"}
DTYPE_BY_NAME = {v: k for k, v in DTYPE_NAMES.items()}
# (elements per block, bytes per block)  src/tensor/tensor.h:26-52
BLOCK = {F32: (1, 4), F16: (1, 2), I32: (1, 4), I64: (1, 8), I16: (1, 2), BF16: (1, 2),
         Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210)}

LAYOUT_NATURAL, LAYOUT_R32 = 0, 1   # tensor.h:24-27; tag 1 means "backend-packed" for cuda_sm100

# scrapgpu_status (status.h:10-17)
OK, UNSUPPORTED, INVALID_ARGUMENT, OUT_OF_MEMORY, BACKEND_ERROR, DEVICE_LOST = range(6)

# scrapgpu_op (op.h:10-48)
OP_NONE, OP_RESHAPE, OP_VIEW, OP_PERMUTE, OP_TRANSPOSE = 0, 1, 2, 3, 4
OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_SCALE = 10, 11, 12, 13, 14
OP_GLU, OP_RMS_NORM, OP_ROPE, OP_SOFT_MAX, OP_GET_ROWS, OP_SET_ROWS, OP_CPY = 19, 20, 21, 22, 23, 24, 25
OP_DUP, OP_CONT, OP_MUL_MAT = 26, 27, 28
OP_ARGSORT, OP_TOP_K = 35, 36
OP_RMS_NORM_MUL, OP_ADD_RMS_NORM_MUL, OP_SET_ROWS_PAIR, OP_MUL_MAT_MULTI, OP_CONT_MUL_MAT = 100, 101, 102, 103, 104

GLU_SWIGLU, GLU_REGLU = 0, 1
ROPE_NORMAL, ROPE_NEOX = 0, 1


def row_size(dtype: int, ne0: int) -> int:
    be, bb = BLOCK[dtype]
    return (ne0 + be - 1) // be * bb


# ---- structures ----------------------------------------------------------------------------------
class TensorDesc(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("dtype", C.c_int), ("ne", C.c_int64 * 4),
                ("nb", C.c_uint64 * 4), ("buffer", C.c_void_p), ("offset", C.c_uint64),
                ("layout", C.c_int)]


class OpDesc(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("op", C.c_int), ("inputs", C.POINTER(TensorDesc)),
                ("input_count", C.c_size_t), ("outputs", C.POINTER(TensorDesc)),
                ("output_count", C.c_size_t), ("params", C.c_void_p), ("params_size", C.c_size_t)]


class MulMatParams(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("allow_broadcast", C.c_int)]


class RmsNormParams(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("eps", C.c_float)]


class RopeParams(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("mode", C.c_int), ("n_dims", C.c_int32),
                ("n_ctx_orig", C.c_int32), ("freq_base", C.c_float), ("freq_scale", C.c_float),
                ("ext_factor", C.c_float), ("attn_factor", C.c_float), ("beta_fast", C.c_float),
                ("beta_slow", C.c_float), ("freq_factors", C.c_void_p), ("n_offs", C.c_void_p)]


class SoftMaxParams(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("scale", C.c_float), ("mask", C.c_void_p)]


class GluParams(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("kind", C.c_int), ("split_inputs", C.c_int),
                ("swapped", C.c_int)]


class GetRowsParams(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("indices_are_i64", C.c_int)]


SetRowsParams = GetRowsParams


class CpyParams(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("allow_transpose", C.c_int)]


class ArgsortParams(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("order", C.c_int), ("top_k", C.c_uint32)]


class AttentionParams(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("query", C.POINTER(TensorDesc)),
                ("key", C.POINTER(TensorDesc)), ("value", C.POINTER(TensorDesc)),
                ("mask", C.POINTER(TensorDesc)), ("output", C.POINTER(TensorDesc)),
                ("query_position_offset", C.c_uint64), ("max_workspace_bytes", C.c_uint64),
                ("causal", C.c_int), ("scale", C.c_float)]


class DeviceInfo(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("name", C.c_char_p), ("vendor", C.c_char_p),
                ("platform_name", C.c_char_p), ("driver_version", C.c_char_p),
                ("backend_name", C.c_char_p), ("reported_api_version", C.c_char_p),
                ("used_api_version", C.c_char_p), ("generation", C.c_int),
                ("generation_reason", C.c_char_p), ("total_memory_bytes", C.c_uint64),
                ("max_allocation_reported_bytes", C.c_uint64), ("max_allocation_used_bytes", C.c_uint64),
                ("max_work_group_size", C.c_uint64), ("local_memory_bytes", C.c_uint64),
                ("compute_units", C.c_uint32), ("warp_or_wave_width", C.c_uint32),
                ("quirks", C.c_uint64), ("probed_quirks", C.c_uint64),
                ("tuning_profile_name", C.c_char_p), ("tuning_overrides", C.c_char_p)]


class PlanNode(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("op", OpDesc), ("output_use_count", C.c_uint32)]


class PlanDesc(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("nodes", C.POINTER(PlanNode)), ("node_count", C.c_size_t)]


_st = C.c_int
_vp = C.c_void_p
_fn = C.CFUNCTYPE


class Vtable(C.Structure):
    """scrapgpu_backend_vtable, ABI 0.4 (backend.h:29-57)."""
    _fields_ = [
        ("struct_size", C.c_size_t), ("name", C.c_char_p), ("userdata", _vp),
        ("get_device_count", _fn(C.c_size_t, _vp)),
        ("get_device", _fn(_st, _vp, C.c_size_t, C.POINTER(_vp))),
        ("device_get_info", _fn(_st, _vp, C.POINTER(DeviceInfo))),
        ("buffer_alloc", _fn(_st, _vp, C.c_size_t, C.POINTER(_vp))),
        ("buffer_free", _fn(_st, _vp)),
        ("buffer_write", _fn(_st, _vp, _vp, C.c_uint64, _vp, C.c_size_t, C.c_int)),
        ("buffer_read", _fn(_st, _vp, _vp, C.c_uint64, _vp, C.c_size_t, C.c_int)),
        ("buffer_copy", _fn(_st, _vp, _vp, C.c_uint64, _vp, C.c_uint64, C.c_size_t, C.c_int)),
        ("buffer_fill", _fn(_st, _vp, _vp, C.c_uint64, C.c_size_t, C.c_uint8, C.c_int)),
        ("stream_sync", _fn(_st, _vp)),
        ("op_supported", _fn(_st, _vp, C.POINTER(OpDesc), C.POINTER(C.c_char_p))),
        ("plan_build", _fn(_st, _vp, C.POINTER(PlanDesc), C.POINTER(_vp))),
        ("plan_execute", _fn(_st, _vp, _vp)),
        ("plan_free", _fn(_st, _vp)),
        ("stream_create", _fn(_st, _vp, C.POINTER(_vp))),
        ("stream_free", _fn(_st, _vp)),
        ("tensor_upload", _fn(_st, _vp, C.POINTER(TensorDesc), _vp, C.c_size_t)),
        ("tensor_download", _fn(_st, _vp, C.POINTER(TensorDesc), _vp, C.c_size_t)),
        ("op_execute", _fn(_st, _vp, C.POINTER(OpDesc))),
        ("stream_device", _fn(_vp, _vp)),
    ]


# ---- helpers -------------------------------------------------------------------------------------
def tensor_desc(dtype: int, ne, buffer=None, offset: int = 0, layout: int = LAYOUT_NATURAL, nb=None) -> TensorDesc:
    """A contiguous descriptor: nb[0] = block bytes, nb[1] = row bytes, nb[i] = nb[i-1]*ne[i-1]."""
    ne = list(ne) + [1] * (4 - len(ne))
    t = TensorDesc()
    t.struct_size = C.sizeof(TensorDesc)
    t.dtype = dtype
    be, bb = BLOCK[dtype]
    if nb is None:
        nb = [bb, row_size(dtype, ne[0]), 0, 0]
        nb[2] = nb[1] * ne[1]
        nb[3] = nb[2] * ne[2]
    for i in range(4):
        t.ne[i] = ne[i]
        t.nb[i] = nb[i]
    t.buffer = buffer
    t.offset = offset
    t.layout = layout
    return t


def tensor_nbytes(t: TensorDesc) -> int:
    return int(t.nb[3] * t.ne[3]) if t.ne[3] > 1 else int(max(t.nb[1] * t.ne[1], t.nb[2] * t.ne[2]))


class Op:
    """Keeps the arrays an OpDesc points to alive."""

    def __init__(self, op: int, inputs, outputs, params=None):
        self.inputs = (TensorDesc * max(1, len(inputs)))(*inputs)
        self.outputs = (TensorDesc * max(1, len(outputs)))(*outputs)
        self.params = params
        d = OpDesc()
        d.struct_size = C.sizeof(OpDesc)
        d.op = op
        d.inputs = self.inputs
        d.input_count = len(inputs)
        d.outputs = self.outputs
        d.output_count = len(outputs)
        if params is not None:
            params.struct_size = C.sizeof(params)
            d.params = C.cast(C.pointer(params), C.c_void_p)
            d.params_size = C.sizeof(params)
        self.desc = d

    def ptr(self):
        return C.byref(self.desc)
