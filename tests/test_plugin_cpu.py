"""Host-side contract of the cuda_sm100 plugin that needs no GPU: it loads next to the reference core, registers
idempotently with zero devices, exports what its header declares, and answers foreign or NULL objects with
INVALID_ARGUMENT instead of touching them (the contract tests/cpu/cpu_tests.cpp:279-338 checks on the CPU
backend)."""
import ctypes as C
import os
import re

import pytest

from oracle import refapi
from scrapgpulibrary_b200 import _build, abi

pytestmark = pytest.mark.skipif(not (refapi.available() and os.path.exists(_build.PLUGIN_SO)),
                                reason="needs oracle/_ref and the prebuilt plugin (built where the reference headers are present)")


@pytest.fixture(scope="module")
def env():
    from tests import refsession
    P = refsession.plugin()
    return refapi.lib(), P, P.scrapgpu_cuda_sm100_vtable().contents


def test_exports_and_vtable_shape(env):
    L, P, vt = env
    header = open(os.path.join(_build.INCLUDE, "scrapgpu", "cuda_sm100.h")).read()
    names = set(re.findall(r"\b(scrapgpu_cuda_sm100_\w+)\s*\(", header))
    assert {"scrapgpu_cuda_sm100_register", "scrapgpu_cuda_sm100_vtable", "scrapgpu_cuda_sm100_attention"} <= names
    for n in names:
        assert hasattr(P, n), n
    assert vt.struct_size == C.sizeof(abi.Vtable)
    assert vt.name == b"cuda_sm100"
    for field, _ in abi.Vtable._fields_[3:]:
        assert C.cast(getattr(vt, field), C.c_void_p).value, f"vtable slot {field} is NULL"


def test_register_is_idempotent_without_devices(env):
    L, P, vt = env
    before = L.scrapgpu_get_device_count()
    assert P.scrapgpu_cuda_sm100_register() == abi.OK
    assert P.scrapgpu_cuda_sm100_register() == abi.OK
    n_own = vt.get_device_count(None)
    assert L.scrapgpu_get_device_count() == before + n_own or L.scrapgpu_get_device_count() == before
    dev = C.c_void_p()
    assert vt.get_device(None, n_own, C.byref(dev)) == abi.INVALID_ARGUMENT  # index out of range


def test_foreign_and_null_objects_are_rejected(env):
    L, P, vt = env
    assert L.scrapgpu_cpu_register() == abi.OK
    cpu = C.c_void_p()
    for i in range(L.scrapgpu_get_device_count()):
        L.scrapgpu_get_device(i, C.byref(cpu))
        info = abi.DeviceInfo()
        L.scrapgpu_device_info_init(C.byref(info), C.sizeof(info))
        L.scrapgpu_device_get_info(cpu, C.byref(info))
        if info.backend_name == b"cpu":
            break
    cpu_buf, cpu_stream = C.c_void_p(), C.c_void_p()
    assert L.scrapgpu_buffer_alloc(cpu, 256, C.byref(cpu_buf)) == abi.OK
    assert L.scrapgpu_stream_create(cpu, C.byref(cpu_stream)) == abi.OK
    out = C.c_void_p()
    data = (C.c_uint8 * 16)()
    info = abi.DeviceInfo()
    info.struct_size = C.sizeof(info)
    # objects of another backend and NULL handles: refused, never dereferenced as our own
    for dev in (cpu, None):
        assert vt.buffer_alloc(dev, 64, C.byref(out)) == abi.INVALID_ARGUMENT
        assert vt.stream_create(dev, C.byref(out)) == abi.INVALID_ARGUMENT
        assert vt.device_get_info(dev, C.byref(info)) == abi.INVALID_ARGUMENT
    for s, b in ((cpu_stream, cpu_buf), (None, None)):
        assert vt.buffer_write(s, b, 0, data, 16, 1) == abi.INVALID_ARGUMENT
        assert vt.buffer_read(s, b, 0, data, 16, 1) == abi.INVALID_ARGUMENT
        assert vt.buffer_fill(s, b, 0, 16, 0, 1) == abi.INVALID_ARGUMENT
        assert vt.buffer_copy(s, b, 0, b, 0, 16, 1) == abi.INVALID_ARGUMENT
        assert vt.stream_sync(s) == abi.INVALID_ARGUMENT
        assert vt.plan_execute(s, None) == abi.INVALID_ARGUMENT
    assert vt.buffer_free(cpu_buf) == abi.INVALID_ARGUMENT
    assert vt.stream_free(cpu_stream) == abi.INVALID_ARGUMENT
    assert vt.plan_free(None) == abi.INVALID_ARGUMENT
    assert not vt.stream_device(cpu_stream)
    t = abi.tensor_desc(abi.F32, [4], buffer=cpu_buf.value)
    assert vt.tensor_upload(cpu_stream, C.byref(t), data, 16) == abi.INVALID_ARGUMENT
    op = abi.Op(abi.OP_ADD, [t, t], [t])
    reason = C.c_char_p()
    assert vt.op_supported(cpu, op.ptr(), C.byref(reason)) == abi.INVALID_ARGUMENT
    assert vt.op_execute(cpu_stream, op.ptr()) == abi.INVALID_ARGUMENT
    assert refapi.last_error() != ""
    L.scrapgpu_buffer_free(cpu_buf)
    L.scrapgpu_stream_free(cpu_stream)
