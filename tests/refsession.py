"""Drives a ScrapGpuLibrary backend through the reference's own public C API (the unmodified core compiled into
oracle/_ref/), the way the reference's tests/ops/ops_tests.cpp does: buffers, uploads, op_execute, downloads.
Used to run the SAME descriptors on the reference's `cpu` device and on `cuda_sm100`."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from oracle import refapi
from scrapgpulibrary_b200 import _build, abi

_PLUGIN = None


def plugin() -> C.CDLL:
    """The cuda_sm100 plugin, loaded after the core so that its core symbols resolve."""
    global _PLUGIN
    if _PLUGIN is None:
        refapi.lib()
        from scrapgpulibrary_b200 import capi
        capi.lib()
        if not os.path.exists(_build.PLUGIN_SO):
            raise FileNotFoundError(f"{_build.PLUGIN_SO} is missing (it is built where the ScrapGpuLibrary headers are present)")
        P = C.CDLL(_build.PLUGIN_SO, mode=C.RTLD_GLOBAL)
        P.scrapgpu_cuda_sm100_vtable.restype = C.POINTER(abi.Vtable)
        P.scrapgpu_cuda_sm100_attention.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(abi.AttentionParams)]
        P.scrapgpu_cuda_sm100_attention_at.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(abi.AttentionParams), C.POINTER(abi.TensorDesc)]
        P.scrapgpu_cuda_sm100_launch_count.restype = C.c_uint64
        _PLUGIN = P
    return _PLUGIN


def register_all() -> None:
    L = refapi.lib()
    refapi.check(L.scrapgpu_cpu_register(), "cpu_register")
    refapi.check(plugin().scrapgpu_cuda_sm100_register(), "cuda_sm100_register")


def find_device(backend: str, index: int = 0):
    L = refapi.lib()
    seen = 0
    for i in range(L.scrapgpu_get_device_count()):
        dev = C.c_void_p()
        refapi.check(L.scrapgpu_get_device(i, C.byref(dev)), "get_device")
        info = abi.DeviceInfo()
        L.scrapgpu_device_info_init(C.byref(info), C.sizeof(info))
        refapi.check(L.scrapgpu_device_get_info(dev, C.byref(info)), "device_get_info")
        if info.backend_name == backend.encode():
            if seen == index:
                return dev, info
            seen += 1
    return None, None


class Tensor:
    """A device tensor with its own buffer (like TT in ops_tests.cpp:120-190)."""

    def __init__(self, sess: "Session", dtype: int, ne, layout=abi.LAYOUT_NATURAL, nb=None, pad: int = 0, offset: int = 0):
        self.sess = sess
        self.desc = abi.tensor_desc(dtype, ne, layout=layout, nb=nb, offset=offset)
        self.nbytes = self.span()
        self.buf = sess.alloc(offset + self.nbytes + pad)
        self.desc.buffer = self.buf.value

    def span(self) -> int:
        d = self.desc
        be, bb = abi.BLOCK[d.dtype]
        n = bb if be == 1 else d.ne[0] * d.nb[0] // be
        for i in range(0 if be == 1 else 1, 4):
            n += (d.ne[i] - 1) * d.nb[i]
        return int(n)

    def upload(self, array: np.ndarray) -> "Tensor":
        a = np.ascontiguousarray(array)
        refapi.check(refapi.lib().scrapgpu_tensor_upload(self.sess.stream, C.byref(self.desc), a.ctypes.data_as(C.c_void_p), a.nbytes), "tensor_upload")
        return self

    def write_raw(self, array: np.ndarray, offset: int = 0) -> "Tensor":
        a = np.ascontiguousarray(array)
        refapi.check(refapi.lib().scrapgpu_buffer_write(self.sess.stream, self.buf, offset, a.ctypes.data_as(C.c_void_p), a.nbytes, 1), "buffer_write")
        return self

    def download(self, dtype, count: int) -> np.ndarray:
        out = np.empty(count, dtype=dtype)
        refapi.check(refapi.lib().scrapgpu_tensor_download(self.sess.stream, C.byref(self.desc), out.ctypes.data_as(C.c_void_p), out.nbytes), "tensor_download")
        return out

    def read_raw(self, dtype, count: int, offset: int = 0) -> np.ndarray:
        out = np.empty(count, dtype=dtype)
        refapi.check(refapi.lib().scrapgpu_buffer_read(self.sess.stream, self.buf, offset, out.ctypes.data_as(C.c_void_p), out.nbytes, 1), "buffer_read")
        return out

    def free(self) -> None:
        if self.buf is not None:
            refapi.lib().scrapgpu_buffer_free(self.buf)
            self.buf = None


class Session:
    def __init__(self, backend: str, index: int = 0):
        register_all()
        self.backend = backend
        self.device, self.info = find_device(backend, index)
        if self.device is None:
            raise RuntimeError(f"no device of backend {backend}")
        self.stream = C.c_void_p()
        refapi.check(refapi.lib().scrapgpu_stream_create(self.device, C.byref(self.stream)), "stream_create")
        self.tensors = []

    def alloc(self, nbytes: int):
        b = C.c_void_p()
        refapi.check(refapi.lib().scrapgpu_buffer_alloc(self.device, max(1, nbytes), C.byref(b)), "buffer_alloc")
        return b

    def tensor(self, dtype: int, ne, **kw) -> Tensor:
        t = Tensor(self, dtype, ne, **kw)
        self.tensors.append(t)
        return t

    def supported(self, op: int, inputs, outputs, params=None):
        o = abi.Op(op, [t.desc for t in inputs], [t.desc for t in outputs], params)
        reason = C.c_char_p()
        st = refapi.lib().scrapgpu_op_supported(self.device, o.ptr(), C.byref(reason))
        return st, (reason.value or b"").decode()

    def execute(self, op: int, inputs, outputs, params=None, expect=abi.OK) -> int:
        o = abi.Op(op, [t.desc for t in inputs], [t.desc for t in outputs], params)
        st = refapi.lib().scrapgpu_op_execute(self.stream, o.ptr())
        if expect is not None and st != expect:
            raise AssertionError(f"op {op} on {self.backend}: status {st}, expected {expect}: {refapi.last_error()}")
        return st

    def sync(self) -> None:
        refapi.check(refapi.lib().scrapgpu_stream_sync(self.stream), "stream_sync")

    def close(self) -> None:
        for t in self.tensors:
            t.free()
        self.tensors = []
        if self.stream:
            refapi.lib().scrapgpu_stream_free(self.stream)
            self.stream = None
