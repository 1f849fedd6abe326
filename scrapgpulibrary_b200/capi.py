"""ctypes binding of libscrapgpu_sm100.so (include/scrapgpu_sm100.h).

There is no fallback: if the CUDA library is missing, or no CUDA device is present, the calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import _build

_LIB = None


class Sm100Error(RuntimeError):
    def __init__(self, status: int, what: str, message: str):
        super().__init__(f"{what}: status {status}: {message}")
        self.status = status


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        if not os.path.exists(_build.SM100_SO):
            raise FileNotFoundError(
                f"{_build.SM100_SO} is missing: build it with `python -m scrapgpulibrary_b200._build` "
                "(there is no CPU fallback for the device path)")
        L = C.CDLL(_build.SM100_SO, mode=C.RTLD_GLOBAL)
        vp, i64, i32, sz = C.c_void_p, C.c_int64, C.c_int, C.c_size_t
        pv = C.POINTER(C.c_void_p)
        L.sm100_last_error.restype = C.c_char_p
        L.sm100_device_info.argtypes = [i32, C.c_char_p, sz, C.POINTER(C.c_uint64), C.POINTER(C.c_uint32),
                                        C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)]
        L.sm100_malloc.argtypes = [i32, sz, pv]
        L.sm100_free.argtypes = [i32, vp]
        L.sm100_host_alloc.argtypes = [sz, pv]
        L.sm100_host_free.argtypes = [vp]
        L.sm100_stream_create.argtypes = [i32, pv]
        L.sm100_stream_destroy.argtypes = [i32, vp]
        L.sm100_stream_sync.argtypes = [vp]
        for f in (L.sm100_memcpy_h2d, L.sm100_memcpy_d2h, L.sm100_memcpy_d2d):
            f.argtypes = [vp, vp, vp, sz, i32]
        L.sm100_memset.argtypes = [vp, vp, i32, sz, i32]
        L.sm100_memcpy_peer.argtypes = [vp, i32, vp, vp, i32, vp, sz]
        L.sm100_event_create.argtypes = [pv]
        L.sm100_event_destroy.argtypes = [vp]
        L.sm100_event_record.argtypes = [vp, vp]
        L.sm100_stream_wait_event.argtypes = [vp, vp]
        L.sm100_event_sync.argtypes = [vp]
        L.sm100_event_elapsed_ms.argtypes = [vp, vp, C.POINTER(C.c_float)]
        L.sm100_graph_begin.argtypes = [vp]
        L.sm100_graph_end.argtypes = [vp, pv]
        L.sm100_graph_launch.argtypes = [vp, vp]
        L.sm100_graph_destroy.argtypes = [vp]
        L.sm100_launch_count.restype = C.c_uint64
        L.sm100_set_pdl.argtypes = [i32]
        L.sm100_row_bytes.restype = sz
        L.sm100_row_bytes.argtypes = [i32, i64]
        L.sm100_pack.argtypes = [i32, i64, i64, vp, vp]
        L.sm100_unpack.argtypes = [i32, i64, i64, vp, vp]
        L.sm100_pack_device.argtypes = [vp, i32, i64, i64, vp, vp]
        L.sm100_unpack_device.argtypes = [vp, i32, i64, i64, vp, vp]
        L.sm100_mul_mat.argtypes = [vp, i32, i32, vp, i64, i64, i64, vp, i64, i64, vp, i64]
        L.sm100_hostpipe_create.argtypes = [i32, i32, sz, sz, pv]
        L.sm100_hostpipe_destroy.argtypes = [vp]
        L.sm100_hostpipe_stream.argtypes = [vp, i32, pv]
        L.sm100_hostpipe_mul_mat.argtypes = [vp, i32, i32, vp, i64, i64, i64, vp, i64, vp]
        L.sm100_hostpipe_mul_mat_many.argtypes = [vp, i32, vp]
        L.sm100_hostpipe_sync.argtypes = [vp]
        L.sm100_head_post.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, vp, vp, i64, i64, i64, i64, C.c_float, C.c_float, i32]
        L.sm100_attention_decode.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, vp, vp, vp, i64, i64, i64, i64, C.c_float, C.c_float, i32, C.c_float]
        L.sm100_ipc_handle_bytes.restype = sz
        L.sm100_ipc_export.argtypes = [vp, vp]
        L.sm100_ipc_open.argtypes = [vp, pv]
        L.sm100_ipc_close.argtypes = [vp]
        L.sm100_allreduce_area_bytes.restype = sz
        L.sm100_allreduce_area_bytes.argtypes = [i32, i32]
        L.sm100_allreduce_create.argtypes = [i32, i32, i32, pv, pv]
        L.sm100_allreduce_sum.argtypes = [vp, vp, vp, i32]
        L.sm100_allreduce_set_wait_limit.argtypes = [vp, C.c_uint32]
        L.sm100_argmax_allreduce.argtypes = [vp, vp, vp, i64, i64, vp]
        L.sm100_mul_mat_glu.argtypes = [vp, i32, vp, vp, vp, C.c_float, vp, vp, i32, i32, vp, vp, i64, i64, vp, vp, vp]
        L.sm100_mul_mat_allreduce.argtypes = [vp, vp, i32, vp, vp, i32, i32, vp, i64, i64, vp]
        L.sm100_allreduce_fault.argtypes = [vp, C.POINTER(i32)]
        L.sm100_allreduce_destroy.argtypes = [vp]
        L.sm100_mul_mat_fused.argtypes = [vp, i32, vp, vp, vp, C.c_float, vp, vp, i32, C.POINTER(i32), C.POINTER(i32), pv, i64, C.POINTER(i64), pv]
        L.sm100_mul_mat_multi.argtypes = [vp, i32, C.POINTER(i32), C.POINTER(i32), pv, i64, C.POINTER(i64), vp, pv]
        L.sm100_get_rows.argtypes = [vp, i32, i32, vp, i64, i64, i64, vp, i64, vp, i64]
        L.sm100_rms_norm.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, C.c_float]
        L.sm100_rope.argtypes = [vp, vp, vp, vp, C.c_int32, C.c_int32, vp, i64, i64, i64, i32, i32]
        L.sm100_rope_direct.argtypes = [vp, vp, vp, vp, i64, i64, i64, i32, i32, C.c_float, C.c_float, C.c_float]
        L.sm100_soft_max.argtypes = [vp, vp, vp, i64, vp, i64, i64, C.c_float]
        L.sm100_swiglu.argtypes = [vp, vp, vp, vp, i64]
        L.sm100_add.argtypes = [vp, vp, vp, vp, i64]
        L.sm100_set_rows.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64]
        L.sm100_argmax.argtypes = [vp, vp, i64, vp]
        L.sm100_launch_serialized.argtypes = [i32]
        L.sm100_attention.argtypes = [vp, vp, vp, vp, vp, i64, vp, i64, i64, i64, i64, i64, i64, i32, i64, vp, C.c_float]
        L.sm100_attention_static.argtypes = L.sm100_attention.argtypes
        L.sm100_attention_kvcache.argtypes = L.sm100_attention.argtypes + [i32]
        L.sm100_attention_static_capacity.restype = C.c_size_t
        L.sm100_attention_static_prepare.argtypes = [pv]
        L.sm100_matvec_last_kernel.restype = C.c_char_p
        L.sm100_cont_mul_mat.argtypes = [vp, vp, i32, vp, vp]
        _LIB = L
    return _LIB


def check(status: int, what: str = "sm100") -> None:
    if status != 0:
        raise Sm100Error(status, what, (lib().sm100_last_error() or b"").decode())


_DEFAULT_DEVICE = 0


def set_default_device(device: int) -> None:
    """Device used by Stream() / Buffer() when none is given (one process per GPU: the local rank)."""
    global _DEFAULT_DEVICE
    _DEFAULT_DEVICE = int(device)
    check(lib().sm100_set_device(_DEFAULT_DEVICE), "set_device")


def device_count() -> int:
    return lib().sm100_device_count()


def require_device() -> None:
    if device_count() < 1:
        raise RuntimeError("no CUDA device: the cuda_sm100 path has no CPU fallback")


class Stream:
    def __init__(self, device: int | None = None):
        self.device = device = _DEFAULT_DEVICE if device is None else device
        h = C.c_void_p()
        check(lib().sm100_stream_create(device, C.byref(h)), "stream_create")
        self.handle = h

    def sync(self) -> None:
        check(lib().sm100_stream_sync(self.handle), "stream_sync")

    def wait(self, event: "Event") -> None:
        """Later work on this stream starts only after the work recorded in `event` (on another stream) is done."""
        check(lib().sm100_stream_wait_event(self.handle, event.handle), "stream_wait_event")

    def close(self) -> None:
        if self.handle:
            lib().sm100_stream_destroy(self.device, self.handle)
            self.handle = None


class HostPipeItem(C.Structure):
    """sm100_hostpipe_item"""
    _fields_ = [("dtype", C.c_int), ("layout", C.c_int), ("w", C.c_void_p), ("w_row_stride", C.c_int64), ("k", C.c_int64), ("n", C.c_int64),
                ("host_x", C.c_void_p), ("m", C.c_int64), ("host_y", C.c_void_p)]


class HostPipe:
    """MUL_MAT with host activations in and host results out, one call per product (sm100_hostpipe_*): copies and
    kernels on three streams of the pipe's own.  Host pointers are raw addresses of pinned memory."""

    def __init__(self, depth: int, max_x_bytes: int, max_y_bytes: int, device: int | None = None):
        self.device = _DEFAULT_DEVICE if device is None else device
        h = C.c_void_p()
        check(lib().sm100_hostpipe_create(self.device, depth, max_x_bytes, max_y_bytes, C.byref(h)), "hostpipe_create")
        self.handle = h

    def stream(self, which: int) -> "Stream":
        """0: copy-in, 1: kernels, 2: read-back.  A view: closing it is not the caller's business."""
        h = C.c_void_p()
        check(lib().sm100_hostpipe_stream(self.handle, which, C.byref(h)), "hostpipe_stream")
        s = Stream.__new__(Stream)
        s.device, s.handle = self.device, h
        return s

    def mul_mat(self, dtype: int, layout: int, w: "Buffer", k: int, n: int, host_x, m: int, host_y) -> None:
        check(lib().sm100_hostpipe_mul_mat(self.handle, dtype, layout, w.at(), 0, k, n, host_x, m, host_y), "hostpipe_mul_mat")

    def mul_mat_many(self, items, count: int) -> None:
        """items: a ctypes array of HostPipeItem"""
        check(lib().sm100_hostpipe_mul_mat_many(self.handle, count, C.cast(items, C.c_void_p)), "hostpipe_mul_mat_many")

    def sync(self) -> None:
        check(lib().sm100_hostpipe_sync(self.handle), "hostpipe_sync")

    def close(self) -> None:
        if self.handle:
            lib().sm100_hostpipe_destroy(self.handle)
            self.handle = None


class Event:
    def __init__(self):
        h = C.c_void_p()
        check(lib().sm100_event_create(C.byref(h)), "event_create")
        self.handle = h

    def record(self, stream: Stream) -> None:
        check(lib().sm100_event_record(self.handle, stream.handle), "event_record")

    def sync(self) -> None:
        check(lib().sm100_event_sync(self.handle), "event_sync")

    def elapsed_ms(self, stop: "Event") -> float:
        ms = C.c_float()
        check(lib().sm100_event_elapsed_ms(self.handle, stop.handle, C.byref(ms)), "event_elapsed")
        return float(ms.value)


class Buffer:
    """A device allocation (the backend's buffer_alloc)."""

    def __init__(self, nbytes: int, device: int | None = None):
        self.device = device = _DEFAULT_DEVICE if device is None else device
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        check(lib().sm100_malloc(device, max(1, self.nbytes), C.byref(p)), "malloc")
        self.ptr = p.value

    def at(self, offset: int = 0) -> C.c_void_p:
        return C.c_void_p(self.ptr + offset)

    def upload(self, stream: Stream, array: np.ndarray, offset: int = 0) -> None:
        a = np.ascontiguousarray(array)
        assert offset + a.nbytes <= self.nbytes
        check(lib().sm100_memcpy_h2d(stream.handle, self.at(offset), a.ctypes.data_as(C.c_void_p), a.nbytes, 1), "h2d")

    def download(self, stream: Stream, dtype, count: int, offset: int = 0) -> np.ndarray:
        out = np.empty(count, dtype=dtype)
        assert offset + out.nbytes <= self.nbytes
        check(lib().sm100_memcpy_d2h(stream.handle, out.ctypes.data_as(C.c_void_p), self.at(offset), out.nbytes, 1), "d2h")
        return out

    def fill(self, stream: Stream, byte: int) -> None:
        check(lib().sm100_memset(stream.handle, self.at(), byte, self.nbytes, 1), "memset")

    def free(self) -> None:
        if self.ptr:
            lib().sm100_free(self.device, C.c_void_p(self.ptr))
            self.ptr = None


class Graph:
    """Captured launch sequence (what a plan of the reference API becomes on this backend)."""

    def __init__(self, stream: Stream):
        self.stream = stream
        self.handle = None

    def __enter__(self):
        check(lib().sm100_graph_begin(self.stream.handle), "graph_begin")
        return self

    def __exit__(self, et, ev, tb):
        h = C.c_void_p()
        st = lib().sm100_graph_end(self.stream.handle, C.byref(h))
        if et is None:
            check(st, "graph_end")
            self.handle = h
        return False

    def launch(self) -> None:
        check(lib().sm100_graph_launch(self.handle, self.stream.handle), "graph_launch")

    def destroy(self) -> None:
        if self.handle:
            lib().sm100_graph_destroy(self.handle)
            self.handle = None


def pack(dtype: int, k: int, natural: np.ndarray) -> np.ndarray:
    """natural uint8 [n, row_bytes] -> packed uint8 [n * row_bytes] (host side)."""
    natural = np.ascontiguousarray(natural, dtype=np.uint8)
    n = natural.shape[0]
    out = np.empty(natural.size, dtype=np.uint8)
    check(lib().sm100_pack(dtype, k, n, natural.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p)), "pack")
    return out


def unpack(dtype: int, k: int, n: int, packed: np.ndarray) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty((n, packed.size // n), dtype=np.uint8)
    check(lib().sm100_unpack(dtype, k, n, packed.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p)), "unpack")
    return out


def mul_mat(stream: Stream, dtype: int, layout: int, w: Buffer | int, k: int, n: int, x, m: int, y, ldx=None, ldy=None,
            w_row_stride: int = 0) -> None:
    """y[N, M] = W[K, N] . x[K, M]; w, x, y are device pointers (int) or Buffers."""
    p = lambda b: C.c_void_p(b.ptr if isinstance(b, Buffer) else b)
    check(lib().sm100_mul_mat(stream.handle, dtype, layout, p(w), w_row_stride, k, n, p(x), ldx or k, m, p(y), ldy or n), "mul_mat")
