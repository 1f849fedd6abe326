"""The unmodified reference (core + CPU backend + CPU reference ops), compiled by oracle/Makefile from the
reference's own sources into oracle/_ref/libscrapgpu_ref.so and driven through its public C API.
Test infrastructure only.  The library is loaded RTLD_GLOBAL so that a backend plugin loaded afterwards
resolves scrapgpu_register_backend / scrapgpu_op_desc_validate / scrapgpu_set_last_error against it,
exactly as it would inside a real ScrapGpuLibrary process.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import threading

import numpy as np

from scrapgpulibrary_b200 import abi

_HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(_HERE, "_ref", "libscrapgpu_ref.so")
REFERENCE_DIR = os.environ.get("SCRAPGPU_REFERENCE_DIR", "/root/reference")
_LIB = None


def build() -> bool:
    """Compile the reference in place when its checkout is present; True if the library exists afterwards."""
    if os.path.isdir(os.path.join(REFERENCE_DIR, "src", "core")):
        subprocess.run(["make", "-C", _HERE, "ref", f"REF={REFERENCE_DIR}"], check=True, capture_output=True)
    return os.path.exists(SO)


EXAMPLE = os.path.join(_HERE, "_ref", "standalone_matmul")


def build_example() -> bool:
    """The reference's unchanged standalone_matmul example linked against the plugin; True if the binary exists."""
    if os.path.isdir(os.path.join(REFERENCE_DIR, "examples")):
        subprocess.run(["make", "-C", _HERE, "example", f"REF={REFERENCE_DIR}"], check=True, capture_output=True)
    return os.path.exists(EXAMPLE)


OPS_TESTS = os.path.join(_HERE, "_ref", "ops_tests")
ATTENTION_TESTS = os.path.join(_HERE, "_ref", "attention_tests")
OPS_TESTS_REMOTE = os.path.join(_HERE, "_ref", "ops_tests_remote")
DEVICE_SERVER = os.path.join(_HERE, "_ref", "scrapgpu-device-server")


def build_device_tests() -> bool:
    """The reference's own device test programs (tests/ops/ops_tests.cpp, tests/attention/attention_tests.cpp),
    compiled unchanged and linked against the plugin; True if both binaries exist afterwards."""
    if os.path.isfile(os.path.join(REFERENCE_DIR, "tests", "ops", "ops_tests.cpp")):
        subprocess.run(["make", "-C", _HERE, "device_tests", f"REF={REFERENCE_DIR}"], check=True, capture_output=True)
    return os.path.exists(OPS_TESTS) and os.path.exists(ATTENTION_TESTS)


def build_remote_tests() -> bool:
    """The reference's device server and its ops suite with the remote switch (src/backends/remote/server.cpp, client.cpp),
    compiled unchanged against the plugin; True if both binaries exist afterwards."""
    if os.path.isfile(os.path.join(REFERENCE_DIR, "src", "backends", "remote", "server.cpp")):
        subprocess.run(["make", "-C", _HERE, "remote_tests", f"REF={REFERENCE_DIR}"], check=True, capture_output=True)
    return os.path.exists(OPS_TESTS_REMOTE) and os.path.exists(DEVICE_SERVER)


def available() -> bool:
    return os.path.exists(SO)


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        if not available():
            raise FileNotFoundError(f"{SO} is missing (build it with `make -C oracle ref` where the reference is checked out)")
        L = C.CDLL(SO, mode=C.RTLD_GLOBAL)
        vp = C.c_void_p
        L.scrapgpu_ref_quantize.argtypes = [C.c_int, vp, vp, C.c_int64]
        L.scrapgpu_ref_dequantize.argtypes = [C.c_int, vp, vp, C.c_int64]
        L.scrapgpu_ref_execute.argtypes = [C.POINTER(abi.OpDesc), C.POINTER(vp), C.POINTER(vp)]
        L.scrapgpu_last_error.restype = C.c_char_p
        L.scrapgpu_status_string.restype = C.c_char_p
        L.scrapgpu_status_string.argtypes = [C.c_int]
        L.scrapgpu_get_device_count.restype = C.c_size_t
        L.scrapgpu_get_device.argtypes = [C.c_size_t, C.POINTER(vp)]
        L.scrapgpu_device_get_info.argtypes = [vp, C.POINTER(abi.DeviceInfo)]
        L.scrapgpu_device_info_init.argtypes = [C.POINTER(abi.DeviceInfo), C.c_size_t]
        L.scrapgpu_buffer_alloc.argtypes = [vp, C.c_size_t, C.POINTER(vp)]
        L.scrapgpu_buffer_free.argtypes = [vp]
        L.scrapgpu_buffer_write.argtypes = [vp, vp, C.c_uint64, vp, C.c_size_t, C.c_int]
        L.scrapgpu_buffer_read.argtypes = [vp, vp, C.c_uint64, vp, C.c_size_t, C.c_int]
        L.scrapgpu_buffer_copy.argtypes = [vp, vp, C.c_uint64, vp, C.c_uint64, C.c_size_t, C.c_int]
        L.scrapgpu_buffer_fill.argtypes = [vp, vp, C.c_uint64, C.c_size_t, C.c_uint8, C.c_int]
        L.scrapgpu_stream_create.argtypes = [vp, C.POINTER(vp)]
        L.scrapgpu_stream_free.argtypes = [vp]
        L.scrapgpu_stream_sync.argtypes = [vp]
        L.scrapgpu_tensor_upload.argtypes = [vp, C.POINTER(abi.TensorDesc), vp, C.c_size_t]
        L.scrapgpu_tensor_download.argtypes = [vp, C.POINTER(abi.TensorDesc), vp, C.c_size_t]
        L.scrapgpu_tensor_copy.argtypes = [vp, C.POINTER(abi.TensorDesc), vp, C.POINTER(abi.TensorDesc)]
        L.scrapgpu_op_supported.argtypes = [vp, C.POINTER(abi.OpDesc), C.POINTER(C.c_char_p)]
        L.scrapgpu_op_execute.argtypes = [vp, C.POINTER(abi.OpDesc)]
        L.scrapgpu_op_desc_validate.argtypes = [C.POINTER(abi.OpDesc)]
        L.scrapgpu_plan_build.argtypes = [vp, C.POINTER(abi.PlanDesc), C.POINTER(vp)]
        L.scrapgpu_plan_execute.argtypes = [vp, vp]
        L.scrapgpu_plan_free.argtypes = [vp]
        L.scrapgpu_scaled_dot_product_attention.argtypes = [vp, vp, C.POINTER(abi.AttentionParams)]
        L.scrapgpu_register_backend.argtypes = [vp]
        _LIB = L
    return _LIB


def last_error() -> str:
    e = lib().scrapgpu_last_error()
    return e.decode() if e else ""


def check(st: int, what: str = "") -> None:
    if st != abi.OK:
        raise RuntimeError(f"{what}: status {st} ({lib().scrapgpu_status_string(st).decode()}): {last_error()}")


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def quantize(dtype: int, w: np.ndarray, threads: int | None = None) -> np.ndarray:
    """float32 [rows, k] -> uint8 [rows, row_bytes] through scrapgpu_ref_quantize (row by row)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, k = w.shape
    rb = abi.row_size(dtype, k)
    out = np.empty((rows, rb), dtype=np.uint8)
    L = lib()
    t = max(1, min(threads or (os.cpu_count() or 1), rows))
    bounds = [rows * i // t for i in range(t + 1)]

    def part(lo, hi):
        if hi > lo:
            # rows are contiguous block runs, so a slice of rows is one call
            check(L.scrapgpu_ref_quantize(dtype, _p(w[lo:hi]), _p(out[lo:hi]), (hi - lo) * k), "ref_quantize")

    ths = [threading.Thread(target=part, args=(bounds[i], bounds[i + 1])) for i in range(t)]
    [th.start() for th in ths]
    [th.join() for th in ths]
    return out


def dequantize(dtype: int, q: np.ndarray, k: int) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.uint8)
    rows = q.shape[0]
    out = np.empty((rows, k), dtype=np.float32)
    check(lib().scrapgpu_ref_dequantize(dtype, _p(q), _p(out), rows * k), "ref_dequantize")
    return out


def execute(op: int, inputs, outputs, params=None) -> None:
    """scrapgpu_ref_execute on host arrays.  inputs/outputs: lists of (TensorDesc, ndarray)."""
    o = abi.Op(op, [t for t, _ in inputs], [t for t, _ in outputs], params)
    ins = (C.c_void_p * max(1, len(inputs)))(*[a.ctypes.data for _, a in inputs])
    outs = (C.c_void_p * max(1, len(outputs)))(*[a.ctypes.data for _, a in outputs])
    check(lib().scrapgpu_ref_execute(o.ptr(), ins, outs), f"ref_execute(op {op})")


def mul_mat(dtype: int, wq: np.ndarray, k: int, x: np.ndarray, threads: int | None = None) -> np.ndarray:
    """MUL_MAT through scrapgpu_ref_execute.  wq [n, row_bytes], x float32 [m, k] -> y float32 [m, n].
    With threads > 1 the weight rows are split into slices, each slice one unmodified
    scrapgpu_ref_execute call on a row-slice view (the reference itself is single-threaded,
    src/backends/cpu/api.cpp:1-6)."""
    wq = np.ascontiguousarray(wq)
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, m = wq.shape[0], x.shape[0]
    y = np.empty((m, n), dtype=np.float32)
    t = max(1, min(threads or 1, n))
    bounds = [n * i // t for i in range(t + 1)]
    rb = abi.row_size(dtype, k)
    errs = []

    def part(lo, hi):
        try:
            if hi <= lo:
                return
            wt = abi.tensor_desc(dtype, [k, hi - lo])
            xt = abi.tensor_desc(abi.F32, [k, m])
            yt = abi.tensor_desc(abi.F32, [hi - lo, m], nb=[4, 4 * n, 4 * n * m, 4 * n * m])
            p = abi.MulMatParams()
            o = abi.Op(abi.OP_MUL_MAT, [wt, xt], [yt], p)
            ins = (C.c_void_p * 2)(wq.ctypes.data + lo * rb, x.ctypes.data)
            outs = (C.c_void_p * 1)(y.ctypes.data + 4 * lo)
            check(lib().scrapgpu_ref_execute(o.ptr(), ins, outs), "ref_execute(MUL_MAT)")
        except Exception as e:  # pragma: no cover
            errs.append(e)

    if t == 1:
        part(0, n)
    else:
        ths = [threading.Thread(target=part, args=(bounds[i], bounds[i + 1])) for i in range(t)]
        [th.start() for th in ths]
        [th.join() for th in ths]
    if errs:
        raise errs[0]
    return y
