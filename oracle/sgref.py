"""numpy front end of libsgref.so (the C restatement in sgref.c).  Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import threading

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

F32, F16, Q4_0, Q8_0, Q4_K, Q6_K = 0, 1, 16, 17, 32, 33


def build() -> str:
    """Compile sgref.c if the library is missing or older than its source."""
    so = os.path.join(_HERE, "libsgref.so")
    src = os.path.join(_HERE, "sgref.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "libsgref.so"], check=True, capture_output=True)
    return so


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        L = C.CDLL(build())
        i64, fp, vp, ip = C.c_int64, C.POINTER(C.c_float), C.c_void_p, C.POINTER(C.c_int32)
        L.sgref_half_to_float.restype = C.c_float
        L.sgref_half_to_float.argtypes = [C.c_uint16]
        L.sgref_float_to_half.restype = C.c_uint16
        L.sgref_float_to_half.argtypes = [C.c_float]
        L.sgref_dequantize.argtypes = [C.c_int, vp, vp, i64]
        L.sgref_quantize.argtypes = [C.c_int, vp, vp, i64]
        L.sgref_quantize_rows.argtypes = [C.c_int, vp, vp, i64, i64]
        L.sgref_mul_mat.argtypes = [C.c_int, vp, i64, i64, vp, i64, i64, vp, i64]
        L.sgref_rms_norm.restype = None
        L.sgref_rms_norm.argtypes = [vp, vp, vp, vp, vp, i64, i64, C.c_float]
        L.sgref_rope.restype = None
        L.sgref_rope.argtypes = [vp, vp, vp, i64, i64, i64, C.c_int, C.c_int, C.c_float, C.c_float, C.c_float]
        L.sgref_rope_cos_sin.restype = None
        L.sgref_rope_cos_sin.argtypes = [C.c_int32, C.c_int, C.c_int, C.c_float, C.c_float, C.c_float, fp, fp]
        L.sgref_soft_max.restype = None
        L.sgref_soft_max.argtypes = [vp, vp, vp, i64, i64, C.c_float]
        L.sgref_swiglu.restype = None
        L.sgref_swiglu.argtypes = [vp, vp, vp, i64]
        L.sgref_add.restype = None
        L.sgref_add.argtypes = [vp, vp, vp, i64]
        L.sgref_get_rows.argtypes = [C.c_int, vp, i64, i64, vp, i64, vp]
        L.sgref_argmax.restype = C.c_int32
        L.sgref_argmax.argtypes = [vp, i64]
        L.sgref_attention.restype = None
        L.sgref_attention.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, C.c_int, i64, C.c_float]
        _LIB = L
    return _LIB


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def type_size(dtype: int) -> int:
    return lib().sgref_type_size(dtype)


def block_size(dtype: int) -> int:
    return lib().sgref_block_size(dtype)


def row_bytes(dtype: int, k: int) -> int:
    return k // block_size(dtype) * type_size(dtype)


def _threads(n_items: int, threads: int | None) -> int:
    t = threads if threads else (os.cpu_count() or 1)
    return max(1, min(t, n_items))


def _run_split(n_items: int, threads: int | None, fn) -> None:
    """Calls fn(lo, hi) on contiguous slices of range(n_items) from worker threads (ctypes drops the GIL)."""
    t = _threads(n_items, threads)
    if t == 1:
        fn(0, n_items)
        return
    bounds = [n_items * i // t for i in range(t + 1)]
    errs = []

    def work(lo, hi):
        try:
            fn(lo, hi)
        except Exception as e:  # pragma: no cover
            errs.append(e)

    ths = [threading.Thread(target=work, args=(bounds[i], bounds[i + 1])) for i in range(t)]
    for th in ths:
        th.start()
    for th in ths:
        th.join()
    if errs:
        raise errs[0]


def quantize(dtype: int, w: np.ndarray, threads: int | None = None) -> np.ndarray:
    """w: float32 [rows, k] -> uint8 [rows, row_bytes] of natural blocks."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, k = w.shape
    rb = row_bytes(dtype, k)
    out = np.empty((rows, rb), dtype=np.uint8)

    def part(lo, hi):
        if hi > lo:
            st = lib().sgref_quantize_rows(dtype, _p(w[lo:hi]), _p(out[lo:hi]), k, hi - lo)
            if st:
                raise ValueError(f"sgref_quantize_rows status {st}")

    _run_split(rows, threads, part)
    return out


def dequantize(dtype: int, q: np.ndarray, k: int) -> np.ndarray:
    """q: uint8 [rows, row_bytes] -> float32 [rows, k]."""
    q = np.ascontiguousarray(q, dtype=np.uint8)
    rows = q.shape[0]
    out = np.empty((rows, k), dtype=np.float32)
    st = lib().sgref_dequantize(dtype, _p(q), _p(out), rows * k)
    if st:
        raise ValueError(f"sgref_dequantize status {st}")
    return out


def mul_mat(dtype: int, wq: np.ndarray, k: int, x: np.ndarray, threads: int | None = None) -> np.ndarray:
    """wq: [n, row_bytes] blocks (or f32/f16 rows), x: float32 [m, k] -> y float32 [m, n]."""
    wq = np.ascontiguousarray(wq)
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, m = wq.shape[0], x.shape[0]
    y = np.empty((m, n), dtype=np.float32)
    rb = wq.strides[0]

    def part(lo, hi):
        if hi > lo:
            st = lib().sgref_mul_mat(dtype, C.c_void_p(wq.ctypes.data + lo * rb), k, hi - lo, _p(x), m, k,
                                     C.c_void_p(y.ctypes.data + lo * 4), n)
            if st:
                raise ValueError(f"sgref_mul_mat status {st}")

    _run_split(n, threads, part)
    return y


def rms_norm(x, w=None, add=None, eps=1e-6):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, ne0 = x.reshape(-1, x.shape[-1]).shape
    y = np.empty_like(x)
    s = np.empty_like(x) if add is not None else None
    if add is not None:
        add = np.ascontiguousarray(add, dtype=np.float32)
    if w is not None:
        w = np.ascontiguousarray(w, dtype=np.float32)
    lib().sgref_rms_norm(_p(x), _p(add) if add is not None else None, _p(w) if w is not None else None,
                         _p(s) if s is not None else None, _p(y), ne0, rows, eps)
    return (s, y) if add is not None else y


def rope(x, positions, n_dims, neox=True, freq_base=10000.0, freq_scale=1.0, attn_factor=1.0):
    """x: float32 [tokens, heads, ne0]; positions int32 [tokens]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    positions = np.ascontiguousarray(positions, dtype=np.int32)
    tokens, heads, ne0 = x.shape
    y = np.empty_like(x)
    lib().sgref_rope(_p(x), _p(positions), _p(y), ne0, heads, tokens, n_dims, int(neox), freq_base, freq_scale,
                     attn_factor)
    return y


def rope_table(positions, n_dims, freq_base, freq_scale=1.0, attn_factor=1.0) -> np.ndarray:
    """float32 [len(positions), n_dims/2, 2] of (cos, sin) exactly as the reference ROPE evaluates them."""
    out = np.empty((len(positions), n_dims // 2, 2), dtype=np.float32)
    cs, sn = C.c_float(), C.c_float()
    for i, p in enumerate(positions):
        for j in range(n_dims // 2):
            lib().sgref_rope_cos_sin(int(p), j, n_dims, freq_base, freq_scale, attn_factor, C.byref(cs), C.byref(sn))
            out[i, j, 0] = cs.value
            out[i, j, 1] = sn.value
    return out


def soft_max(x, mask=None, scale=1.0):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, ne0 = x.reshape(-1, x.shape[-1]).shape
    y = np.empty_like(x)
    if mask is not None:
        mask = np.ascontiguousarray(np.broadcast_to(mask, x.shape), dtype=np.float32)
    lib().sgref_soft_max(_p(x), _p(mask) if mask is not None else None, _p(y), ne0, rows, scale)
    return y


def swiglu(x, g):
    x = np.ascontiguousarray(x, dtype=np.float32)
    g = np.ascontiguousarray(g, dtype=np.float32)
    y = np.empty_like(x)
    lib().sgref_swiglu(_p(x), _p(g), _p(y), x.size)
    return y


def add(a, b):
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    y = np.empty_like(a)
    lib().sgref_add(_p(a), _p(b), _p(y), a.size)
    return y


def get_rows(dtype, table, k, ids):
    table = np.ascontiguousarray(table)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    out = np.empty((ids.size, k), dtype=np.float32)
    st = lib().sgref_get_rows(dtype, _p(table), k, table.shape[0], _p(ids), ids.size, _p(out))
    if st:
        raise ValueError(f"sgref_get_rows status {st}")
    return out


def argmax(x) -> int:
    x = np.ascontiguousarray(x, dtype=np.float32)
    return int(lib().sgref_argmax(_p(x), x.size))


def attention(q, k, v, causal=True, offset=0, scale=None):
    """q [Hq, nq, D], k [Hkv, nk, D], v [Hkv, nk, Dv] -> out [Hq, nq, Dv] (float32, C order)."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    hq, nq, d = q.shape
    hkv, nk, _ = k.shape
    dv = v.shape[2]
    if scale is None:
        scale = 1.0 / np.sqrt(np.float32(d))
    out = np.empty((hq, nq, dv), dtype=np.float32)
    lib().sgref_attention(_p(q), _p(k), _p(v), _p(out), d, dv, nq, nk, hq, hkv, int(causal), offset, float(scale))
    return out


def nmse(got, want) -> float:
    """sum((got-want)^2)/sum(want^2) in float64: the comparison the reference's device tests use
    (tests/ops/ops_tests.cpp:296-304)."""
    g = np.asarray(got, dtype=np.float64).ravel()
    w = np.asarray(want, dtype=np.float64).ravel()
    den = float(np.dot(w, w))
    num = float(np.dot(g - w, g - w))
    return num / den if den > 0 else num
