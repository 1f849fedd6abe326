"""Shared helpers of the GPU parity tests: seeded inputs, upload/download through the C ABI."""
from __future__ import annotations

import ctypes as C

import numpy as np

from oracle import sgref

Q4_0, Q8_0, Q4_K, Q6_K, F32, F16 = 16, 17, 32, 33, 0, 1
QUANT = (Q4_0, Q8_0, Q4_K, Q6_K)
NAMES = {16: "q4_0", 17: "q8_0", 32: "q4_k", 33: "q6_k", 0: "f32", 1: "f16"}
NATURAL, PACKED = 0, 1

GUARD = 64  # guard floats on each side of an output (canaries, like tests/ref/ref_ops_tests.cpp:684-752)
CANARY = np.float32(-1234.5)


def seeded_weights(seed: int, n: int, k: int) -> np.ndarray:
    """f32 weights ~ N(0, 0.02), the distribution the benchmark configs name."""
    return (np.random.default_rng(seed).standard_normal((n, k)) * 0.02).astype(np.float32)


def seeded_acts(seed: int, m: int, k: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((m, k)).astype(np.float32)


def quantize(dtype: int, w: np.ndarray) -> np.ndarray:
    if dtype == F32:
        return np.ascontiguousarray(w).view(np.uint8).reshape(w.shape[0], -1)
    if dtype == F16:
        return np.ascontiguousarray(w.astype(np.float16)).view(np.uint8).reshape(w.shape[0], -1)
    return sgref.quantize(dtype, w)


def to_device(capi, stream, array: np.ndarray):
    a = np.ascontiguousarray(array)
    b = capi.Buffer(a.nbytes)
    b.upload(stream, a)
    return b


def guarded_output(capi, stream, count: int):
    """Device float buffer of `count` floats with canaries before and after."""
    host = np.full(count + 2 * GUARD, CANARY, dtype=np.float32)
    b = to_device(capi, stream, host)
    return b, b.ptr + 4 * GUARD


def read_guarded(capi, stream, buf, count: int) -> np.ndarray:
    host = buf.download(stream, np.float32, count + 2 * GUARD)
    assert np.all(host[:GUARD] == CANARY), "kernel wrote before its output"
    assert np.all(host[GUARD + count:] == CANARY), "kernel wrote past its output"
    return host[GUARD:GUARD + count]


def device_mul_mat(capi, stream, dtype, layout, wq: np.ndarray, k: int, x: np.ndarray) -> np.ndarray:
    """Runs sm100_mul_mat on (natural or packed) weights; returns y [m, n] and checks the canaries."""
    n, m = wq.shape[0], x.shape[0]
    img = capi.pack(dtype, k, wq) if layout == PACKED else np.ascontiguousarray(wq).ravel()
    wb = to_device(capi, stream, img)
    xb = to_device(capi, stream, x)
    yb, yptr = guarded_output(capi, stream, m * n)
    capi.mul_mat(stream, dtype, layout, wb, k, n, xb, m, yptr)
    stream.sync()
    y = read_guarded(capi, stream, yb, m * n).reshape(m, n).copy()
    for b in (wb, xb, yb):
        b.free()
    return y
