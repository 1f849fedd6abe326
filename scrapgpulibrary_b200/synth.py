"""Seeded synthetic weights for the benchmark: valid GGUF blocks made with vectorised numpy.

The benchmark configs name weights ~ N(0, 0.02) quantized to Q4_0 / Q8_0 / Q4_K / Q6_K.  Real model files
and the reference's iterative K-quant search are not part of the timed product path, so the benchmark
builds its blocks here: Q4_0 / Q8_0 use the same absmax rule as the reference quantizer
(src/core/ref/quant.cpp:111-155); Q4_K / Q6_K use the plain min/max rule per sub-block (no iterative
refinement) in the exact block format, which decodes with the reference's dequantizer.  Throughput does
not depend on which valid bytes a block holds.  Parity tests do not use this module: they quantize with
the CPU oracle.
"""
from __future__ import annotations

import numpy as np

Q4_0, Q8_0, Q4_K, Q6_K = 16, 17, 32, 33


def gaussian_weights(seed: int, n: int, k: int, std: float = 0.02) -> np.ndarray:
    return (np.random.default_rng(seed).standard_normal((n, k), dtype=np.float32) * np.float32(std))


def _f16_bytes(a: np.ndarray) -> np.ndarray:
    return a.astype(np.float16).view(np.uint8).reshape(a.shape + (2,))


def quantize_q4_0(w: np.ndarray) -> np.ndarray:
    n, k = w.shape
    b = w.reshape(n, k // 32, 32)
    idx = np.abs(b).argmax(axis=2)
    vmax = np.take_along_axis(b, idx[..., None], axis=2)[..., 0]
    d = vmax / np.float32(-8.0)
    inv = np.where(d != 0, np.float32(1.0) / np.where(d != 0, d, 1), np.float32(0.0)).astype(np.float32)
    q = np.minimum(15, (b * inv[..., None] + np.float32(8.5)).astype(np.int32).clip(0, 255)).astype(np.uint8)
    out = np.empty((n, k // 32, 18), np.uint8)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:] = q[..., :16] | (q[..., 16:] << 4)
    return out.reshape(n, -1)


def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    n, k = w.shape
    b = w.reshape(n, k // 32, 32)
    d = np.abs(b).max(axis=2) / np.float32(127.0)
    inv = np.where(d != 0, np.float32(1.0) / np.where(d != 0, d, 1), np.float32(0.0)).astype(np.float32)
    q = np.rint(b * inv[..., None]).clip(-127, 127).astype(np.int8)
    out = np.empty((n, k // 32, 34), np.uint8)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(n, -1)


def quantize_q4_k(w: np.ndarray) -> np.ndarray:
    n, k = w.shape
    nb = k // 256
    b = w.reshape(n, nb, 8, 32)
    lo = np.minimum(b.min(axis=3), 0.0)
    hi = b.max(axis=3)
    scale = (hi - lo) / np.float32(15.0)          # per sub-block
    mins = -lo                                    # >= 0
    d = (scale.max(axis=2) / np.float32(63.0)).astype(np.float16).astype(np.float32)
    dmin = (mins.max(axis=2) / np.float32(63.0)).astype(np.float16).astype(np.float32)
    ls = np.where(d[..., None] > 0, np.rint(scale / np.where(d > 0, d, 1)[..., None]), 0).clip(0, 63).astype(np.uint8)
    lm = np.where(dmin[..., None] > 0, np.rint(mins / np.where(dmin > 0, dmin, 1)[..., None]), 0).clip(0, 63).astype(np.uint8)
    eff_d = d[..., None] * ls
    eff_m = dmin[..., None] * lm
    q = np.where(eff_d[..., None] > 0, np.rint((b + eff_m[..., None]) / np.where(eff_d > 0, eff_d, 1)[..., None]), 0).clip(0, 15).astype(np.uint8)
    out = np.zeros((n, nb, 144), np.uint8)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:4] = _f16_bytes(dmin)
    sc = out[..., 4:16]
    sc[..., 0:4] = ls[..., 0:4] | ((ls[..., 4:8] >> 4) << 6)
    sc[..., 4:8] = lm[..., 0:4] | ((lm[..., 4:8] >> 4) << 6)
    sc[..., 8:12] = (ls[..., 4:8] & 15) | ((lm[..., 4:8] & 15) << 4)
    qq = q.reshape(n, nb, 4, 2, 32)
    out[..., 16:] = (qq[..., 0, :] | (qq[..., 1, :] << 4)).reshape(n, nb, 128)
    return out.reshape(n, -1)


def quantize_q6_k(w: np.ndarray) -> np.ndarray:
    n, k = w.shape
    nb = k // 256
    b = w.reshape(n, nb, 16, 16)
    scale = np.abs(b).max(axis=3) / np.float32(31.0)   # per group of 16, values in [-31, 31]
    d = (scale.max(axis=2) / np.float32(127.0)).astype(np.float16).astype(np.float32)
    sc = np.where(d[..., None] > 0, np.rint(scale / np.where(d > 0, d, 1)[..., None]), 0).clip(0, 127).astype(np.int8)
    eff = d[..., None] * sc
    q = (np.where(eff[..., None] > 0, np.rint(b / np.where(eff > 0, eff, 1)[..., None]), 0).clip(-32, 31) + 32).astype(np.uint8)
    L = q.reshape(n, nb, 2, 4, 32)                     # [half][group of 32][l]
    out = np.zeros((n, nb, 210), np.uint8)
    ql = out[..., 0:128].reshape(n, nb, 2, 64)
    qh = out[..., 128:192].reshape(n, nb, 2, 32)
    ql[..., 0:32] = (L[..., 0, :] & 15) | ((L[..., 2, :] & 15) << 4)
    ql[..., 32:64] = (L[..., 1, :] & 15) | ((L[..., 3, :] & 15) << 4)
    qh[...] = (L[..., 0, :] >> 4) | ((L[..., 1, :] >> 4) << 2) | ((L[..., 2, :] >> 4) << 4) | ((L[..., 3, :] >> 4) << 6)
    out[..., 0:128] = ql.reshape(n, nb, 128)
    out[..., 128:192] = qh.reshape(n, nb, 64)
    out[..., 192:208] = sc.view(np.uint8)
    out[..., 208:210] = _f16_bytes(d)
    return out.reshape(n, -1)


QUANTIZERS = {Q4_0: quantize_q4_0, Q8_0: quantize_q8_0, Q4_K: quantize_q4_k, Q6_K: quantize_q6_k}


def quantized_matrix(dtype: int, seed: int, n: int, k: int, chunk_rows: int = 2048) -> np.ndarray:
    """uint8 [n, row_bytes] natural blocks of seeded N(0, 0.02) weights, generated in row chunks."""
    parts = []
    for r0 in range(0, n, chunk_rows):
        r = min(chunk_rows, n - r0)
        parts.append(QUANTIZERS[dtype](gaussian_weights(seed * 7919 + r0, r, k)))
    return np.concatenate(parts, axis=0)
