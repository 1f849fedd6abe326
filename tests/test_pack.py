"""Packing contract of the B200 plane layout, modelled on the reference's R32 tests (tests/r32/r32_tests.cpp:61-183):
same byte count, unpack(pack(w)) == w for every shape including ragged ones, exact byte positions."""
import ctypes as C
import re
import os

import numpy as np
import pytest

from oracle import sgref
from scrapgpulibrary_b200 import capi, _build

QUANT = (16, 17, 32, 33)


@pytest.mark.parametrize("dtype", QUANT)
@pytest.mark.parametrize("shape", [(1, 1), (24, 1), (33, 3), (7, 5), (64, 16)])
def test_round_trip_random_bytes(dtype, shape):
    n, blocks = shape
    k = blocks * sgref.block_size(dtype)
    rb = sgref.row_bytes(dtype, k)
    raw = np.random.default_rng(n * 100 + blocks + dtype).integers(0, 256, size=(n, rb), dtype=np.uint8)
    packed = capi.pack(dtype, k, raw)
    assert packed.size == raw.size
    assert np.array_equal(capi.unpack(dtype, k, n, packed), raw)
    # a permutation (or re-encoding) that keeps every byte's information: distinct inputs stay distinct
    raw2 = raw.copy()
    raw2[n - 1, rb - 1] ^= 0x01
    assert not np.array_equal(capi.pack(dtype, k, raw2), packed)


def test_q4_0_byte_positions():
    # 3 rows x 2 blocks: quant bytes of block t at [16 t, 16 t + 16), scale of block t at 96 + 2 t
    k, n = 64, 3
    raw = np.arange(n * 2 * 18, dtype=np.uint8).reshape(n, 36)
    p = capi.pack(16, k, raw)
    blocks = raw.reshape(-1, 18)
    for t in range(6):
        assert np.array_equal(p[16 * t:16 * t + 16], blocks[t, 2:])
        assert np.array_equal(p[96 + 2 * t:98 + 2 * t], blocks[t, :2])


def test_q8_0_byte_positions():
    k, n = 32, 4
    raw = np.random.default_rng(0).integers(0, 256, size=(n, 34), dtype=np.uint8)
    p = capi.pack(17, k, raw)
    for t in range(n):
        assert np.array_equal(p[32 * t:32 * t + 32], raw[t, 2:])
        assert np.array_equal(p[32 * n + 2 * t:32 * n + 2 * t + 2], raw[t, :2])


def q4k_q_offset(n_rows, bpr, r, b, i):
    """Position of quant byte i of block b of row r in the tile-ordered Q plane (sm100_layout.h)."""
    full = n_rows // 16 * 16
    if r >= full:
        return full * bpr * 128 + ((r - full) * bpr + b) * 128 + i
    c = b * 4 + i // 32
    i32 = i % 32
    lane = (r % 8) * 4 + (i32 % 16) // 4
    return ((r // 16) * bpr * 4 + c) * 512 + lane * 16 + ((r // 8) % 2) * 8 + (i32 // 16) * 4 + i32 % 4


def test_q4_k_planes_and_scale_fields():
    k, n = 512, 19   # one full 16-row tile plus 3 leftover rows, two blocks per row
    raw = np.random.default_rng(1).integers(0, 256, size=(n, 288), dtype=np.uint8)
    p = capi.pack(32, k, raw)
    blocks = raw.reshape(n, 2, 144)
    T = n * 2
    for r in range(n):
        for b in range(2):
            for i in (0, 1, 3, 4, 15, 16, 31, 32, 77, 127):
                assert p[q4k_q_offset(n, 2, r, b, i)] == blocks[r, b, 16 + i], (r, b, i)
            h = p[128 * T + 16 * (r * 2 + b):128 * T + 16 * (r * 2 + b) + 16]
            assert np.array_equal(h[:4], blocks[r, b, :4])
            s = blocks[r, b, 4:16].astype(int)
            for pair in range(4):
                f = int(h[4 + 3 * pair]) | int(h[5 + 3 * pair]) << 8 | int(h[6 + 3 * pair]) << 16
                for e in range(2):
                    j = 2 * pair + e
                    if j < 4:
                        sc, mn = s[j] & 63, s[j + 4] & 63
                    else:
                        sc = (s[j + 4] & 15) | ((s[j - 4] >> 6) << 4)
                        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4)
                    assert (f >> (12 * e)) & 63 == sc and (f >> (12 * e + 6)) & 63 == mn
    # a warp's tile: 512 contiguous bytes, lane 4g + t = row g bytes [4t, 4t+4), [16+4t, 16+4t+4), then row g + 8
    tile = p[512 * 5:512 * 6]          # row tile 0, pair 5 = block 1, pair 1
    for g in range(8):
        for t in range(4):
            lane = tile[(4 * g + t) * 16:(4 * g + t) * 16 + 16]
            for half, row in ((0, g), (1, g + 8)):
                qs = blocks[row, 1, 16 + 32:16 + 64]
                assert np.array_equal(lane[8 * half:8 * half + 4], qs[4 * t:4 * t + 4])
                assert np.array_equal(lane[8 * half + 4:8 * half + 8], qs[16 + 4 * t:16 + 4 * t + 4])


def test_q6_k_planes():
    k, n = 512, 1
    raw = np.random.default_rng(2).integers(0, 256, size=(n, 420), dtype=np.uint8)
    p = capi.pack(33, k, raw)
    T = 2
    for t in range(T):
        blk = raw.reshape(-1, 210)[t]
        for h in range(2):
            for c in range(2):
                u = 2 * h + c
                assert np.array_equal(p[128 * t + 32 * u:128 * t + 32 * u + 16], blk[64 * h + 16 * c:64 * h + 16 * c + 16])
                assert np.array_equal(p[128 * t + 32 * u + 16:128 * t + 32 * u + 32], blk[64 * h + 32 + 16 * c:64 * h + 48 + 16 * c])
                assert np.array_equal(p[128 * T + 64 * T + 16 * t + 4 * u:128 * T + 64 * T + 16 * t + 4 * u + 4], blk[192 + 8 * h + c:192 + 8 * h + c + 7:2])
        assert np.array_equal(p[128 * T + 64 * t:128 * T + 64 * t + 64], blk[128:192])
        assert np.array_equal(p[208 * T + 2 * t:208 * T + 2 * t + 2], blk[208:210])


def test_pack_argument_errors():
    L = capi.lib()
    buf = np.zeros(256, np.uint8)
    p = buf.ctypes.data_as(C.c_void_p)
    assert L.sm100_pack(0, 32, 1, p, p) == 1          # F32 has no packed layout
    assert L.sm100_pack(32, 100, 1, p, p) == 2        # K not a whole number of blocks
    assert L.sm100_pack(32, 256, 1, None, p) == 2
    assert L.sm100_row_bytes(32, 4096) == 2304 and L.sm100_row_bytes(33, 4096) == 3360
    assert L.sm100_row_bytes(16, 4096) == 2304 and L.sm100_row_bytes(17, 4096) == 4352


def test_library_exports_every_declared_symbol():
    """Every function include/scrapgpu_sm100.h declares is exported by the built library."""
    header = open(os.path.join(_build.INCLUDE, "scrapgpu_sm100.h")).read()
    names = set(re.findall(r"SM100_API\s+[\w\s\*]+?\b(sm100_\w+)\s*\(", header))
    assert len(names) > 30
    L = capi.lib()
    missing = [n for n in sorted(names) if not hasattr(L, n)]
    assert not missing, missing
