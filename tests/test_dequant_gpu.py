"""Bit-exact dequantization on the GPU (GET_ROWS over all four block formats, both layouts) against the
oracle, plus the hand-built blocks of the reference's own unit tests (tests/ref/ref_quant_tests.cpp:23-105)."""
import ctypes as C
import json
import os

import numpy as np
import pytest

from oracle import sgref
from tests import util as U

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def device_get_rows(capi, stream, dtype, layout, table: np.ndarray, k: int, ids: np.ndarray) -> np.ndarray:
    n = table.shape[0]
    img = capi.pack(dtype, k, table) if layout == U.PACKED else np.ascontiguousarray(table).ravel()
    tb = U.to_device(capi, stream, img)
    ib = U.to_device(capi, stream, ids.astype(np.int32))
    ob, optr = U.guarded_output(capi, stream, ids.size * k)
    capi.check(capi.lib().sm100_get_rows(stream.handle, dtype, layout, tb.at(), 0, k, n, ib.at(), ids.size, C.c_void_p(optr), k), "get_rows")
    stream.sync()
    out = U.read_guarded(capi, stream, ob, ids.size * k).reshape(ids.size, k).copy()
    for b in (tb, ib, ob):
        b.free()
    return out


@pytest.mark.parametrize("dtype", U.QUANT, ids=lambda d: U.NAMES[d])
@pytest.mark.parametrize("layout", [U.NATURAL, U.PACKED], ids=["natural", "packed"])
def test_dequant_bit_exact(sm100, stream, dtype, layout):
    k, n = 1024, 96
    w = U.seeded_weights(31 + dtype, n, k)
    w[3, :256] = 0.0                                  # an all-zero block
    w[5, :256] = -1.0 - 0.5 * np.abs(w[5, :256])      # an all-negative block (exercises the Q4_K min)
    w[7] *= 300.0                                     # large scales
    q = U.quantize(dtype, w)
    ids = np.array([5, 0, 95, 3, 3, 7, 42], dtype=np.int32)
    want = sgref.dequantize(dtype, q, k)[ids]
    got = device_get_rows(sm100, stream, dtype, layout, q, k, ids)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("dtype", U.QUANT, ids=lambda d: U.NAMES[d])
def test_dequant_random_bytes_bit_exact(sm100, stream, dtype):
    """Arbitrary block bytes (every scale / nibble pattern, subnormal and large fp16 scales; NaN/Inf scales
    excluded by clearing the top exponent bit) decode to the oracle's bits."""
    k, n = 512, 64
    rb = sgref.row_bytes(dtype, k)
    raw = np.random.default_rng(77 + dtype).integers(0, 256, size=(n, rb), dtype=np.uint8)
    bb = sgref.type_size(dtype)
    blocks = raw.reshape(-1, bb)
    for off in {U.Q4_0: (1,), U.Q8_0: (1,), U.Q4_K: (1, 3), U.Q6_K: (209,)}[dtype]:
        blocks[:, off] &= 0xBF  # exponent < 16: finite halves
    ids = np.arange(n, dtype=np.int32)
    want = sgref.dequantize(dtype, raw, k)
    for layout in (U.NATURAL, U.PACKED):
        got = device_get_rows(sm100, stream, dtype, layout, raw, k, ids)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"layout {layout}"


def test_reference_known_answer_blocks(sm100, stream):
    with open(os.path.join(GOLDEN, "ref_known_answers.json")) as f:
        gold = json.load(f)
    for case in gold["dequant_blocks"]:
        dtype = case["dtype"]
        blk = np.array(case["block"], dtype=np.uint8)[None, :]
        k = sgref.block_size(dtype)
        want = np.array(case["values"], dtype=np.float32)
        for layout in (U.NATURAL, U.PACKED):
            got = device_get_rows(sm100, stream, dtype, layout, blk, k, np.zeros(1, dtype=np.int32))[0]
            assert np.array_equal(got, want), case["name"]


def test_get_rows_float_tables(sm100, stream):
    k, n = 96, 10
    w = U.seeded_weights(3, n, k)
    ids = np.array([9, 0, 4], dtype=np.int32)
    got = device_get_rows(sm100, stream, U.F32, U.NATURAL, U.quantize(U.F32, w), k, ids)
    assert np.array_equal(got, w[ids])
    got = device_get_rows(sm100, stream, U.F16, U.NATURAL, U.quantize(U.F16, w), k, ids)
    assert np.array_equal(got, w.astype(np.float16).astype(np.float32)[ids])
