"""Pins the CPU oracle (oracle/sgref.c) against the reference: the known answers of the reference's own unit
tests, the committed outputs of the compiled reference on seeded inputs (tests/golden/ref_seeded.npz), and,
where oracle/_ref/ is present, the compiled reference itself on fresh seeded inputs.  Runs without a GPU."""
import json
import os

import numpy as np
import pytest

from oracle import refapi, sgref
from scrapgpulibrary_b200 import abi

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
QUANT = (abi.Q4_0, abi.Q8_0, abi.Q4_K, abi.Q6_K)


@pytest.fixture(scope="module")
def gold():
    with open(os.path.join(GOLDEN, "ref_known_answers.json")) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def seeded():
    return np.load(os.path.join(GOLDEN, "ref_seeded.npz"))


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_known_answer_blocks(gold):
    for c in gold["dequant_blocks"]:
        got = sgref.dequantize(c["dtype"], np.array(c["block"], np.uint8)[None, :], len(c["values"]))[0]
        assert np.array_equal(got, np.array(c["values"], np.float32)), c["name"]


def test_f16_bits(gold):
    L = sgref.lib()
    for c in gold["f16_bits"]:
        assert L.sgref_float_to_half(c["value"]) == c["bits"]
    # every half value survives half -> float -> half (NaNs keep being NaNs)
    for h in range(0, 65536):
        f = L.sgref_half_to_float(h)
        back = L.sgref_float_to_half(f)
        if (h & 0x7C00) == 0x7C00 and (h & 0x3FF):
            assert (back & 0x7C00) == 0x7C00 and (back & 0x3FF)
        else:
            assert back == h
    assert np.array_equal(np.array([L.sgref_half_to_float(h) for h in range(0, 0x7C00)], np.float32),
                          np.arange(0, 0x7C00, dtype=np.uint16).view(np.float16).astype(np.float32))


def test_mul_mat_known_answers(gold):
    for c in gold["mul_mat"]:
        w = np.array(c["w"], np.float32)
        got = sgref.mul_mat(abi.F32, w.view(np.uint8).reshape(w.shape[0], -1), c["k"], np.array(c["x"], np.float32), threads=1)
        assert np.array_equal(got, np.array(c["y"], np.float32)), c["name"]


@pytest.mark.parametrize("dtype", QUANT, ids=lambda d: abi.DTYPE_NAMES[d])
def test_seeded_quant_and_mul_mat(seeded, dtype):
    nm = abi.DTYPE_NAMES[dtype]
    w, x = seeded["w"], seeded["x"]
    k = w.shape[1]
    q = sgref.quantize(dtype, w)
    assert np.array_equal(q, seeded[f"{nm}_blocks"])
    assert np.array_equal(bits(sgref.dequantize(dtype, q, k)), bits(seeded[f"{nm}_dequant"]))
    for m in (1, 3, 4, 8):
        assert np.array_equal(bits(sgref.mul_mat(dtype, q, k, x[:m])), bits(seeded[f"{nm}_mul_mat_m{m}"]))


def test_round_trip_error_bounds():
    """The bounds the reference states for quantize -> dequantize (tests/ref/ref_quant_tests.cpp:142-146), on
    its LCG inputs (:107-116) including the all-negative super-block."""
    def lcg(state, n):
        out = np.empty(n, np.float32)
        for i in range(n):
            state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
            out[i] = np.float32((np.float32(state >> 8) / np.float32(16777216.0) - np.float32(0.5)) * np.float32(2.0))
        return state, out

    for dtype, n, bound in ((abi.Q4_0, 32 * 7, 1 / 7), (abi.Q8_0, 32 * 5, 1 / 200), (abi.Q4_K, 256 * 3, 0.10), (abi.Q6_K, 256 * 3, 0.02)):
        state, x = lcg(12345 + dtype, n)
        x = (x * np.float32(3.0)).astype(np.float32)
        amax = float(np.abs(x).max())
        if abi.BLOCK[dtype][0] == 256:
            state, r = lcg(state, 256)
            x[:256] = -1.0 - 0.5 * np.abs(r)
            amax = max(amax, 1.5)
        y = sgref.dequantize(dtype, sgref.quantize(dtype, x[None, :]), n)[0]
        assert np.abs(x.astype(np.float64) - y).max() <= bound * amax
    z = sgref.dequantize(abi.Q4_0, sgref.quantize(abi.Q4_0, np.zeros((1, 32), np.float32)), 32)
    assert np.all(z == 0.0)


def test_argument_errors():
    L = sgref.lib()
    buf = np.zeros(64, np.uint8)
    y = np.zeros(64, np.float32)
    p = lambda a: a.ctypes.data
    assert L.sgref_dequantize(abi.Q4_0, p(buf), p(y), 31) == abi.INVALID_ARGUMENT   # ref_quant_tests.cpp:160-176
    assert L.sgref_quantize(abi.Q8_0, p(y), p(buf), 33) == abi.INVALID_ARGUMENT
    assert L.sgref_dequantize(abi.F32, p(buf), p(y), 4) == abi.UNSUPPORTED
    assert L.sgref_dequantize(abi.Q4_0, None, p(y), 32) == abi.INVALID_ARGUMENT
    assert L.sgref_dequantize(abi.Q4_0, p(buf), p(y), 0) == abi.INVALID_ARGUMENT


def test_seeded_norms(seeded):
    a, b, w = seeded["norm_a"], seeded["norm_b"], seeded["norm_w"]
    assert np.array_equal(bits(sgref.rms_norm(a)), bits(seeded["rms_norm"]))
    assert np.array_equal(bits(sgref.rms_norm(a, w)), bits(seeded["rms_norm_mul"]))
    s, y = sgref.rms_norm(a, w, add=b)
    assert np.array_equal(bits(s), bits(seeded["add_rms_norm_mul_sum"]))
    assert np.array_equal(bits(y), bits(seeded["add_rms_norm_mul"]))


def test_seeded_rope(seeded):
    x, pos = seeded["rope_x"], seeded["rope_pos"]
    for mode, nd in ((abi.ROPE_NEOX, 64), (abi.ROPE_NORMAL, 64), (abi.ROPE_NEOX, 32)):
        got = sgref.rope(x, pos, nd, neox=(mode == abi.ROPE_NEOX), freq_base=1e6)
        assert np.array_equal(bits(got), bits(seeded[f"rope_mode{mode}_nd{nd}"]))


def test_seeded_softmax_glu(seeded):
    x, mk = seeded["softmax_x"], seeded["softmax_mask"]
    assert np.array_equal(bits(sgref.soft_max(x, mk, 0.125)), bits(seeded["softmax_masked"]))
    assert np.array_equal(bits(sgref.soft_max(x, None, 0.125)), bits(seeded["softmax_plain"]))
    assert np.array_equal(bits(sgref.swiglu(seeded["glu_x"], seeded["glu_g"])), bits(seeded["swiglu"]))


def test_seeded_attention(seeded):
    q, k, v = seeded["att_q"], seeded["att_k"], seeded["att_v"]
    s = float(1.0 / np.sqrt(32.0))
    assert np.array_equal(bits(sgref.attention(q, k, v, True, 29, s)), bits(seeded["att_causal_off29"]))
    assert np.array_equal(bits(sgref.attention(q, k, v, False, 0, s)), bits(seeded["att_full"]))
    assert np.array_equal(bits(sgref.attention(seeded["att_q3"], k, v, True, 2, 0.2)), bits(seeded["att_causal_q3_off2"]))


def test_argmax_ties():
    x = np.array([1, 5, 3, 5, 2], np.float32)
    assert sgref.argmax(x) == 1  # lowest index wins (src/core/ref/ops.cpp:1189-1228: stable descending sort)


@pytest.mark.skipif(not refapi.available(), reason="oracle/_ref/ is not built here")
@pytest.mark.parametrize("dtype", QUANT, ids=lambda d: abi.DTYPE_NAMES[d])
def test_against_compiled_reference(dtype):
    rng = np.random.default_rng(1234 + dtype)
    k, n = 2048, 40
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    w[1] *= 1000.0
    q = sgref.quantize(dtype, w)
    assert np.array_equal(q, refapi.quantize(dtype, w))
    assert np.array_equal(bits(sgref.dequantize(dtype, q, k)), bits(refapi.dequantize(dtype, q, k)))
    for m in (1, 2, 4, 7, 8):
        x = rng.standard_normal((m, k)).astype(np.float32)
        assert np.array_equal(bits(sgref.mul_mat(dtype, q, k, x)), bits(refapi.mul_mat(dtype, q, k, x)))
