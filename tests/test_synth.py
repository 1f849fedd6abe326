"""The benchmark's synthetic blocks are valid: the oracle's dequantizer recovers the seeded weights within the
round-trip bounds the reference states for its own quantizers (tests/ref/ref_quant_tests.cpp:142-146)."""
import numpy as np
import pytest

from oracle import sgref
from scrapgpulibrary_b200 import synth


@pytest.mark.parametrize("dtype,bound", [(16, 1 / 7), (17, 1 / 200), (32, 0.10), (33, 0.04)])
def test_synthetic_blocks_decode(dtype, bound):
    n, k = 24, 1024
    w = synth.gaussian_weights(5, n, k)
    w[2, :256] = 0
    q = synth.QUANTIZERS[dtype](w)
    assert q.shape == (n, sgref.row_bytes(dtype, k))
    y = sgref.dequantize(dtype, q, k)
    assert np.abs(y - w).max() <= bound * np.abs(w).max()
    assert np.all(y[2, :256] == 0)


def test_q4_0_q8_0_match_oracle_quantizer():
    w = synth.gaussian_weights(6, 8, 512)
    assert np.array_equal(synth.quantize_q4_0(w), sgref.quantize(16, w))
    assert np.array_equal(synth.quantize_q8_0(w), sgref.quantize(17, w))
