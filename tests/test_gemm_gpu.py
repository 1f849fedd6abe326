"""GPU parity of the prefill MUL_MAT (M > 32: tcgen05 tensor-core GEMM) through the C ABI against the CPU oracle.

Tolerance: NMSE <= 1e-6 (tests/ops/ops_tests.cpp:725 of the reference; the benchmark's north star repeats it).
The kernel multiplies f16 roundings of the weights and of the per-token normalised activations, so the
expected NMSE is about 2e-7.
"""
import numpy as np
import pytest

from oracle import sgref
from tests import util as U

pytestmark = pytest.mark.gpu
TOL = 1e-6

# (K, N, M): one chunk; a K with a half chunk at the end and ragged N and M; several token tiles;
# a long K; N below one tile
SHAPES = [(64, 128, 33), (96, 130, 100), (512, 257, 129), (4096, 256, 64), (12288, 40, 48)]


def _check(sm100, stream, dtype, layout, k, n, m, seed=0):
    wq = U.quantize(dtype, U.seeded_weights(2000 + dtype + k + seed, n, k))
    x = U.seeded_acts(11 * m + k + seed, m, k)
    want = sgref.mul_mat(dtype, wq, k, x)
    got = U.device_mul_mat(sm100, stream, dtype, layout, wq, k, x)
    assert np.isfinite(got).all()
    e = sgref.nmse(got, want)
    assert e <= TOL, f"{U.NAMES[dtype]} layout {layout} K={k} N={n} M={m}: NMSE {e:.3e}"
    # per token too: a token tile or a row tile that went wrong must not hide in the average
    for t in range(m):
        et = sgref.nmse(got[t], want[t])
        assert et <= 4 * TOL, f"token {t}: NMSE {et:.3e}"


@pytest.mark.parametrize("dtype", [U.Q8_0, U.Q4_0], ids=lambda d: U.NAMES[d])
@pytest.mark.parametrize("layout", [U.NATURAL, U.PACKED], ids=["natural", "packed"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"k{s[0]}n{s[1]}m{s[2]}")
def test_gemm_block32_formats(sm100, stream, dtype, layout, shape):
    k, n, m = shape
    _check(sm100, stream, dtype, layout, k, n, m)


@pytest.mark.parametrize("shape", [(256, 24, 40), (512, 130, 100), (4096, 256, 64), (12288, 48, 33)],
                         ids=lambda s: f"k{s[0]}n{s[1]}m{s[2]}")
def test_gemm_q4_k_packed(sm100, stream, shape):
    k, n, m = shape
    _check(sm100, stream, U.Q4_K, U.PACKED, k, n, m)


@pytest.mark.parametrize("shape", [(64, 128, 33), (160, 70, 90), (4096, 256, 64)], ids=lambda s: f"k{s[0]}n{s[1]}m{s[2]}")
def test_gemm_f16_weights(sm100, stream, shape):
    k, n, m = shape
    _check(sm100, stream, U.F16, U.NATURAL, k, n, m)


@pytest.mark.parametrize("dtype,layout", [(U.Q6_K, U.PACKED), (U.Q4_K, U.NATURAL), (U.F32, U.NATURAL)],
                         ids=["q6_k_packed", "q4_k_natural", "f32"])
def test_wide_batches_without_a_tensor_core_source_still_work(sm100, stream, dtype, layout):
    """Formats the GEMM does not read take the matvec in column panels of 8."""
    _check(sm100, stream, dtype, layout, 512, 40, 40)


def test_gemm_token_magnitudes(sm100, stream):
    """Tokens of very different magnitude in one batch: each is normalised on its own, so each keeps
    the tolerance (a plain f16 conversion would overflow the first and flush the second to zero)."""
    k, n, m = 1024, 256, 64
    wq = U.quantize(U.Q8_0, U.seeded_weights(5, n, k))
    x = U.seeded_acts(6, m, k)
    x[0] *= 1e7
    x[1] *= 1e-9
    x[2] = 0.0
    x[3, 5] = 3e4
    want = sgref.mul_mat(U.Q8_0, wq, k, x)
    got = U.device_mul_mat(sm100, stream, U.Q8_0, U.PACKED, wq, k, x)
    assert np.all(got[2] == 0.0)
    for t in (0, 1, 3, 4, 63):
        assert sgref.nmse(got[t], want[t]) <= TOL, t


@pytest.mark.parametrize("n", [4096, 12288])
def test_gemm_q8_0_prefill_shapes(sm100, stream, n):
    """M = 512 x K = 4096 x N in {4096, 12288}, the prefill configuration of the benchmark.  The oracle
    checks a seeded sample of weight rows (rows are independent); the whole output is compared with the
    decode matvec run over the same weights in column panels, and linearity W(a + b) = Wa + Wb holds."""
    k, m = 4096, 512
    wq = U.quantize(U.Q8_0, U.seeded_weights(77 + n, n, k))
    x = U.seeded_acts(78, m, k)
    got = U.device_mul_mat(sm100, stream, U.Q8_0, U.PACKED, wq, k, x)
    rows = np.sort(np.random.default_rng(n).choice(n, 160, replace=False))
    want = sgref.mul_mat(U.Q8_0, np.ascontiguousarray(wq[rows]), k, x)
    assert sgref.nmse(got[:, rows], want) <= TOL
    panels = np.concatenate([U.device_mul_mat(sm100, stream, U.Q8_0, U.PACKED, wq, k, x[c:c + 8]) for c in range(0, 64, 8)])
    assert sgref.nmse(got[:64], panels) <= TOL
    s = np.concatenate([x[:40] + x[40:80], x[:40]])
    gs = U.device_mul_mat(sm100, stream, U.Q8_0, U.PACKED, wq, k, s)
    assert sgref.nmse(gs[:40], got[:40] + got[40:80]) <= TOL
    assert sgref.nmse(gs[40:], got[:40]) <= 1e-12


@pytest.mark.parametrize("tn,rt,tmem_a", [(128, 1, 1), (256, 1, 1), (128, 2, 1), (128, 1, 0), (256, 1, 0), (128, 2, 0), (256, 2, 0)],
                         ids=lambda v: str(v))
def test_gemm_forced_tiles(sm100, tn, rt, tmem_a):
    """Every variant of the kernel (tokens per tile x row tiles per CTA x weights staged in tensor or shared memory)
    on ragged shapes: the variant is chosen from the problem size, so small problems reach the others only when a
    child process pins them."""
    import json
    import os
    import subprocess
    import sys
    env = dict(os.environ, SM100_GEMM_TN=str(tn), SM100_GEMM_RT=str(rt), SM100_GEMM_TMEM_A=str(tmem_a))
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gemm_tiles_worker.py")
    r = subprocess.run([sys.executable, worker], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    res = json.loads(r.stdout.strip().splitlines()[-1])
    assert res["cases"] == 6
    assert res["worst"] <= TOL, res
