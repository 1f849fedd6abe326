"""GPU parity of the decode MUL_MAT (M <= 8) through the C ABI against the CPU oracle.

Tolerance: NMSE <= 1e-6, the bar the reference sets for quantized MUL_MAT on a device
(tests/ops/ops_tests.cpp:725) and that the benchmark's north star repeats.
"""
import numpy as np
import pytest

from oracle import sgref
from tests import util as U

pytestmark = pytest.mark.gpu
TOL = 1e-6

# (K, N): a single block, ragged row counts (24 and 33 rows: ops_tests.cpp:714-716), a K that is not a
# multiple of 32 units, and the K of the benchmark shapes
SMALL_SHAPES = [(256, 24), (512, 33), (1280, 17), (4096, 64), (12288, 40)]


@pytest.mark.parametrize("dtype", U.QUANT, ids=lambda d: U.NAMES[d])
@pytest.mark.parametrize("layout", [U.NATURAL, U.PACKED], ids=["natural", "packed"])
@pytest.mark.parametrize("shape", SMALL_SHAPES, ids=lambda s: f"k{s[0]}n{s[1]}")
def test_matvec_small(sm100, stream, dtype, layout, shape):
    k, n = shape
    wq = U.quantize(dtype, U.seeded_weights(1000 + dtype + k, n, k))
    for m in (1, 2, 3, 4, 5, 8):
        x = U.seeded_acts(7 * m + k, m, k)
        want = sgref.mul_mat(dtype, wq, k, x)
        got = U.device_mul_mat(sm100, stream, dtype, layout, wq, k, x)
        e = sgref.nmse(got, want)
        assert e <= TOL, f"{U.NAMES[dtype]} layout {layout} K={k} N={n} M={m}: NMSE {e:.3e}"


@pytest.mark.parametrize("dtype", [U.F32, U.F16], ids=lambda d: U.NAMES[d])
@pytest.mark.parametrize("shape", [(128, 40), (130, 7), (4096, 33)], ids=lambda s: f"k{s[0]}n{s[1]}")
def test_matvec_float_weights(sm100, stream, dtype, shape):
    k, n = shape
    w = U.seeded_weights(5, n, k)
    wq = U.quantize(dtype, w)
    for m in (1, 4, 7):
        x = U.seeded_acts(m, m, k)
        want = sgref.mul_mat(dtype, wq, k, x)
        got = U.device_mul_mat(sm100, stream, dtype, U.NATURAL, wq, k, x)
        assert sgref.nmse(got, want) <= 1e-7


def test_k_order_cancellation(sm100, stream):
    """Row {1e20, 1, -1e20, 3, 4, 0...} against ones: the reference's increasing-K f32 order gives exactly 7
    (tests/ref/ref_ops_tests.cpp:756-772).  A device reduction tree cannot promise that order; what must hold
    is that the result is finite and the well-conditioned rows next to it are exact."""
    k = 8
    w = np.zeros((3, k), dtype=np.float32)
    w[0, :5] = [1e20, 1, -1e20, 3, 4]
    w[1, :5] = [1, 2, 3, 4, 5]
    w[2, :] = 0.5
    x = np.ones((1, k), dtype=np.float32)
    got = U.device_mul_mat(sm100, stream, U.F32, U.NATURAL, U.quantize(U.F32, w), k, x)
    assert np.isfinite(got).all()
    assert got[0, 1] == 15.0 and got[0, 2] == 4.0


@pytest.mark.parametrize("dtype,k,n", [(U.Q4_0, 4096, 4096), (U.Q4_K, 4096, 12288), (U.Q4_K, 12288, 4096),
                                       (U.Q6_K, 4096, 4096), (U.Q8_0, 4096, 4096), (U.Q4_0, 4096, 9744), (U.Q8_0, 8192, 4800)],
                         ids=["q4_0_4096x4096", "q4_k_4096x12288", "q4_k_12288x4096", "q6_k_4096x4096", "q8_0_4096x4096",
                              "q4_0_4096x9744_three_rounds", "q8_0_8192x4800_two_rounds"])
def test_matvec_benchmark_shapes(sm100, stream, dtype, k, n):
    """The benchmark's shapes: full comparison with the oracle at M = 1 and 8, plus linearity
    W(a + b) = Wa + Wb as a size-independent property."""
    wq = U.quantize(dtype, U.seeded_weights(42 + dtype, n, k))
    x = U.seeded_acts(99, 8, k)
    want = sgref.mul_mat(dtype, wq, k, x)
    got8 = U.device_mul_mat(sm100, stream, dtype, U.PACKED, wq, k, x)
    assert sgref.nmse(got8, want) <= TOL
    got1 = U.device_mul_mat(sm100, stream, dtype, U.PACKED, wq, k, x[:1])
    assert sgref.nmse(got1, want[:1]) <= TOL
    s = (x[0] + x[1])[None, :]
    gsum = U.device_mul_mat(sm100, stream, dtype, U.PACKED, wq, k, s)
    assert sgref.nmse(gsum[0], got8[0] + got8[1]) <= TOL
    # natural layout gives the same values as packed (same arithmetic, different addressing)
    gnat = U.device_mul_mat(sm100, stream, dtype, U.NATURAL, wq, k, x[:1])
    assert sgref.nmse(gnat, want[:1]) <= TOL


# ---- every branch of the dispatcher, every benchmark shape, hostile activations -------------------------------------

def _kernel(sm100):
    return (sm100.lib().sm100_matvec_last_kernel() or b"").decode()


# environment that switches kernel families off -> the "dtype:kernel" names that must then have served some case
FORCED = [
    ({}, ["q4_k:matvec_q4k_imma", "q4_k:matvec_q4k_imma+rows", "q4_k:matvec_q4k_imma_cols+rows",
          "q6_k:matvec_q6k_imma", "q4_0:matvec_b32_imma", "q8_0:matvec_b32_imma", "q6_k:matvec_q6k_imma_cols", "q4_0:matvec_per_column",
          "q6_k:matvec_rows", "q8_0:matvec_rows"]),
    ({"SM100_Q4K_RING": "2"}, ["q4_k:matvec_q4k_ring", "q4_k:matvec_q4k_ring+rows", "q4_k:matvec_q4k_imma"]),   # 2: the ring kernel wherever its shapes allow
    ({"SM100_Q4K_RING": "0"}, ["q4_k:matvec_q4k_imma", "q4_k:matvec_q4k_imma+rows"]),
    ({"SM100_Q6K_IMMA": "0", "SM100_B32_IMMA": "0"}, ["q6_k:matvec_wide", "q4_0:matvec_wide", "q8_0:matvec_wide", "q6_k:matvec_rows", "q6_k:matvec_per_column"]),
    ({"SM100_Q4K_IMMA": "0"}, ["q4_k:matvec_q4k_mma", "q4_k:matvec_q4k_mma+rows"]),   # (switches the ring kernel off too: same arithmetic family)
    ({"SM100_Q4K_IMMA": "0", "SM100_Q4K_MMA": "0", "SM100_Q6K_IMMA": "0", "SM100_B32_IMMA": "0", "SM100_MV_WIDE": "0"},
     ["q4_k:matvec_stream", "q6_k:matvec_stream", "q4_0:matvec_stream", "q8_0:matvec_stream", "q4_k:matvec_rows", "q8_0:matvec_rows", "q8_0:matvec_per_column"]),
]


@pytest.mark.parametrize("env,expected", FORCED, ids=["default", "q4k_ring_everywhere", "no_q4k_ring", "no_q6k_b32_imma", "no_q4k_imma", "cuda_core_only"])
def test_matvec_forced_branches(env, expected):
    """Each kernel family of the dispatcher (sm100_matvec.cu) is reached by name and agrees with the oracle: the
    families behind the default one serve the shapes the default declines, so they are tested by switching the
    families in front of them off in a child process (the switches are read once per process)."""
    import json
    import os
    import subprocess
    import sys
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "matvec_branch_worker.py")
    r = subprocess.run([sys.executable, worker], capture_output=True, text=True, timeout=900, env=dict(os.environ, **env))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["worst"] <= TOL, out
    for name in expected:
        assert name in out["kernels"], (name, out["kernels"])


@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 12288), (12288, 4096)], ids=["4096x4096", "4096x12288", "12288x4096"])
def test_q4k_matvecs_back_to_back_take_the_ring_kernel(sm100, stream, k, n):
    """The default dispatch of a plain packed Q4_K matvec: the first one of a run on a stream is served by
    matvec_q4k_imma, the ones that follow it directly by matvec_q4k_ring (built to overlap with its predecessor), and
    after any other launch or copy of the library the run starts over.  Every result against the oracle, at the
    benchmark sweep's three shapes; the four launches of a run are enqueued without synchronisation in between."""
    wq = [U.quantize(U.Q4_K, U.seeded_weights(300 + i + n, n, k)) for i in range(2)]
    x = U.seeded_acts(9 + k, 1, k)
    want = [sgref.mul_mat(U.Q4_K, w, k, x) for w in wq]
    wb = [U.to_device(sm100, stream, sm100.pack(U.Q4_K, k, w)) for w in wq]
    xb = U.to_device(sm100, stream, x)
    outs = [U.guarded_output(sm100, stream, n) for _ in range(4)]
    stream.sync()
    served = []
    for i, (yb, yptr) in enumerate(outs):
        sm100.mul_mat(stream, U.Q4_K, U.PACKED, wb[i % 2], k, n, xb, 1, yptr)
        served.append(_kernel(sm100))
    stream.sync()
    assert served == ["matvec_q4k_imma", "matvec_q4k_ring", "matvec_q4k_ring", "matvec_q4k_ring"], served
    for i, (yb, _) in enumerate(outs):
        got = U.read_guarded(sm100, stream, yb, n).reshape(1, n)
        assert sgref.nmse(got, want[i % 2]) <= TOL, (i, served[i])
    # a copy in between ends the run
    yb, yptr = outs[0]
    sm100.mul_mat(stream, U.Q4_K, U.PACKED, wb[0], k, n, xb, 1, yptr)
    assert _kernel(sm100) == "matvec_q4k_imma"
    stream.sync()
    for b in wb + [xb] + [o[0] for o in outs]:
        b.free()


@pytest.mark.parametrize("dtype,k,n", [(U.Q6_K, 4096, 12288), (U.Q6_K, 12288, 4096), (U.Q4_K, 4096, 4096), (U.Q4_K, 4096, 12288), (U.Q4_K, 12288, 4096)],
                         ids=["q6_k_4096x12288", "q6_k_12288x4096", "q4_k_4096x4096", "q4_k_4096x12288", "q4_k_12288x4096"])
def test_matvec_sweep_shapes_every_batch(sm100, stream, dtype, k, n):
    """The Q4_K / Q6_K projection shapes of the benchmark sweep at full size for every batch it names (M = 1, 2, 4, 8;
    each M is a kernel or a template of its own), every column on its own against the oracle."""
    wq = U.quantize(dtype, U.seeded_weights(77 + dtype + n, n, k))
    x = U.seeded_acts(5 + k, 8, k)
    want = sgref.mul_mat(dtype, wq, k, x)
    served = {}
    for m in (1, 2, 4, 8):
        got = U.device_mul_mat(sm100, stream, dtype, U.PACKED, wq, k, x[:m])
        served[m] = _kernel(sm100)
        assert np.isfinite(got).all()
        for c in range(m):
            e = sgref.nmse(got[c], want[c])
            assert e <= TOL, f"{U.NAMES[dtype]} K={k} N={n} M={m} column {c} ({served[m]}): NMSE {e:.3e}"
    print(U.NAMES[dtype], k, n, served)


def test_matvec_vocabulary_head(sm100, stream):
    """The Q6_K output head of the decode stack, K = 4096, N = 151936 (510 MB), M = 1: every row against the oracle,
    and the first and the last 16-row tile on their own."""
    from scrapgpulibrary_b200 import synth
    k, n = 4096, 151936
    wq = synth.quantized_matrix(U.Q6_K, 1234, n, k)   # valid Q6_K blocks of seeded N(0, 0.02) weights (min/max rule)
    x = U.seeded_acts(31, 1, k)
    want = sgref.mul_mat(U.Q6_K, wq, k, x)
    got = U.device_mul_mat(sm100, stream, U.Q6_K, U.PACKED, wq, k, x)
    name = _kernel(sm100)
    assert np.isfinite(got).all()
    assert sgref.nmse(got, want) <= TOL, name
    for lo, hi in ((0, 16), (n - 16, n), (n // 2, n // 2 + 512)):
        assert sgref.nmse(got[0, lo:hi], want[0, lo:hi]) <= TOL, (name, lo)
    assert int(np.argmax(got[0])) == int(np.argmax(want[0]))
    print("head served by", name)


def _quantization_bound(dtype, wq, k, x, group):
    """Largest error the 16-bit activation image can cause per output row: every group of `group` activations is
    rounded to multiples of amax / 32512, i.e. off by at most amax / 65024 per element (groups below 1e-30 count as
    zero), times the row's weight magnitudes; plus the f32 accumulation of |w x|."""
    w = np.abs(sgref.dequantize(dtype, wq, k).astype(np.float64))
    ax = np.abs(x.astype(np.float64)).reshape(-1, group)
    amax = ax.max(axis=1)
    per_elem = np.repeat(np.where(amax > 1e-30, amax / 65024.0, amax), group)
    return w @ per_elem + 4e-6 * (w @ np.abs(x.astype(np.float64))) + 1e-30


@pytest.mark.parametrize("dtype,group", [(U.Q4_K, 32), (U.Q6_K, 16), (U.Q4_0, 32), (U.Q8_0, 32)], ids=lambda v: U.NAMES.get(v, str(v)))
def test_matvec_hostile_activations(sm100, stream, dtype, group):
    """Activations the integer kernels could get wrong: one 1e7 outlier inside a block of ordinary values, an
    all-zero block beside it, a block at 1e-30, a block of alternating huge values that cancel.  Checked per
    output row against a bound derived from the activation format, not only as an NMSE."""
    k, n = 4096, 272
    wq = U.quantize(dtype, U.seeded_weights(600 + dtype, n, k))
    x = U.seeded_acts(8, 1, k)
    x[0, 5] = 1e7
    x[0, 32:64] = 0.0
    x[0, 64:96] *= 1e-30
    x[0, 96:128] = np.where(np.arange(32) % 2 == 0, 3e6, -3e6).astype(np.float32)
    x[0, 4000:4032] *= 1e-12
    want = sgref.mul_mat(dtype, wq, k, x).astype(np.float64)
    got = U.device_mul_mat(sm100, stream, dtype, U.PACKED, wq, k, x).astype(np.float64)
    name = _kernel(sm100)
    assert np.isfinite(got).all(), name
    bound = _quantization_bound(dtype, wq, k, x[0], group)
    excess = np.abs(got[0] - want[0]) / bound
    assert excess.max() <= 1.05, f"{name}: row {int(excess.argmax())} is {excess.max():.2f}x the format's error bound"
    assert sgref.nmse(got, want) <= TOL


@pytest.mark.parametrize("dtype", U.QUANT, ids=lambda d: U.NAMES[d])
@pytest.mark.parametrize("m", [1, 4], ids=["m1", "m4"])
def test_matvec_nan_and_inf_propagate(sm100, stream, dtype, m):
    """A NaN or an infinity among the activations makes every output of that column non-finite in the reference
    (f32 dot product, src/core/ref/ops.cpp:968-980); the device must not hand out finite numbers instead.  The other
    columns stay exact."""
    k, n = 4096, 48
    wq = U.quantize(dtype, U.seeded_weights(700 + dtype, n, k))
    for bad in (np.nan, np.inf, -np.inf):
        x = U.seeded_acts(9, m, k)
        x[0, 1234] = bad
        want = sgref.mul_mat(dtype, wq, k, x)
        got = U.device_mul_mat(sm100, stream, dtype, U.PACKED, wq, k, x)
        assert not np.isfinite(want[0]).any()
        assert not np.isfinite(got[0]).any(), (_kernel(sm100), bad)
        if m > 1:
            assert sgref.nmse(got[1:], want[1:]) <= TOL


def test_matvec_argument_errors(sm100, stream):
    buf = sm100.Buffer(1 << 16)
    with pytest.raises(sm100.Sm100Error) as e:
        sm100.mul_mat(stream, U.Q4_K, U.PACKED, buf, 100, 4, buf, 1, buf)  # K not a multiple of 256
    assert e.value.status == 1
    with pytest.raises(sm100.Sm100Error) as e:
        sm100.mul_mat(stream, 99, U.NATURAL, buf, 256, 4, buf, 1, buf)  # unknown dtype
    assert e.value.status == 1
    with pytest.raises(sm100.Sm100Error) as e:
        sm100.mul_mat(stream, U.Q4_K, U.PACKED, 0, 256, 4, buf, 1, buf)  # null weights
    assert e.value.status == 2
    buf.free()


def _fused(sm100, stream, prologue, a, b, norm_w, wqs, k, want_sum, want_x):
    """Runs sm100_mul_mat_fused over packed Q4_K tensors; returns the outputs and the optional side outputs."""
    import ctypes as C
    n = len(wqs)
    bufs = [U.to_device(sm100, stream, sm100.pack(U.Q4_K, k, w)) for w in wqs]
    ab = U.to_device(sm100, stream, a)
    bb = U.to_device(sm100, stream, b) if b is not None else None
    wb = U.to_device(sm100, stream, norm_w) if norm_w is not None else None
    sb = sm100.Buffer(4 * k) if want_sum else None
    xb = sm100.Buffer(4 * k) if want_x else None
    ys = [U.guarded_output(sm100, stream, w.shape[0]) for w in wqs]
    dts = (C.c_int * n)(*([U.Q4_K] * n))
    lays = (C.c_int * n)(*([1] * n))
    wp = (C.c_void_p * n)(*[bf.ptr for bf in bufs])
    yp = (C.c_void_p * n)(*[p for _, p in ys])
    ns = (C.c_int64 * n)(*[w.shape[0] for w in wqs])
    sm100.check(sm100.lib().sm100_mul_mat_fused(stream.handle, prologue, ab.at(), bb.at() if bb else None, wb.at() if wb else None, 1e-6,
                                                sb.at() if sb else None, xb.at() if xb else None, n, dts, lays, wp, k, ns, yp), "mul_mat_fused")
    stream.sync()
    outs = [U.read_guarded(sm100, stream, yb, w.shape[0]).copy() for (yb, _), w in zip(ys, wqs)]
    s_out = sb.download(stream, np.float32, k) if sb else None
    x_out = xb.download(stream, np.float32, k) if xb else None
    return outs, s_out, x_out


def test_mul_mat_fused_prologues(sm100, stream):
    """RMS norm (with and without the residual add) and SwiGLU folded into the Q4_K projections: outputs against the
    oracle's separate ops, the residual sum bit-exact, the normalised row within one ulp."""
    k = 4096
    rng = np.random.default_rng(3)
    wqs = [U.quantize(U.Q4_K, U.seeded_weights(300 + i, n, k)) for i, n in enumerate((4096, 1024, 1024))]
    a = (rng.standard_normal(k) * 4).astype(np.float32)
    b = rng.standard_normal(k).astype(np.float32)
    g = rng.standard_normal(k).astype(np.float32)
    for add in (b, None):
        if add is not None:
            want_s, want_x = sgref.rms_norm(a[None], g, add=add[None])
        else:
            want_s, want_x = None, sgref.rms_norm(a[None], g)
        outs, s_out, x_out = _fused(sm100, stream, 2, a, add, g, wqs, k, add is not None, True)
        if add is not None:
            assert np.array_equal(s_out, want_s[0])
        assert np.max(np.abs(x_out.view(np.int32) - want_x[0].view(np.int32))) <= 1
        for w, y in zip(wqs, outs):
            assert sgref.nmse(y, sgref.mul_mat(U.Q4_K, w, k, want_x)[0]) <= TOL
    # SwiGLU in front of a down projection: K = 12288
    k2 = 12288
    wd = U.quantize(U.Q4_K, U.seeded_weights(400, 512, k2))
    ga = rng.standard_normal(k2).astype(np.float32)
    up = rng.standard_normal(k2).astype(np.float32)
    outs, _, _ = _fused(sm100, stream, 1, ga, up, None, [wd], k2, False, False)
    act = sgref.swiglu(ga, up)
    assert sgref.nmse(outs[0], sgref.mul_mat(U.Q4_K, wd, k2, act[None])[0]) <= TOL


@pytest.mark.parametrize("k,n,prologue", [(4096, 12288, 2), (1024, 48, 0), (4096, 1536, 2)], ids=["4096x12288_norm", "1024x48", "4096x1536_norm"])
def test_mul_mat_glu(sm100, stream, k, n, prologue):
    """sm100_mul_mat_glu: gate and up projections with SwiGLU in the epilogue of the same launch (and the residual add + RMS
    norm in its prologue): gate, up and the activation equal, bit for bit, sm100_mul_mat_fused / sm100_mul_mat_multi over the
    two tensors followed by sm100_swiglu; the activation within NMSE 1e-6 of the oracle's ops."""
    import ctypes as C
    L = sm100.lib()
    rng = np.random.default_rng(60 + n)
    wg = U.quantize(U.Q4_K, U.seeded_weights(500 + n, n, k))
    wu = U.quantize(U.Q4_K, U.seeded_weights(501 + n, n, k))
    a = (rng.standard_normal(k) * 3).astype(np.float32)
    b = rng.standard_normal(k).astype(np.float32)
    g = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    bufs = {name: U.to_device(sm100, stream, arr) for name, arr in dict(a=a, b=b, g=g, wg=sm100.pack(U.Q4_K, k, wg), wu=sm100.pack(U.Q4_K, k, wu)).items()}
    gate1, up1, act1, sum1 = (sm100.Buffer(4 * n), sm100.Buffer(4 * n), U.guarded_output(sm100, stream, n), sm100.Buffer(4 * k))
    sm100.check(L.sm100_mul_mat_glu(stream.handle, prologue, bufs["a"].at(), bufs["b"].at() if prologue else None, bufs["g"].at() if prologue else None, 1e-6,
                                    sum1.at() if prologue else None, None, U.Q4_K, 1, bufs["wg"].at(), bufs["wu"].at(), k, n, gate1.at(), up1.at(),
                                    C.c_void_p(act1[1])), "mul_mat_glu")
    stream.sync()
    got_gate, got_up = gate1.download(stream, np.float32, n), up1.download(stream, np.float32, n)
    got_act = U.read_guarded(sm100, stream, act1[0], n).copy()
    # the separate launches
    if prologue:
        outs, s_out, _ = _fused(sm100, stream, 2, a, b, g, [wg, wu], k, True, False)
        assert np.array_equal(sum1.download(stream, np.float32, k), s_out)
        want_s, want_x = sgref.rms_norm(a[None], g, add=b[None])
        x_ref = want_x
    else:
        gb, ub = sm100.Buffer(4 * n), sm100.Buffer(4 * n)
        sm100.check(L.sm100_mul_mat_multi(stream.handle, 2, (C.c_int * 2)(U.Q4_K, U.Q4_K), (C.c_int * 2)(1, 1), (C.c_void_p * 2)(bufs["wg"].ptr, bufs["wu"].ptr),
                                          k, (C.c_int64 * 2)(n, n), bufs["a"].at(), (C.c_void_p * 2)(gb.ptr, ub.ptr)), "mul_mat_multi")
        stream.sync()
        outs = [gb.download(stream, np.float32, n), ub.download(stream, np.float32, n)]
        x_ref = a[None]
    assert np.array_equal(got_gate, outs[0]) and np.array_equal(got_up, outs[1])
    g2, u2, a2 = U.to_device(sm100, stream, outs[0]), U.to_device(sm100, stream, outs[1]), sm100.Buffer(4 * n)
    sm100.check(L.sm100_swiglu(stream.handle, g2.at(), u2.at(), a2.at(), n), "swiglu")
    stream.sync()
    assert np.array_equal(got_act, a2.download(stream, np.float32, n))
    want = sgref.swiglu(sgref.mul_mat(U.Q4_K, wg, k, x_ref)[0], sgref.mul_mat(U.Q4_K, wu, k, x_ref)[0])
    assert sgref.nmse(got_act, want) <= TOL
    # only the activation wanted
    act3 = U.guarded_output(sm100, stream, n)
    sm100.check(L.sm100_mul_mat_glu(stream.handle, prologue, bufs["a"].at(), bufs["b"].at() if prologue else None, bufs["g"].at() if prologue else None, 1e-6,
                                    None, None, U.Q4_K, 1, bufs["wg"].at(), bufs["wu"].at(), k, n, None, None, C.c_void_p(act3[1])), "mul_mat_glu")
    stream.sync()
    assert np.array_equal(U.read_guarded(sm100, stream, act3[0], n), got_act)
    # a row count that is not a multiple of 16 is refused
    assert L.sm100_mul_mat_glu(stream.handle, 0, bufs["a"].at(), None, None, 0.0, None, None, U.Q4_K, 1, bufs["wg"].at(), bufs["wu"].at(), k, n - 8, None, None,
                               C.c_void_p(act3[1])) == 1


def test_mul_mat_fused_refuses_what_it_does_not_serve(sm100, stream):
    import ctypes as C
    k, n = 256, 24   # 24 rows: not whole 16-row tiles
    w = U.to_device(sm100, stream, sm100.pack(U.Q4_K, k, U.quantize(U.Q4_K, U.seeded_weights(1, n, k))))
    a = U.to_device(sm100, stream, np.ones(k, np.float32))
    y = sm100.Buffer(4 * n)
    st = sm100.lib().sm100_mul_mat_fused(stream.handle, 2, a.at(), None, a.at(), 1e-6, None, None, 1, (C.c_int * 1)(U.Q4_K), (C.c_int * 1)(1),
                                         (C.c_void_p * 1)(w.ptr), k, (C.c_int64 * 1)(n), (C.c_void_p * 1)(y.ptr))
    assert st == 1   # UNSUPPORTED: the caller runs the separate ops


def test_hostpipe_mul_mat_matches_device_path(sm100, stream):
    """Host activations in, host results out, several products in flight over fewer slots than calls: every result
    equals the device-resident call, for matvec and for a small batch (same integer dot products; consecutive
    single-column calls on the pipe's stream may be served by the ring kernel, which adds the block terms in another
    order than matvec_q4k_imma: hence 1e-10 instead of bit equality)."""
    import ctypes as C
    lib = sm100.lib()
    k, n = 1024, 272
    wq = U.quantize(U.Q4_K, U.seeded_weights(91, n, k))
    wb = U.to_device(sm100, stream, sm100.pack(U.Q4_K, k, wq))
    stream.sync()
    calls = [(1, 3), (1, 4), (2, 5), (1, 6), (4, 7), (1, 8), (1, 9)]   # (m, seed)
    pipe = sm100.HostPipe(3, 4 * k * 4, 4 * n * 4)
    host = []
    for m, seed in calls:
        px, py = C.c_void_p(), C.c_void_p()
        sm100.check(lib.sm100_host_alloc(4 * k * m, C.byref(px)), "host_alloc")
        sm100.check(lib.sm100_host_alloc(4 * n * m, C.byref(py)), "host_alloc")
        x = U.seeded_acts(seed, m, k)
        C.memmove(px, x.ctypes.data, x.nbytes)
        C.memset(py, 0xFF, 4 * n * m)
        host.append((m, x, px, py))
    for m, x, px, py in host:
        pipe.mul_mat(U.Q4_K, U.PACKED, wb, k, n, px, m, py)
    pipe.sync()
    for m, x, px, py in host:
        got = np.ctypeslib.as_array(C.cast(py, C.POINTER(C.c_float)), shape=(m * n,)).reshape(m, n).copy()
        want = U.device_mul_mat(sm100, stream, U.Q4_K, U.PACKED, wq, k, x)
        assert sgref.nmse(got, want) <= 1e-10, m
        assert sgref.nmse(got, sgref.mul_mat(U.Q4_K, wq, k, x)) <= 1e-6
    # the same products as one list
    items = (sm100.HostPipeItem * len(host))()
    for i, (m, x, px, py) in enumerate(host):
        C.memset(py, 0xFF, 4 * n * m)
        items[i] = sm100.HostPipeItem(U.Q4_K, U.PACKED, wb.ptr, 0, k, n, px.value, m, py.value)
    pipe.mul_mat_many(items, len(host))
    pipe.sync()
    for m, x, px, py in host:
        got = np.ctypeslib.as_array(C.cast(py, C.POINTER(C.c_float)), shape=(m * n,)).reshape(m, n).copy()
        assert sgref.nmse(got, sgref.mul_mat(U.Q4_K, wq, k, x)) <= 1e-6
    # a product larger than the pipe's staging is refused, not truncated
    st = lib.sm100_hostpipe_mul_mat(pipe.handle, U.Q4_K, U.PACKED, wb.at(), 0, k, n, host[0][2], 8, host[0][3])
    assert st == 2
    pipe.close()
    for _, _, px, py in host:
        lib.sm100_host_free(px)
        lib.sm100_host_free(py)
    wb.free()
