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
    equals the device-resident call bit for bit (same kernels), for matvec and for a small batch."""
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
        assert np.array_equal(got, want), m
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
