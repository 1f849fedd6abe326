"""GPU parity of the decode ops around the matvec (RMS_NORM family, ROPE, SOFT_MAX, SwiGLU, ADD, SET_ROWS,
arg-max, fused attention) through the C ABI: against the committed outputs of the compiled reference
(tests/golden/ref_seeded.npz) and against the CPU oracle on larger seeded inputs.

Tolerances: exact bits for ADD / SET_ROWS / arg-max and for the RMS_NORM family (same IEEE operations, the
double-precision sum of squares differs from the sequential one only far below f32 resolution);
NMSE <= 1e-6 (north star) -- in practice ~1e-13 -- for ROPE, SOFT_MAX, SwiGLU and attention, whose cos / sin /
exp come from the CUDA math library rather than glibc."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import sgref
from tests import util as U

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
TOL = 1e-6


@pytest.fixture(scope="module")
def seeded():
    return np.load(os.path.join(GOLDEN, "ref_seeded.npz"))


def vp(x):
    return C.c_void_p(x.ptr if hasattr(x, "ptr") else x)


def run_rms(capi, stream, x, w=None, add=None, eps=1e-6):
    rows, ne0 = x.shape
    xb = U.to_device(capi, stream, x)
    wb = U.to_device(capi, stream, w) if w is not None else None
    ab = U.to_device(capi, stream, add) if add is not None else None
    sb, sptr = U.guarded_output(capi, stream, x.size)
    yb, yptr = U.guarded_output(capi, stream, x.size)
    capi.check(capi.lib().sm100_rms_norm(stream.handle, xb.at(), ab.at() if ab else None, wb.at() if wb else None,
                                         C.c_void_p(sptr) if add is not None else None, C.c_void_p(yptr), ne0, rows, eps), "rms_norm")
    stream.sync()
    y = U.read_guarded(capi, stream, yb, x.size).reshape(x.shape).copy()
    s = U.read_guarded(capi, stream, sb, x.size).reshape(x.shape).copy()
    return s, y


def test_rms_norm_family(sm100, stream, seeded):
    a, b, w = seeded["norm_a"], seeded["norm_b"], seeded["norm_w"]
    _, y = run_rms(sm100, stream, a)
    assert np.array_equal(y, seeded["rms_norm"])
    _, y = run_rms(sm100, stream, a, w)
    assert np.array_equal(y, seeded["rms_norm_mul"])
    s, y = run_rms(sm100, stream, a, w, b)
    assert np.array_equal(s, seeded["add_rms_norm_mul_sum"])
    assert np.array_equal(y, seeded["add_rms_norm_mul"])
    # decode sizes: hidden 4096 and per-head 128
    for rows, ne0 in ((1, 4096), (40, 128), (3, 12288)):
        x = U.seeded_acts(rows, rows, ne0) * 5
        g = U.seeded_acts(11, 1, ne0)[0]
        r = U.seeded_acts(12, rows, ne0)
        ws, wy = sgref.rms_norm(x, g, add=r)
        s, y = run_rms(sm100, stream, x, g, r)
        assert np.array_equal(s, ws)
        assert sgref.nmse(y, wy) <= 1e-12 and np.max(np.abs(y.view(np.int32) - wy.view(np.int32))) <= 1


def run_rope(capi, stream, x, pos, n_dims, neox, base, table=None, first=0):
    tokens, heads, ne0 = x.shape
    xb, pb = U.to_device(capi, stream, x), U.to_device(capi, stream, pos.astype(np.int32))
    yb, yptr = U.guarded_output(capi, stream, x.size)
    if table is None:
        capi.check(capi.lib().sm100_rope_direct(stream.handle, xb.at(), pb.at(), C.c_void_p(yptr), ne0, heads, tokens, n_dims, int(neox),
                                                base, 1.0, 1.0), "rope_direct")
    else:
        tb = U.to_device(capi, stream, table)
        capi.check(capi.lib().sm100_rope(stream.handle, xb.at(), pb.at(), tb.at(), first, table.shape[0], C.c_void_p(yptr), ne0, heads, tokens,
                                         n_dims, int(neox)), "rope")
    stream.sync()
    return U.read_guarded(capi, stream, yb, x.size).reshape(x.shape).copy()


def test_rope(sm100, stream, seeded):
    x, pos = seeded["rope_x"], seeded["rope_pos"]
    for mode, nd in ((1, 64), (0, 64), (1, 32)):
        want = seeded[f"rope_mode{mode}_nd{nd}"]
        got = run_rope(sm100, stream, x, pos, nd, mode == 1, 1e6)
        assert sgref.nmse(got, want) <= TOL
        # with the reference-recipe table the rotation is bit exact
        table = sgref.rope_table(pos, nd, 1e6)
        for i, p in enumerate(pos):
            g = run_rope(sm100, stream, x[i:i + 1], pos[i:i + 1], nd, mode == 1, 1e6, table[i:i + 1], int(p))
            assert np.array_equal(g, want[i:i + 1])
    # decode shape: 32 heads of 128 at position 1024 + t, table covering 1024..1151
    xq = U.seeded_acts(5, 32, 128).reshape(1, 32, 128)
    positions = np.arange(1024, 1152)
    table = sgref.rope_table(positions, 128, 1e6)
    for p in (1024, 1100, 1151):
        want = sgref.rope(xq, np.array([p], np.int32), 128, True, 1e6)
        got = run_rope(sm100, stream, xq, np.array([p], np.int32), 128, True, 1e6, table, 1024)
        assert np.array_equal(got, want)


def run_softmax(capi, stream, x, mask, scale, in_place=False):
    rows, ne0 = x.shape
    mb = U.to_device(capi, stream, mask) if mask is not None else None
    if in_place:
        xb, xptr = U.guarded_output(capi, stream, x.size)
        capi.check(capi.lib().sm100_memcpy_h2d(stream.handle, C.c_void_p(xptr), x.ctypes.data_as(C.c_void_p), x.nbytes, 1), "h2d")
        yb, yptr = xb, xptr
    else:
        xb = U.to_device(capi, stream, x)
        xptr = xb.ptr
        yb, yptr = U.guarded_output(capi, stream, x.size)
    capi.check(capi.lib().sm100_soft_max(stream.handle, C.c_void_p(xptr), mb.at() if mb else None, ne0, C.c_void_p(yptr), ne0, rows, scale), "soft_max")
    stream.sync()
    return U.read_guarded(capi, stream, yb, x.size).reshape(x.shape).copy()


def test_soft_max(sm100, stream, seeded):
    x, mk = np.ascontiguousarray(seeded["softmax_x"]), np.ascontiguousarray(seeded["softmax_mask"])
    assert sgref.nmse(run_softmax(sm100, stream, x, mk, 0.125), seeded["softmax_masked"]) <= TOL
    assert sgref.nmse(run_softmax(sm100, stream, x, None, 0.125), seeded["softmax_plain"]) <= TOL
    assert sgref.nmse(run_softmax(sm100, stream, x, mk, 0.125, in_place=True), seeded["softmax_masked"]) <= TOL
    big = U.seeded_acts(1, 32, 1152) * 6
    assert sgref.nmse(run_softmax(sm100, stream, big, None, 0.088), sgref.soft_max(big, None, 0.088)) <= TOL


def test_swiglu_add(sm100, stream, seeded):
    lib = sm100.lib()
    for x, g, want in ((seeded["glu_x"], seeded["glu_g"], seeded["swiglu"]),):
        xb, gb = U.to_device(sm100, stream, x), U.to_device(sm100, stream, g)
        yb, yptr = U.guarded_output(sm100, stream, x.size)
        sm100.check(lib.sm100_swiglu(stream.handle, xb.at(), gb.at(), C.c_void_p(yptr), x.size), "swiglu")
        stream.sync()
        assert sgref.nmse(U.read_guarded(sm100, stream, yb, x.size), want) <= TOL
    a, b = U.seeded_acts(1, 1, 12288)[0] * 4, U.seeded_acts(2, 1, 12288)[0]
    ab, bb = U.to_device(sm100, stream, a), U.to_device(sm100, stream, b)
    yb, yptr = U.guarded_output(sm100, stream, a.size)
    sm100.check(lib.sm100_swiglu(stream.handle, ab.at(), bb.at(), C.c_void_p(yptr), a.size), "swiglu")
    stream.sync()
    assert sgref.nmse(U.read_guarded(sm100, stream, yb, a.size), sgref.swiglu(a, b)) <= TOL
    sm100.check(lib.sm100_add(stream.handle, ab.at(), bb.at(), C.c_void_p(yptr), a.size), "add")
    stream.sync()
    assert np.array_equal(U.read_guarded(sm100, stream, yb, a.size), sgref.add(a, b))


def test_set_rows_and_argmax(sm100, stream):
    lib = sm100.lib()
    ne0, heads, n_ctx = 128, 8, 64
    cache = np.zeros((heads, n_ctx, ne0), np.float32)
    src = U.seeded_acts(3, heads, ne0).reshape(heads, 1, ne0)
    cb, sb = U.to_device(sm100, stream, cache), U.to_device(sm100, stream, src)
    ib = U.to_device(sm100, stream, np.array([37], np.int32))
    sm100.check(lib.sm100_set_rows(stream.handle, sb.at(), ib.at(), cb.at(), ne0, 1, heads, n_ctx), "set_rows")
    stream.sync()
    got = cb.download(stream, np.float32, cache.size).reshape(cache.shape)
    want = cache.copy()
    want[:, 37, :] = src[:, 0, :]
    assert np.array_equal(got, want)

    for n in (5, 1000, 151936):
        x = U.seeded_acts(n, 1, n)[0]
        x[n // 2] = x[n - 1] = x.max() + 1.0  # a tie: the lower index must win
        xb = U.to_device(sm100, stream, x)
        ob = U.to_device(sm100, stream, np.array([-1], np.int32))
        sm100.check(lib.sm100_argmax(stream.handle, xb.at(), n, ob.at()), "argmax")
        stream.sync()
        assert int(ob.download(stream, np.int32, 1)[0]) == sgref.argmax(x) == n // 2
    # a vector that does not start on a 16-byte boundary, ties inside one 16-byte group and in the ragged tail
    x = U.seeded_acts(99, 1, 4100)[0]
    x[[1001, 1002, 4098]] = x.max() + 2.0
    xb = U.to_device(sm100, stream, x)
    for skip, want in ((1, 1000), (0, 1001), (1003, 4098 - 1003)):
        sm100.check(lib.sm100_argmax(stream.handle, C.c_void_p(xb.ptr + 4 * skip), 4100 - skip, ob.at()), "argmax")
        stream.sync()
        assert int(ob.download(stream, np.int32, 1)[0]) == want == sgref.argmax(x[skip:])


def run_attention(capi, stream, q, k, v, causal, offset, scale, positions=None, mask=None, mask_heads=1):
    hq, nq, d = q.shape
    hkv, nk, _ = k.shape
    dv = v.shape[2]
    qb, kb, vb = (U.to_device(capi, stream, a) for a in (q, k, v))
    ob, optr = U.guarded_output(capi, stream, hq * nq * dv)
    pb = U.to_device(capi, stream, np.asarray(positions, np.int32)) if positions is not None else None
    mb = U.to_device(capi, stream, mask) if mask is not None else None
    capi.check(capi.lib().sm100_attention(stream.handle, qb.at(), kb.at(), vb.at(), mb.at() if mb else None, mask_heads, C.c_void_p(optr), d, dv, nq, nk,
                                          hq, hkv, int(causal), offset, pb.at() if pb else None, scale), "attention")
    stream.sync()
    return U.read_guarded(capi, stream, ob, hq * nq * dv).reshape(hq, nq, dv).copy()


def test_attention_golden(sm100, stream, seeded):
    q, k, v = seeded["att_q"], seeded["att_k"], seeded["att_v"]
    s = float(1.0 / np.sqrt(32.0))
    assert sgref.nmse(run_attention(sm100, stream, q, k, v, True, 29, s), seeded["att_causal_off29"]) <= TOL
    assert sgref.nmse(run_attention(sm100, stream, q, k, v, False, 0, s), seeded["att_full"]) <= TOL
    assert sgref.nmse(run_attention(sm100, stream, seeded["att_q3"], k, v, True, 2, 0.2), seeded["att_causal_q3_off2"]) <= TOL
    # offset taken from a device-side position (graph replay reads it there)
    assert sgref.nmse(run_attention(sm100, stream, q, k, v, True, 0, s, positions=[29]), seeded["att_causal_off29"]) <= TOL


def test_attention_decode_shape(sm100, stream):
    """Qwen3-8B-shaped decode attention: 32 query heads on 8 KV heads, head_dim 128, f32 cache of 1152
    positions zero beyond the current one, causal offset 1024 + t."""
    hq, hkv, d, n_ctx = 32, 8, 128, 1152
    rng = np.random.default_rng(8)
    for t in (0, 57, 127):
        n_valid = 1024 + t + 1
        k = np.zeros((hkv, n_ctx, d), np.float32)
        v = np.zeros((hkv, n_ctx, d), np.float32)
        k[:, :n_valid] = rng.standard_normal((hkv, n_valid, d))
        v[:, :n_valid] = rng.standard_normal((hkv, n_valid, d))
        q = rng.standard_normal((hq, 1, d)).astype(np.float32)
        want = sgref.attention(q, k, v, True, 1024 + t, 1.0 / np.sqrt(d))
        got = run_attention(sm100, stream, q, k, v, True, 1024 + t, float(1.0 / np.sqrt(d)))
        assert sgref.nmse(got, want) <= TOL
        assert np.max(np.abs(got - want)) <= 3e-4  # the reference's own absolute bound (tests/attention/attention_tests.cpp:40)


def test_attention_masks(sm100, stream):
    hq, hkv, d, nk, nq = 4, 2, 32, 50, 2
    rng = np.random.default_rng(9)
    q = rng.standard_normal((hq, nq, d)).astype(np.float32)
    k = rng.standard_normal((hkv, nk, d)).astype(np.float32)
    v = rng.standard_normal((hkv, nk, d)).astype(np.float32)
    # an additive mask that hides every key of query 1: the output row must be zero (attention.cpp:497-516)
    mask = np.zeros((1, nq, nk), np.float32)
    mask[0, 0, 10:] = -np.inf
    mask[0, 1, :] = -np.inf
    got = run_attention(sm100, stream, q, k, v, False, 0, 0.3, mask=mask, mask_heads=1)
    want0 = sgref.attention(q[:, :1], k[:, :10], v[:, :10], False, 0, 0.3)
    assert sgref.nmse(got[:, :1], want0) <= TOL
    assert np.all(got[:, 1] == 0.0)


def test_attention_graph_survives_scratch_growth(sm100, stream):
    """A captured graph names the library's scratch block by address.  A later, larger call makes the library
    allocate a bigger block; the earlier block must stay valid (it is never freed or moved), so a replay of the
    graph afterwards still gives the right result."""
    import ctypes as C
    lib = sm100.lib()
    hq, hkv, d, nk = 32, 8, 128, 1152
    rng = np.random.default_rng(12)
    q = rng.standard_normal((hq, 1, d)).astype(np.float32)
    k = rng.standard_normal((hkv, nk, d)).astype(np.float32)
    v = rng.standard_normal((hkv, nk, d)).astype(np.float32)
    scale = float(1.0 / np.sqrt(d))
    want = sgref.attention(q, k, v, True, 1100, scale)
    qb, kb, vb = (U.to_device(sm100, stream, a) for a in (q, k, v))
    ob, optr = U.guarded_output(sm100, stream, hq * d)

    def enqueue():
        sm100.check(lib.sm100_attention(stream.handle, qb.at(), kb.at(), vb.at(), None, 1, C.c_void_p(optr), d, d, 1, nk, hq, hkv, 1, 1100, None, scale), "attention")
    enqueue()              # outside the capture: the scratch block comes into being
    stream.sync()
    with sm100.Graph(stream) as g:
        enqueue()
    g.launch()
    stream.sync()
    assert sgref.nmse(U.read_guarded(sm100, stream, ob, hq * d).reshape(hq, 1, d), want) <= TOL
    # a prefill-sized call: 640 queries x 32 heads x (128 + 4) floats per split is beyond the 8 MiB the first block has
    nq2 = 640
    q2 = rng.standard_normal((hq, nq2, d)).astype(np.float32)
    got2 = run_attention(sm100, stream, q2, k[:, :256], v[:, :256], True, 0, scale)
    assert sgref.nmse(got2, sgref.attention(q2, k[:, :256], v[:, :256], True, 0, scale)) <= TOL
    # dirty everything the allocator could have recycled, then replay the old graph
    junk = [sm100.Buffer(8 << 20) for _ in range(4)]
    for j in junk:
        sm100.check(lib.sm100_memset(stream.handle, j.at(), 0x7F, 8 << 20, 1), "memset")
    sm100.check(lib.sm100_memset(stream.handle, C.c_void_p(optr), 0, 4 * hq * d, 1), "memset")
    g.launch()
    stream.sync()
    assert sgref.nmse(U.read_guarded(sm100, stream, ob, hq * d).reshape(hq, 1, d), want) <= TOL
    g.destroy()
    for b in junk + [qb, kb, vb, ob]:
        b.free()


def test_attention_argument_errors(sm100, stream):
    b = sm100.Buffer(1 << 16)
    lib = sm100.lib()
    st = lib.sm100_attention(stream.handle, b.at(), b.at(), b.at(), None, 1, b.at(), 32, 32, 1, 8, 5, 2, 1, 0, None, 1.0)
    assert st == 2  # Hq not divisible by Hkv
    st = lib.sm100_attention(stream.handle, None, b.at(), b.at(), None, 1, b.at(), 32, 32, 1, 8, 4, 2, 1, 0, None, 1.0)
    assert st == 2
    b.free()


@pytest.mark.parametrize("with_norm", [True, False], ids=["qk_norm", "no_norm"])
def test_head_post_matches_separate_reference_ops(sm100, stream, with_norm):
    """The fused decode step (per-head RMS_NORM_MUL, ROPE from the table, SET_ROWS_PAIR into the caches) against the
    oracle's separate ops: 32 query heads, 8 KV heads of 128, cache of 64 rows, positions inside and outside the table."""
    d, hq, hkv, rows = 128, 32, 8, 64
    rng = np.random.default_rng(77)
    qw = rng.standard_normal(d).astype(np.float32)
    kw = rng.standard_normal(d).astype(np.float32)
    table_pos = np.arange(16, 48)
    table = sgref.rope_table(table_pos, d, 1e6)
    for pos in (16, 40, 47, 5, 63):
        q = (rng.standard_normal((hq, d)) * 3).astype(np.float32)
        k = (rng.standard_normal((hkv, d)) * 3).astype(np.float32)
        v = rng.standard_normal((hkv, d)).astype(np.float32)
        kc = rng.standard_normal((hkv, rows, d)).astype(np.float32)
        vc = rng.standard_normal((hkv, rows, d)).astype(np.float32)
        qn = sgref.rms_norm(q, qw) if with_norm else q
        kn = sgref.rms_norm(k, kw) if with_norm else k
        p = np.array([pos], np.int32)
        want_q = sgref.rope(qn.reshape(1, hq, d), p, d, True, 1e6)[0]
        want_k = sgref.rope(kn.reshape(1, hkv, d), p, d, True, 1e6)[0]
        bufs = {n: U.to_device(sm100, stream, a) for n, a in dict(q=q, k=k, v=v, kc=kc, vc=vc, qw=qw, kw=kw, t=table, p=p).items()}
        sm100.check(sm100.lib().sm100_head_post(stream.handle, bufs["q"].at(), bufs["k"].at(), bufs["v"].at(),
                                                bufs["qw"].at() if with_norm else None, bufs["kw"].at() if with_norm else None,
                                                bufs["p"].at(), bufs["t"].at(), 16, len(table_pos), bufs["kc"].at(), bufs["vc"].at(),
                                                d, hq, hkv, rows, 1e-6, 1e6, 1), "head_post")
        stream.sync()
        got_q = bufs["q"].download(stream, np.float32, q.size).reshape(q.shape)
        got_k = bufs["k"].download(stream, np.float32, k.size).reshape(k.shape)
        got_kc = bufs["kc"].download(stream, np.float32, kc.size).reshape(kc.shape)
        got_vc = bufs["vc"].download(stream, np.float32, vc.size).reshape(vc.shape)
        in_table = 16 <= pos < 48
        tol = 1e-12 if in_table else TOL   # outside the table the device evaluates cosf / sinf itself
        assert sgref.nmse(got_q, want_q) <= tol and sgref.nmse(got_k, want_k) <= tol
        if in_table and not with_norm:
            assert np.array_equal(got_q, want_q) and np.array_equal(got_k, want_k)
        want_kc, want_vc = kc.copy(), vc.copy()
        want_kc[:, pos] = got_k
        want_vc[:, pos] = v
        assert np.array_equal(got_kc, want_kc) and np.array_equal(got_vc, want_vc)
        for b in bufs.values():
            b.free()


@pytest.mark.parametrize("hq,hkv,d,rows,with_norm", [(32, 8, 128, 1200, True), (32, 8, 128, 96, False), (8, 4, 256, 300, True), (4, 4, 128, 64, True)],
                         ids=lambda v: str(v))
def test_attention_decode_one_launch(sm100, stream, hq, hkv, d, rows, with_norm):
    """sm100_attention_decode (per-head norm + rotation of the new token's Q and K, K / V stored into the caches, attention
    over the cache, in one launch) against sm100_head_post + sm100_attention_kvcache on the same inputs and against the
    oracle's separate ops: caches equal (the new K row up to the order of additions in the norm's sum: NMSE 1e-12), outputs
    within 1e-6, for positions inside and outside the rotation table, first and last row of the cache included."""
    rng = np.random.default_rng(hq * 100 + rows)
    L = sm100.lib()
    qw = rng.standard_normal(d).astype(np.float32)
    kw = rng.standard_normal(d).astype(np.float32)
    first, count = 4, rows - 8
    table = sgref.rope_table(np.arange(first, first + count), d, 1e6)
    scale = float(1.0 / np.sqrt(d))
    for pos in (0, first, rows // 2, rows - 5, rows - 1):
        q = (rng.standard_normal((hq, d)) * 2).astype(np.float32)
        k = (rng.standard_normal((hkv, d)) * 2).astype(np.float32)
        v = rng.standard_normal((hkv, d)).astype(np.float32)
        kc = rng.standard_normal((hkv, rows, d)).astype(np.float32)
        vc = rng.standard_normal((hkv, rows, d)).astype(np.float32)
        p = np.array([pos], np.int32)
        res = []
        for fused in (True, False):
            b = {n: U.to_device(sm100, stream, a) for n, a in dict(q=q, k=k, v=v, kc=kc, vc=vc, qw=qw, kw=kw, t=table, p=p).items()}
            ob, optr = U.guarded_output(sm100, stream, hq * d)
            if fused:
                sm100.check(L.sm100_attention_decode(stream.handle, b["q"].at(), b["k"].at(), b["v"].at(), b["qw"].at() if with_norm else None,
                                                     b["kw"].at() if with_norm else None, b["p"].at(), b["t"].at(), first, count, b["kc"].at(),
                                                     b["vc"].at(), C.c_void_p(optr), d, hq, hkv, rows, 1e-6, 1e6, 1, scale), "attention_decode")
            else:
                sm100.check(L.sm100_head_post(stream.handle, b["q"].at(), b["k"].at(), b["v"].at(), b["qw"].at() if with_norm else None,
                                              b["kw"].at() if with_norm else None, b["p"].at(), b["t"].at(), first, count, b["kc"].at(), b["vc"].at(),
                                              d, hq, hkv, rows, 1e-6, 1e6, 1), "head_post")
                sm100.check(L.sm100_attention_kvcache(stream.handle, b["q"].at(), b["kc"].at(), b["vc"].at(), None, 1, C.c_void_p(optr), d, d, 1, rows,
                                                      hq, hkv, 1, 0, b["p"].at(), scale, 1), "attention_kvcache")
            stream.sync()
            res.append((U.read_guarded(sm100, stream, ob, hq * d).reshape(hq, d).copy(),
                        b["kc"].download(stream, np.float32, kc.size).reshape(kc.shape), b["vc"].download(stream, np.float32, vc.size).reshape(vc.shape)))
            for x in list(b.values()) + [ob]:
                x.free()
        (o1, kc1, vc1), (o2, kc2, vc2) = res
        assert np.array_equal(vc1, vc2)
        other = np.ones(rows, bool)
        other[pos] = False
        assert np.array_equal(kc1[:, other], kc2[:, other]) and np.array_equal(kc1[:, other], kc[:, other])
        assert sgref.nmse(kc1[:, pos], kc2[:, pos]) <= 1e-12
        assert sgref.nmse(o1, o2) <= 1e-10, pos
        # the oracle's separate ops
        qn = sgref.rms_norm(q, qw) if with_norm else q
        qr = sgref.rope(qn.reshape(1, hq, d), p, d, True, 1e6)[0]
        want = sgref.attention(qr.reshape(hq, 1, d), kc2[:, :pos + 1], vc2[:, :pos + 1], False, 0, scale).reshape(hq, d)
        assert sgref.nmse(o1, want) <= TOL, pos


@pytest.mark.parametrize("hq,hkv,d,nk,nq", [(8, 8, 128, 300, 1), (8, 4, 128, 777, 2), (32, 8, 128, 1500, 1), (16, 2, 256, 130, 3), (4, 4, 256, 64, 1)],
                         ids=lambda v: str(v))
def test_attention_single_pass_kernel(sm100, stream, hq, hkv, d, nk, nq):
    """Head dimensions 128 / 256 with 1, 2, 4, 8 query heads per KV head take the single-pass kernel with the merge
    of the splits folded in: causal with an offset (from the host and from the device), full, and masked."""
    rng = np.random.default_rng(hq * 1000 + nk)
    q = rng.standard_normal((hq, nq, d)).astype(np.float32)
    k = rng.standard_normal((hkv, nk, d)).astype(np.float32)
    v = rng.standard_normal((hkv, nk, d)).astype(np.float32)
    s = float(1.0 / np.sqrt(d))
    off = nk - nq - 7
    want = sgref.attention(q, k, v, True, off, s)
    assert sgref.nmse(run_attention(sm100, stream, q, k, v, True, off, s), want) <= TOL
    assert sgref.nmse(run_attention(sm100, stream, q, k, v, True, 0, s, positions=[off]), want) <= TOL
    # twice in a row: the merge counters of the first call must be back at zero
    assert sgref.nmse(run_attention(sm100, stream, q, k, v, False, 0, s), sgref.attention(q, k, v, False, 0, s)) <= TOL
    mask = np.zeros((1, nq, nk), np.float32)
    mask[0, :, nk // 3:] = -np.inf
    got = run_attention(sm100, stream, q, k, v, False, 0, s, mask=mask, mask_heads=1)
    assert sgref.nmse(got, sgref.attention(q, k[:, :nk // 3], v[:, :nk // 3], False, 0, s)) <= TOL


def test_attention_kvcache_entry(sm100, stream):
    """The KV-cache entry requests the older rows before its dependency wait.  Each round first stores the new
    token's K and V rows with SET_ROWS (the launch right before the attention, as in a decode step), then attends
    with fresh_keys = 1; the values must be those of the plain entry and of the oracle, round after round (a
    stale row would show as the previous round's values)."""
    hq, hkv, d, n_ctx = 32, 8, 128, 1152
    lib = sm100.lib()
    rng = np.random.default_rng(21)
    start = 1024
    k = np.zeros((hkv, n_ctx, d), np.float32)
    v = np.zeros((hkv, n_ctx, d), np.float32)
    k[:, :start] = rng.standard_normal((hkv, start, d))
    v[:, :start] = rng.standard_normal((hkv, start, d))
    kb, vb = U.to_device(sm100, stream, k), U.to_device(sm100, stream, v)
    ob = sm100.Buffer(hq * d * 4)
    scale = float(1.0 / np.sqrt(d))
    for t in range(6):
        pos = start + t
        q = rng.standard_normal((hq, 1, d)).astype(np.float32)
        k_new = (10.0 * rng.standard_normal((hkv, 1, d))).astype(np.float32)   # large: the new key dominates the softmax
        v_new = rng.standard_normal((hkv, 1, d)).astype(np.float32)
        k[:, pos], v[:, pos] = k_new[:, 0], v_new[:, 0]
        qb, knb, vnb = (U.to_device(sm100, stream, a) for a in (q, k_new, v_new))
        pb = U.to_device(sm100, stream, np.array([pos], np.int32))
        stream.sync()
        sm100.check(lib.sm100_set_rows(stream.handle, knb.at(), pb.at(), kb.at(), d, 1, hkv, n_ctx), "set_rows k")
        sm100.check(lib.sm100_set_rows(stream.handle, vnb.at(), pb.at(), vb.at(), d, 1, hkv, n_ctx), "set_rows v")
        sm100.check(lib.sm100_attention_kvcache(stream.handle, qb.at(), kb.at(), vb.at(), None, 1, ob.at(), d, d, 1, n_ctx, hq, hkv, 1, 0, pb.at(),
                                                scale, 1), "attention_kvcache")   # one fresh key: its V row comes from the launch right before
        stream.sync()
        got = ob.download(stream, np.float32, hq * d).reshape(hq, 1, d)
        want = sgref.attention(q, k, v, True, pos, scale)
        assert sgref.nmse(got, want) <= TOL, t
        plain = run_attention(sm100, stream, q, k, v, True, pos, scale)
        assert np.array_equal(got, plain), t
        for b in (qb, knb, vnb, pb):
            b.free()
    st = lib.sm100_attention_kvcache(stream.handle, ob.at(), kb.at(), vb.at(), None, 1, ob.at(), d, d, 1, n_ctx, hq, hkv, 1, 0, None, scale, -1)
    assert st == 2
    for b in (kb, vb, ob):
        b.free()


def test_allreduce_wait_is_bounded_and_reported(sm100, stream):
    """A rank whose peer never arrives: the kernel's wait for the peer's flag is bounded, the kernel returns, the give-up is
    reported through sm100_allreduce_fault and the device stays usable.  One GPU plays both ranks' memory (two areas on the
    same device); only rank 0 calls, so the flag of rank 1 is one that nothing sets.  The wait limit is shortened for the
    test (sm100_allreduce_set_wait_limit); the default is about a second."""
    L = sm100.lib()
    world, cap = 2, 1024
    nbytes = int(L.sm100_allreduce_area_bytes(world, cap))
    areas = [sm100.Buffer(nbytes) for _ in range(world)]
    for a in areas:
        a.fill(stream, 0)
    stream.sync()
    ptrs = (C.c_void_p * world)(*[a.ptr for a in areas])
    ctx = C.c_void_p()
    sm100.check(L.sm100_allreduce_create(0, world, cap, ptrs, C.byref(ctx)), "allreduce_create")
    sm100.check(L.sm100_allreduce_set_wait_limit(ctx, 2000), "set_wait_limit")
    x = np.arange(cap, dtype=np.float32)
    xb = U.to_device(sm100, stream, x)
    sm100.check(L.sm100_allreduce_sum(ctx, stream.handle, C.c_void_p(xb.ptr), cap), "allreduce_sum")
    stream.sync()                                   # returns: the wait ran out instead of spinning
    fault = C.c_int(0)
    sm100.check(L.sm100_allreduce_fault(ctx, C.byref(fault)), "allreduce_fault")
    assert fault.value != 0
    # the context is intact: an ordinary kernel runs and gives the right answer
    yb = sm100.Buffer(4 * cap)
    sm100.check(L.sm100_add(stream.handle, C.c_void_p(xb.ptr), C.c_void_p(xb.ptr), C.c_void_p(yb.ptr), cap), "add")
    stream.sync()
    assert np.array_equal(yb.download(stream, np.float32, cap), 2 * xb.download(stream, np.float32, cap))
    L.sm100_allreduce_destroy(ctx)
    for b in areas + [xb, yb]:
        b.free()
