"""The cuda_sm100 plugin driven through the reference's unchanged public C API, next to the reference's own CPU
backend on identical descriptors and bytes -- the structure of the reference's tests/ops/ops_tests.cpp (device
result vs scrapgpu_ref_execute), tests/attention/attention_tests.cpp and the vtable contract checks of
tests/cpu/cpu_tests.cpp.

Tolerances are the reference's: NMSE 1e-6 for quantized MUL_MAT (ops_tests.cpp:725), 1e-7 otherwise (:411-412),
exact for GET_ROWS / SET_ROWS / CPY (:588-603), 3e-4 absolute for attention (attention_tests.cpp:40)."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import refapi, sgref
from scrapgpulibrary_b200 import _build, abi

pytestmark = [pytest.mark.gpu]

QUANT = (abi.Q4_0, abi.Q8_0, abi.Q4_K, abi.Q6_K)


@pytest.fixture(scope="module")
def both():
    if not refapi.available() or not os.path.exists(_build.PLUGIN_SO):
        pytest.fail("oracle/_ref or the prebuilt plugin is missing on the GPU box: build them where the reference is checked out")
    from tests import refsession
    cpu, gpu = refsession.Session("cpu"), refsession.Session("cuda_sm100")
    yield cpu, gpu
    cpu.close()
    gpu.close()


def rnd(seed, *shape, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


def run_pair(both, op, make, params_factory=None, n_out=1):
    """make(sess) -> (inputs, outputs) as Tensor lists; returns the outputs' float arrays for cpu and gpu."""
    res = []
    for sess in both:
        ins, outs = make(sess)
        params = params_factory() if params_factory else None
        st, why = sess.supported(op, ins, outs, params)
        assert st == abi.OK, f"{sess.backend}: op {op} unsupported: {why}"
        sess.execute(op, ins, outs, params)
        sess.sync()
        res.append([o.read_raw(np.uint8, o.nbytes + o.desc.offset) for o in outs])
    return res[0], res[1]


def as_f32(raw):
    return raw.view(np.float32)


def test_device_info(both):
    cpu, gpu = both
    assert gpu.info.backend_name == b"cuda_sm100"
    assert gpu.info.tuning_profile_name == b"b200"
    assert gpu.info.compute_units >= 100 and gpu.info.warp_or_wave_width == 32
    assert b"B200" in gpu.info.name or gpu.info.total_memory_bytes > (100 << 30)


@pytest.mark.parametrize("dtype", QUANT, ids=lambda d: abi.DTYPE_NAMES[d])
@pytest.mark.parametrize("layout", [abi.LAYOUT_NATURAL, abi.LAYOUT_R32], ids=["natural", "packed"])
def test_mul_mat_quantized(both, dtype, layout):
    """Tile sweep in the spirit of ref_ops_tests.cpp:659-754: M in {1,3,4,5,9} batch columns, ragged row counts."""
    for k, n in ((256, 24), (512, 17), (4096, 33)):
        wq = sgref.quantize(dtype, rnd(k + n, n, k, scale=0.02))
        for m in (1, 3, 4, 5, 9):
            x = rnd(m, m, k)

            def make(sess):
                w = sess.tensor(dtype, [k, n], layout=layout if sess.backend != "cpu" else abi.LAYOUT_NATURAL).upload(wq)
                xt = sess.tensor(abi.F32, [k, m]).upload(x)
                y = sess.tensor(abi.F32, [n, m]).upload(np.full(n * m, -7.0, np.float32))
                return [w, xt], [y]

            p = lambda: abi.MulMatParams()
            c, g = run_pair(both, abi.OP_MUL_MAT, make, p)
            assert sgref.nmse(as_f32(g[0]), as_f32(c[0])) <= 1e-6, (k, n, m)


def test_mul_mat_float_weights_padded_strides(both):
    """F32 / F16 weights with padded row strides and a batch dim with broadcast (ref_ops_tests.cpp:604-623,739-747)."""
    k, n, m = 40, 9, 3
    w = rnd(1, 2, n, k + 8)        # two slices, rows padded by 8 floats
    x = rnd(2, 4, m, k)            # four slices: broadcast 2 -> 4

    def make(sess):
        wt = sess.tensor(abi.F32, [k, n, 2], nb=[4, 4 * (k + 8), 4 * (k + 8) * n, 4 * (k + 8) * n * 2], pad=32).write_raw(w)
        xt = sess.tensor(abi.F32, [k, m, 4]).upload(x)
        y = sess.tensor(abi.F32, [n, m, 4]).upload(np.zeros(n * m * 4, np.float32))
        return [wt, xt], [y]

    def p():
        q = abi.MulMatParams()
        q.allow_broadcast = 1
        return q

    c, g = run_pair(both, abi.OP_MUL_MAT, make, p)
    assert sgref.nmse(as_f32(g[0]), as_f32(c[0])) <= 1e-7
    # the same shapes without permission to broadcast are refused by both
    for sess in both:
        ins, outs = make(sess)
        st, why = sess.supported(abi.OP_MUL_MAT, ins, outs, abi.MulMatParams())
        assert st == abi.UNSUPPORTED and why


def test_mul_mat_multi_matches_single_mul_mats(both):
    """MUL_MAT_MULTI against plain MUL_MATs on the CPU backend (ops_tests.cpp:751-778)."""
    cpu, gpu = both
    k = 1024
    ns = (96, 32, 32)
    x = rnd(5, 1, k)
    ws = [sgref.quantize(abi.Q4_K, rnd(10 + i, n, k, scale=0.02)) for i, n in enumerate(ns)]
    want = []
    for wq, n in zip(ws, ns):
        w = cpu.tensor(abi.Q4_K, [k, n]).upload(wq)
        xt = cpu.tensor(abi.F32, [k, 1]).upload(x)
        y = cpu.tensor(abi.F32, [n, 1])
        cpu.execute(abi.OP_MUL_MAT, [w, xt], [y], abi.MulMatParams())
        want.append(y.download(np.float32, n))
    wt = [gpu.tensor(abi.Q4_K, [k, n], layout=abi.LAYOUT_R32).upload(wq) for wq, n in zip(ws, ns)]
    xt = gpu.tensor(abi.F32, [k, 1]).upload(x)
    ys = [gpu.tensor(abi.F32, [n, 1]) for n in ns]
    st, why = gpu.supported(abi.OP_MUL_MAT_MULTI, wt + [xt], ys)
    assert st == abi.OK, why
    gpu.execute(abi.OP_MUL_MAT_MULTI, wt + [xt], ys)
    gpu.sync()
    for y, n, w_ in zip(ys, ns, want):
        assert sgref.nmse(y.download(np.float32, n), w_) <= 1e-6


def test_packed_upload_download_round_trip(both):
    """Host bytes stay natural: a packed tensor downloads as the bytes that were uploaded, also for a block-aligned
    prefix (the chunked-transfer rule of the R32 path)."""
    cpu, gpu = both
    for dtype in QUANT:
        k, n = 512, 24
        wq = sgref.quantize(dtype, rnd(dtype, n, k, scale=0.02))
        t = gpu.tensor(dtype, [k, n], layout=abi.LAYOUT_R32).upload(wq)
        assert np.array_equal(t.download(np.uint8, wq.size), wq.ravel())
        raw = t.read_raw(np.uint8, wq.size)
        assert not np.array_equal(raw, wq.ravel())          # the device image is the plane layout ...
        assert np.array_equal(np.sort(raw) if dtype != abi.Q4_K else raw.size, np.sort(wq.ravel()) if dtype != abi.Q4_K else wq.size)  # ... of the same bytes
        bb = abi.BLOCK[dtype][1]
        part = np.empty(5 * bb, np.uint8)
        refapi.check(refapi.lib().scrapgpu_tensor_download(gpu.stream, C.byref(t.desc), part.ctypes.data_as(C.c_void_p), part.nbytes), "partial download")
        assert np.array_equal(part, wq.ravel()[:5 * bb])
        st = refapi.lib().scrapgpu_tensor_download(gpu.stream, C.byref(t.desc), part.ctypes.data_as(C.c_void_p), bb + 1)
        assert st == abi.UNSUPPORTED


def test_norms_rope_softmax_glu_add(both):
    rows, ne0 = 6, 256
    a, b, w = rnd(1, rows, ne0, scale=3), rnd(2, rows, ne0), rnd(3, ne0)

    def eps():
        p = abi.RmsNormParams()
        p.eps = 1e-6
        return p

    def mk_norm(sess):
        return [sess.tensor(abi.F32, [ne0, rows]).upload(a)], [sess.tensor(abi.F32, [ne0, rows])]

    c, g = run_pair(both, abi.OP_RMS_NORM, mk_norm, eps)
    assert sgref.nmse(as_f32(g[0]), as_f32(c[0])) <= 1e-7

    def mk_norm_mul(sess):
        return [sess.tensor(abi.F32, [ne0, rows]).upload(a), sess.tensor(abi.F32, [ne0]).upload(w)], [sess.tensor(abi.F32, [ne0, rows])]

    c, g = run_pair(both, abi.OP_RMS_NORM_MUL, mk_norm_mul, eps)
    assert sgref.nmse(as_f32(g[0]), as_f32(c[0])) <= 1e-7

    def mk_add_norm(sess):
        return ([sess.tensor(abi.F32, [ne0, rows]).upload(a), sess.tensor(abi.F32, [ne0, rows]).upload(b), sess.tensor(abi.F32, [ne0]).upload(w)],
                [sess.tensor(abi.F32, [ne0, rows]), sess.tensor(abi.F32, [ne0, rows])])

    c, g = run_pair(both, abi.OP_ADD_RMS_NORM_MUL, mk_add_norm, eps)
    assert np.array_equal(g[0], c[0])
    assert sgref.nmse(as_f32(g[1]), as_f32(c[1])) <= 1e-7

    # ROPE: [128, 8 heads, 3 tokens], NEOX base 1e6 (table path) and NORMAL with frequency factors (direct path)
    x = rnd(4, 3, 8, 128)
    pos = np.array([0, 1024, 1151], np.int32)
    ff = (1.0 + 0.1 * np.arange(64)).astype(np.float32)
    for mode, with_ff in ((abi.ROPE_NEOX, False), (abi.ROPE_NORMAL, True), (abi.ROPE_NEOX, True)):
        def mk_rope(sess):
            ins = [sess.tensor(abi.F32, [128, 8, 3]).upload(x), sess.tensor(abi.I32, [3]).upload(pos)]
            if with_ff:
                ins.append(sess.tensor(abi.F32, [64]).upload(ff))
            return ins, [sess.tensor(abi.F32, [128, 8, 3])]

        def rp():
            p = abi.RopeParams()
            p.mode, p.n_dims, p.n_ctx_orig, p.freq_base, p.freq_scale, p.ext_factor, p.attn_factor = mode, 128, 4096, 1e6, 1.0, 0.0, 1.0
            p.beta_fast, p.beta_slow = 32.0, 1.0
            return p

        c, g = run_pair(both, abi.OP_ROPE, mk_rope, rp)
        if with_ff:
            assert sgref.nmse(as_f32(g[0]), as_f32(c[0])) <= 1e-7
        else:
            assert np.array_equal(g[0], c[0])      # host-built table: the reference's own cos / sin

    # SOFT_MAX with an F32 mask holding -inf, in place (required by the core's attention, attention.cpp:656)
    sx = rnd(5, 4, 77, scale=4)
    mk_ = np.zeros((4, 77), np.float32)
    mk_[:, 60:] = -np.inf

    def mk_sm(sess):
        t = sess.tensor(abi.F32, [77, 4]).upload(sx)
        return [t, sess.tensor(abi.F32, [77, 4]).upload(mk_)], [t]

    def sp():
        p = abi.SoftMaxParams()
        p.scale = 0.125
        return p

    c, g = run_pair(both, abi.OP_SOFT_MAX, mk_sm, sp)
    assert sgref.nmse(as_f32(g[0]), as_f32(c[0])) <= 1e-7

    # SwiGLU split and fused-halves-swapped, ReGLU
    gx, gg = rnd(6, 5, 96, scale=3), rnd(7, 5, 96)
    for kind in (abi.GLU_SWIGLU, abi.GLU_REGLU):
        def gp(split=1, swapped=0):
            p = abi.GluParams()
            p.kind, p.split_inputs, p.swapped = kind, split, swapped
            return p

        c, g = run_pair(both, abi.OP_GLU, lambda s: ([s.tensor(abi.F32, [96, 5]).upload(gx), s.tensor(abi.F32, [96, 5]).upload(gg)], [s.tensor(abi.F32, [96, 5])]), gp)
        assert sgref.nmse(as_f32(g[0]), as_f32(c[0])) <= 1e-7
        fused = np.concatenate([gg, gx], axis=1)
        c, g = run_pair(both, abi.OP_GLU, lambda s: ([s.tensor(abi.F32, [192, 5]).upload(fused)], [s.tensor(abi.F32, [96, 5])]), lambda: gp(0, 1))
        assert sgref.nmse(as_f32(g[0]), as_f32(c[0])) <= 1e-7

    # ADD exact, with a row-broadcast second operand and in place
    def mk_add(sess):
        t = sess.tensor(abi.F32, [ne0, rows]).upload(a)
        return [t, sess.tensor(abi.F32, [ne0]).upload(w)], [t]

    c, g = run_pair(both, abi.OP_ADD, mk_add)
    assert np.array_equal(g[0], c[0])


def test_rows_cpy_topk_exact(both):
    k, n = 512, 40
    for dtype in QUANT + (abi.F32, abi.F16):
        w = rnd(dtype, n, k, scale=0.02)
        table = sgref.quantize(dtype, w) if dtype in QUANT else (w if dtype == abi.F32 else w.astype(np.float16))
        ids = np.array([39, 0, 7, 7, 21], np.int32)
        layouts = (abi.LAYOUT_NATURAL, abi.LAYOUT_R32) if dtype in QUANT else (abi.LAYOUT_NATURAL,)
        for layout in layouts:
            def mk(sess):
                t = sess.tensor(dtype, [k, n], layout=layout if sess.backend != "cpu" else abi.LAYOUT_NATURAL).upload(table)
                return [t, sess.tensor(abi.I32, [5]).upload(ids)], [sess.tensor(abi.F32, [k, 5])]

            c, g = run_pair(both, abi.OP_GET_ROWS, mk, lambda: abi.GetRowsParams())
            assert np.array_equal(g[0], c[0]), (dtype, layout)

    # SET_ROWS: K/V rows of 8 heads into a cache at a position; F32 -> F32 and F32 -> F16
    src = rnd(3, 8, 2, 128)
    ids = np.array([5, 2], np.int32)
    for ddt in (abi.F32, abi.F16):
        def mk(sess):
            cache = sess.tensor(ddt, [128, 16, 8])
            refapi.check(refapi.lib().scrapgpu_buffer_fill(sess.stream, cache.buf, 0, cache.nbytes, 0, 1), "fill")
            return [sess.tensor(abi.F32, [128, 2, 8]).upload(src), sess.tensor(abi.I32, [2]).upload(ids)], [cache]

        c, g = run_pair(both, abi.OP_SET_ROWS, mk, lambda: abi.SetRowsParams())
        assert np.array_equal(g[0], c[0])

    # CPY of a transposed view (the V^T copy of the core's attention, attention.cpp:322-340) and F32 -> F16
    v = rnd(4, 24, 96)

    def mk_t(sess):
        s = sess.tensor(abi.F32, [24, 96], nb=[4 * 96, 4, 4 * 96 * 24, 4 * 96 * 24]).write_raw(v)   # logical [24, 96] over rows of 96
        return [s], [sess.tensor(abi.F32, [24, 96])]

    def cp():
        p = abi.CpyParams()
        p.allow_transpose = 1
        return p

    c, g = run_pair(both, abi.OP_CPY, mk_t, cp)
    assert np.array_equal(g[0], c[0])
    assert np.array_equal(as_f32(g[0]).reshape(96, 24), v.T)
    c, g = run_pair(both, abi.OP_CPY, lambda s: ([s.tensor(abi.F32, [96, 24]).upload(v)], [s.tensor(abi.F16, [96, 24])]), lambda: abi.CpyParams())
    assert np.array_equal(g[0], c[0])

    # TOP_K k = 1: ties resolve to the lowest index
    logits = rnd(9, 3, 1000)
    logits[1, 10] = logits[1, 900] = 99.0

    def tk():
        p = abi.ArgsortParams()
        p.order, p.top_k = 1, 1
        return p

    c, g = run_pair(both, abi.OP_TOP_K, lambda s: ([s.tensor(abi.F32, [1000, 3]).upload(logits)], [s.tensor(abi.I32, [1, 3])]), tk)
    assert np.array_equal(g[0], c[0]) and g[0].view(np.int32)[1] == 10
    for sess in both:   # k > 1 is honest about being unsupported on the device
        st, why = sess.supported(abi.OP_TOP_K, [sess.tensor(abi.F32, [1000, 3])], [sess.tensor(abi.I32, [4, 3])], tk())
        if sess.backend == "cuda_sm100":
            assert st in (abi.UNSUPPORTED, abi.INVALID_ARGUMENT) and why


def test_buffers_bounds_and_plans(both):
    cpu, gpu = both
    L = refapi.lib()
    t = gpu.tensor(abi.F32, [64])
    data = np.arange(64, dtype=np.float32)
    t.upload(data)
    # bounds (cpu_tests.cpp: read/write/copy/fill outside the buffer are INVALID_ARGUMENT)
    assert L.scrapgpu_buffer_write(gpu.stream, t.buf, 250, data.ctypes.data_as(C.c_void_p), 16, 1) == abi.INVALID_ARGUMENT
    assert L.scrapgpu_buffer_read(gpu.stream, t.buf, 0, data.ctypes.data_as(C.c_void_p), 257, 1) == abi.INVALID_ARGUMENT
    assert L.scrapgpu_buffer_fill(gpu.stream, t.buf, 256, 1, 0, 1) == abi.INVALID_ARGUMENT
    # overlapping copy inside one buffer behaves like memmove (ops_tests.cpp:1039-1055)
    assert L.scrapgpu_buffer_copy(gpu.stream, t.buf, 16, t.buf, 0, 128, 1) == abi.OK
    got = t.read_raw(np.float32, 64)
    want = data.copy()
    want[4:36] = data[0:32]
    assert np.array_equal(got, want)
    assert L.scrapgpu_buffer_fill(gpu.stream, t.buf, 0, 8, 0xFF, 1) == abi.OK
    assert np.all(t.read_raw(np.uint8, 8) == 0xFF)
    # a tensor that exceeds its buffer is refused at execute time
    big = abi.tensor_desc(abi.F32, [128], buffer=t.buf.value)
    o = abi.Op(abi.OP_ADD, [big, big], [big])
    assert L.scrapgpu_op_execute(gpu.stream, o.ptr()) == abi.INVALID_ARGUMENT
    # plans: deep copy of descriptors, buffers pinned while the plan lives (ops_tests.cpp:1059-1113)
    a = gpu.tensor(abi.F32, [32]).upload(np.ones(32, np.float32))
    b = gpu.tensor(abi.F32, [32]).upload(np.full(32, 2.0, np.float32))
    y = gpu.tensor(abi.F32, [32])
    op = abi.Op(abi.OP_ADD, [a.desc, b.desc], [y.desc])
    node = abi.PlanNode()
    node.struct_size = C.sizeof(node)
    node.op = op.desc
    pd = abi.PlanDesc()
    pd.struct_size, pd.nodes, pd.node_count = C.sizeof(pd), C.pointer(node), 1
    plan = C.c_void_p()
    refapi.check(L.scrapgpu_plan_build(gpu.device, C.byref(pd), C.byref(plan)), "plan_build")
    op.inputs[0].ne[0] = 999     # scribbling on the caller's descriptors must not reach the plan
    assert L.scrapgpu_buffer_free(y.buf) == abi.INVALID_ARGUMENT
    refapi.check(L.scrapgpu_plan_execute(gpu.stream, plan), "plan_execute")
    gpu.sync()
    assert np.all(y.download(np.float32, 32) == 3.0)
    refapi.check(L.scrapgpu_plan_free(plan), "plan_free")
    # an unsupported node fails the build with a reason
    bad = abi.Op(abi.OP_ARGSORT, [a.desc], [gpu.tensor(abi.I32, [32]).desc], abi.ArgsortParams())
    node.op = bad.desc
    assert L.scrapgpu_plan_build(gpu.device, C.byref(pd), C.byref(plan)) == abi.UNSUPPORTED
    assert "plan node 0" in refapi.last_error()


def test_tensor_copy_between_backends(both):
    """scrapgpu_tensor_copy (core/transport.cpp): same device, and cpu <-> cuda_sm100 through the core's host staging;
    packed tensors are refused by the core (ops_tests.cpp:1118-1219)."""
    cpu, gpu = both
    L = refapi.lib()
    x = rnd(1, 300)
    src = gpu.tensor(abi.F32, [300]).upload(x)
    dst = gpu.tensor(abi.F32, [300])
    refapi.check(L.scrapgpu_tensor_copy(gpu.stream, C.byref(src.desc), gpu.stream, C.byref(dst.desc)), "copy same device")
    gpu.sync()
    assert np.array_equal(dst.download(np.float32, 300), x)
    on_cpu = cpu.tensor(abi.F32, [300])
    refapi.check(L.scrapgpu_tensor_copy(gpu.stream, C.byref(src.desc), cpu.stream, C.byref(on_cpu.desc)), "copy gpu -> cpu")
    assert np.array_equal(on_cpu.download(np.float32, 300), x)
    back = gpu.tensor(abi.F32, [300])
    refapi.check(L.scrapgpu_tensor_copy(cpu.stream, C.byref(on_cpu.desc), gpu.stream, C.byref(back.desc)), "copy cpu -> gpu")
    gpu.sync()
    assert np.array_equal(back.download(np.float32, 300), x)
    wq = sgref.quantize(abi.Q4_0, rnd(2, 8, 64, scale=0.02))
    qa = gpu.tensor(abi.Q4_0, [64, 8]).upload(wq)
    qb = gpu.tensor(abi.Q4_0, [64, 8])
    refapi.check(L.scrapgpu_tensor_copy(gpu.stream, C.byref(qa.desc), gpu.stream, C.byref(qb.desc)), "copy natural q4_0")
    gpu.sync()
    assert np.array_equal(qb.download(np.uint8, wq.size), wq.ravel())
    pa = gpu.tensor(abi.Q4_0, [64, 8], layout=abi.LAYOUT_R32).upload(wq)
    pb = gpu.tensor(abi.Q4_0, [64, 8], layout=abi.LAYOUT_R32)
    assert L.scrapgpu_tensor_copy(gpu.stream, C.byref(pa.desc), gpu.stream, C.byref(pb.desc)) == abi.UNSUPPORTED


def attention_case(sess, q, k, v, causal, offset, scale, fused, position=None):
    from tests import refsession
    L = refapi.lib()
    hq, nq, d = q.shape
    hkv, nk, _ = k.shape
    dv = v.shape[2]
    tq = sess.tensor(abi.F32, [d, nq, hq, 1]).upload(q)
    tk = sess.tensor(abi.F32, [d, nk, hkv, 1]).upload(k)
    tv = sess.tensor(abi.F32, [dv, nk, hkv, 1]).upload(v)
    to = sess.tensor(abi.F32, [dv, nq, hq, 1])
    p = abi.AttentionParams()
    p.struct_size = C.sizeof(p)
    p.query, p.key, p.value, p.output = C.pointer(tq.desc), C.pointer(tk.desc), C.pointer(tv.desc), C.pointer(to.desc)
    p.query_position_offset, p.max_workspace_bytes, p.causal, p.scale = offset, 64 << 20, int(causal), scale
    if fused:
        if position is not None:
            tp = sess.tensor(abi.I32, [1]).upload(np.array([position], np.int32))
            refapi.check(refsession.plugin().scrapgpu_cuda_sm100_attention_at(sess.device, sess.stream, C.byref(p), C.byref(tp.desc)), "fused attention at")
        else:
            refapi.check(refsession.plugin().scrapgpu_cuda_sm100_attention(sess.device, sess.stream, C.byref(p)), "fused attention")
    else:
        refapi.check(L.scrapgpu_scaled_dot_product_attention(sess.device, sess.stream, C.byref(p)), "core attention")
    sess.sync()
    return to.download(np.float32, hq * nq * dv).reshape(hq, nq, dv)


def test_attention_core_composition_and_fused(both):
    """The core's own SDPA composition (CPY + MUL_MAT + SOFT_MAX) runs on cuda_sm100 unchanged, and the fused entry
    gives the same values; both against the composition on the reference's CPU backend."""
    cpu, gpu = both
    rng = np.random.default_rng(3)
    for (hq, hkv, d, nk, nq, causal, off) in ((4, 2, 32, 40, 3, True, 2), (8, 2, 64, 130, 1, True, 100), (4, 4, 32, 50, 2, False, 0)):
        q = rng.standard_normal((hq, nq, d)).astype(np.float32)
        k = rng.standard_normal((hkv, nk, d)).astype(np.float32)
        v = rng.standard_normal((hkv, nk, d)).astype(np.float32)
        scale = float(1.0 / np.sqrt(d))
        want = attention_case(cpu, q, k, v, causal, off, scale, fused=False)
        core_on_gpu = attention_case(gpu, q, k, v, causal, off, scale, fused=False)
        fused = attention_case(gpu, q, k, v, causal, off, scale, fused=True)
        assert np.max(np.abs(core_on_gpu - want)) <= 3e-4 and sgref.nmse(core_on_gpu, want) <= 1e-6
        assert np.max(np.abs(fused - want)) <= 3e-4 and sgref.nmse(fused, want) <= 1e-6
        if causal:
            at = attention_case(gpu, q, k, v, causal, 0, scale, fused=True, position=off)
            assert np.array_equal(at, fused)


def test_decode_attention_qwen_shape(both):
    cpu, gpu = both
    rng = np.random.default_rng(4)
    hq, hkv, d, n_ctx = 32, 8, 128, 1152
    t = 70
    k = np.zeros((hkv, n_ctx, d), np.float32)
    v = np.zeros((hkv, n_ctx, d), np.float32)
    k[:, :1024 + t + 1] = rng.standard_normal((hkv, 1024 + t + 1, d))
    v[:, :1024 + t + 1] = rng.standard_normal((hkv, 1024 + t + 1, d))
    q = rng.standard_normal((hq, 1, d)).astype(np.float32)
    scale = float(1.0 / np.sqrt(d))
    want = attention_case(cpu, q, k, v, True, 1024 + t, scale, fused=False)
    fused = attention_case(gpu, q, k, v, True, 1024 + t, scale, fused=True)
    assert np.max(np.abs(fused - want)) <= 3e-4 and sgref.nmse(fused, want) <= 1e-6


def test_unmodified_reference_example_runs_on_cuda_sm100():
    """examples/standalone_matmul.c of the reference, compiled byte-for-byte unchanged (oracle/Makefile `example`) and
    linked against the plugin through a one-function registration shim: Q4_0 weights uploaded with the packed-layout
    tag, MUL_MAT on the device, NMSE against scrapgpu_ref_execute printed by the program itself."""
    import re
    import subprocess
    if not os.path.exists(refapi.EXAMPLE):
        pytest.fail("oracle/_ref/standalone_matmul is missing on the GPU box: run `make -C oracle example` where the reference is checked out")
    r = subprocess.run([refapi.EXAMPLE], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "(b200)" in r.stdout, r.stdout
    m = re.search(r"NMSE ([0-9.e+-]+)", r.stdout)
    assert m and float(m.group(1)) <= 1e-6, r.stdout


def test_set_rows_pair_matches_two_set_rows(both):
    """SET_ROWS_PAIR (K and V rows of one token into their caches in one op) against two plain SET_ROWS on the CPU
    backend, which does not implement the fused op (src/core/ref/ops.cpp:1428-1429; ops_tests.cpp:765-776 compares
    the same way)."""
    cpu, gpu = both
    ks, vs = rnd(31, 8, 1, 128), rnd(32, 8, 1, 128)
    ids = np.array([9], np.int32)
    want = []
    for src in (ks, vs):
        cache = cpu.tensor(abi.F32, [128, 16, 8])
        refapi.check(refapi.lib().scrapgpu_buffer_fill(cpu.stream, cache.buf, 0, cache.nbytes, 0, 1), "fill")
        cpu.execute(abi.OP_SET_ROWS, [cpu.tensor(abi.F32, [128, 1, 8]).upload(src), cpu.tensor(abi.I32, [1]).upload(ids)], [cache], abi.SetRowsParams())
        want.append(cache.download(np.float32, 128 * 16 * 8))
    caches = [gpu.tensor(abi.F32, [128, 16, 8]) for _ in range(2)]
    for c in caches:
        refapi.check(refapi.lib().scrapgpu_buffer_fill(gpu.stream, c.buf, 0, c.nbytes, 0, 1), "fill")
    ins = [gpu.tensor(abi.F32, [128, 1, 8]).upload(ks), gpu.tensor(abi.I32, [1]).upload(ids),
           gpu.tensor(abi.F32, [128, 1, 8]).upload(vs), gpu.tensor(abi.I32, [1]).upload(ids)]
    st, why = gpu.supported(abi.OP_SET_ROWS_PAIR, ins, caches)
    assert st == abi.OK, why
    gpu.execute(abi.OP_SET_ROWS_PAIR, ins, caches)
    gpu.sync()
    for c, w_ in zip(caches, want):
        assert np.array_equal(c.download(np.float32, 128 * 16 * 8), w_)
    # mixed destination dtypes are refused with a reason
    bad = [gpu.tensor(abi.F32, [128, 16, 8]), gpu.tensor(abi.F16, [128, 16, 8])]
    st, why = gpu.supported(abi.OP_SET_ROWS_PAIR, ins, bad)
    assert st in (abi.UNSUPPORTED, abi.INVALID_ARGUMENT) and why


@pytest.mark.parametrize("between", [0, 1, 3])
def test_mul_mat_over_a_left_operand_written_just_before(both, between):
    """MUL_MAT whose src0 was produced by a kernel enqueued right before it, with no synchronisation in between (the K
    cache of the core's attention composition, src/core/attention.cpp:487-560: CPY then MUL_MAT).  The matvec kernels ask
    for their weights before they wait for earlier kernels, so the backend has to notice that this operand is not an
    upload that sits in memory and serialize the launch; `between` small kernels separate the producer and the matvec.
    The producer is long (a 128 MB copy) and the destination starts as zeros, so a premature read shows."""
    _, gpu = both
    k, n = 4096, 8192
    a = rnd(31, n, k)
    x = rnd(32, k)
    src = gpu.tensor(abi.F32, [k, n]).upload(a)
    dst = gpu.tensor(abi.F32, [k, n]).upload(np.zeros(n * k, np.float32))
    xt = gpu.tensor(abi.F32, [k]).upload(x)
    tmp = gpu.tensor(abi.F32, [k]).upload(np.zeros(k, np.float32))
    want, got = (gpu.tensor(abi.F32, [n]).upload(np.zeros(n, np.float32)) for _ in range(2))
    gpu.execute(abi.OP_MUL_MAT, [src, xt], [want], abi.MulMatParams())
    gpu.sync()
    for trial in range(3):
        dst.upload(np.zeros(n * k, np.float32))
        gpu.sync()
        gpu.execute(abi.OP_CPY, [src], [dst], abi.CpyParams())
        for _ in range(between):
            gpu.execute(abi.OP_ADD, [xt, xt], [tmp])
        gpu.execute(abi.OP_MUL_MAT, [dst, xt], [got], abi.MulMatParams())
        gpu.sync()
        assert np.array_equal(got.download(np.float32, n), want.download(np.float32, n)), f"trial {trial}"
    for t in (src, dst, xt, tmp, want, got):
        t.free()


def test_profile_table():
    """SCRAPGPU_SM100_PROFILE=1: per-op-key event timings like the OpenCL backend's GGML_CL11_PROFILE table
    (src/backends/opencl11/executor.h:41-112): keys carry op, weight type and mv/mm form, MUL_MAT rows report the
    weight bandwidth, the table is also printed when the stream is freed."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, SCRAPGPU_SM100_PROFILE="1", PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-m", "tests.profile_worker"], cwd=root, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = r.stdout.splitlines()
    assert lines[0].startswith("cuda_sm100 profile of ") and "total kernel time" in lines[0]
    mm = [l for l in lines if "MUL_MAT q4_K packed mv n=1" in l]
    assert len(mm) == 1 and "     3 calls" in mm[0] and "weights" in mm[0] and "GB/s" in mm[0], r.stdout
    add = [l for l in lines if l.strip().startswith("ADD")]
    assert len(add) == 1 and "     1 calls" in add[0]
    assert "RESULT_SUM True" in r.stdout
    assert "cuda_sm100 profile of " in r.stderr          # printed at stream_free
