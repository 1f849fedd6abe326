"""Multi-GPU transport of the plugin on real devices: GPU-to-GPU scrapgpu_cuda_sm100_tensor_copy with the ordering
guarantee of include/scrapgpu/tensor.h:55-67, shard upload from a full host image, and the device group's all-reduce
driven from ONE process (the way a C caller of the library would run a tensor-parallel model).  The two-device cases
are skipped on a single-GPU box; the same entry points are exercised there on one device."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import refapi, sgref
from scrapgpulibrary_b200 import _build, abi
from tests import util as U

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    if not refapi.available() or not os.path.exists(_build.PLUGIN_SO):
        pytest.fail("oracle/_ref or the prebuilt plugin is missing on the GPU box")
    from tests import refsession
    refsession.register_all()
    P = refsession.plugin()
    vp = C.c_void_p
    P.scrapgpu_cuda_sm100_tensor_copy.argtypes = [vp, C.POINTER(abi.TensorDesc), vp, C.POINTER(abi.TensorDesc)]
    P.scrapgpu_cuda_sm100_shard.argtypes = [C.POINTER(abi.TensorDesc), C.c_int, C.c_size_t, C.c_size_t, C.POINTER(abi.TensorDesc)]
    P.scrapgpu_cuda_sm100_upload_view.argtypes = [vp, C.POINTER(abi.TensorDesc), vp, C.POINTER(abi.TensorDesc)]
    P.scrapgpu_cuda_sm100_group_create.argtypes = [C.POINTER(vp), C.c_size_t, C.c_size_t, C.POINTER(vp)]
    P.scrapgpu_cuda_sm100_group_all_reduce.argtypes = [vp, C.POINTER(vp), C.POINTER(abi.TensorDesc)]
    P.scrapgpu_cuda_sm100_group_status.argtypes = [vp]
    P.scrapgpu_cuda_sm100_group_free.argtypes = [vp]
    sessions = []
    i = 0
    while True:
        dev, _ = refsession.find_device("cuda_sm100", i)
        if dev is None or i >= 2:
            break
        sessions.append(refsession.Session("cuda_sm100", i))
        i += 1
    assert sessions, "no cuda_sm100 device"
    yield P, sessions
    for s in sessions:
        s.close()


def test_tensor_copy_follows_enqueued_work(env):
    """The copy is ordered after the ADD already enqueued on the source stream and before the ADD enqueued afterwards
    on the destination stream (tests/ops/ops_tests.cpp:1118-1156 checks the same on one device; :1177-1214 across two)."""
    P, sessions = env
    src_s, dst_s = sessions[0], sessions[-1]      # two devices when the box has them, else twice the same one
    n = 4096
    a, b = np.arange(n, dtype=np.float32), np.full(n, 0.5, np.float32)
    ta, tb, tsum = src_s.tensor(abi.F32, [n]).upload(a), src_s.tensor(abi.F32, [n]).upload(b), src_s.tensor(abi.F32, [n])
    src_s.execute(abi.OP_ADD, [ta, tb], [tsum])                                   # enqueued, not synchronised
    other = sessions[-1]
    from tests import refsession
    dst_stream = C.c_void_p()
    refapi.check(refapi.lib().scrapgpu_stream_create(dst_s.device, C.byref(dst_stream)), "stream_create")   # a second stream even on one device
    tdst, tone, tout = dst_s.tensor(abi.F32, [n]), dst_s.tensor(abi.F32, [n]).upload(np.ones(n, np.float32)), dst_s.tensor(abi.F32, [n])
    assert P.scrapgpu_cuda_sm100_tensor_copy(src_s.stream, C.byref(tsum.desc), dst_stream, C.byref(tdst.desc)) == abi.OK
    o = abi.Op(abi.OP_ADD, [tdst.desc, tone.desc], [tout.desc])
    refapi.check(refapi.lib().scrapgpu_op_execute(dst_stream, o.ptr()), "op_execute")
    refapi.check(refapi.lib().scrapgpu_stream_sync(dst_stream), "stream_sync")
    out = np.empty(n, np.float32)
    refapi.check(refapi.lib().scrapgpu_buffer_read(dst_stream, tout.buf, 0, out.ctypes.data_as(C.c_void_p), out.nbytes, 1), "buffer_read")
    assert np.array_equal(out, a + 0.5 + 1.0)
    # quantized natural bytes travel unchanged; packed tensors are refused like the core refuses R32 (transport.cpp:83-86)
    wq = U.quantize(U.Q4_0, U.seeded_weights(3, 8, 64))
    tq, tq2 = src_s.tensor(abi.Q4_0, [64, 8]).upload(wq), dst_s.tensor(abi.Q4_0, [64, 8])
    assert P.scrapgpu_cuda_sm100_tensor_copy(src_s.stream, C.byref(tq.desc), dst_stream, C.byref(tq2.desc)) == abi.OK
    refapi.check(refapi.lib().scrapgpu_stream_sync(dst_stream), "stream_sync")
    back = np.empty(wq.size, np.uint8)
    refapi.check(refapi.lib().scrapgpu_buffer_read(dst_stream, tq2.buf, 0, back.ctypes.data_as(C.c_void_p), back.nbytes, 1), "buffer_read")
    assert np.array_equal(back, wq.ravel())
    tp_ = src_s.tensor(abi.Q4_0, [64, 32], layout=abi.LAYOUT_R32)
    tp2 = dst_s.tensor(abi.Q4_0, [64, 32], layout=abi.LAYOUT_R32)
    assert P.scrapgpu_cuda_sm100_tensor_copy(src_s.stream, C.byref(tp_.desc), dst_stream, C.byref(tp2.desc)) == abi.UNSUPPORTED
    refapi.lib().scrapgpu_stream_free(dst_stream)


def test_sharded_mul_mat_with_group_all_reduce(env):
    """A row-parallel projection the way a C caller would shard it: K-slices of a packed Q4_K weight uploaded from the
    full host image (scrapgpu_cuda_sm100_shard + upload_view), one MUL_MAT per device on its slice of the activations,
    scrapgpu_cuda_sm100_group_all_reduce of the partial outputs: every device then holds the full product, the same
    bits everywhere, within NMSE 1e-6 of the oracle."""
    P, sessions = env
    world = len(sessions)
    k, n = 2048, 272
    wq = U.quantize(U.Q4_K, U.seeded_weights(17, n, k))
    image = np.ascontiguousarray(wq).ravel()
    x = U.seeded_acts(18, 1, k)
    want = sgref.mul_mat(U.Q4_K, wq, k, x)[0]
    full = abi.tensor_desc(abi.Q4_K, [k, n])
    devs = (C.c_void_p * world)(*[s.device.value for s in sessions])
    group = C.c_void_p()
    assert P.scrapgpu_cuda_sm100_group_create(devs, world, 4096, C.byref(group)) == abi.OK, refapi.last_error()
    outs = []
    for r, s in enumerate(sessions):
        view = abi.TensorDesc()
        assert P.scrapgpu_cuda_sm100_shard(C.byref(full), 0, r, world, C.byref(view)) == abi.OK
        kl = k // world
        wt = s.tensor(abi.Q4_K, [kl, n], layout=abi.LAYOUT_R32)
        assert P.scrapgpu_cuda_sm100_upload_view(s.stream, C.byref(wt.desc), image.ctypes.data_as(C.c_void_p), C.byref(view)) == abi.OK, refapi.last_error()
        xt = s.tensor(abi.F32, [kl]).upload(x[0, r * kl:(r + 1) * kl])
        yt = s.tensor(abi.F32, [n])
        s.execute(abi.OP_MUL_MAT, [wt, xt], [yt], abi.MulMatParams(0, 0))
        outs.append(yt)
    streams = (C.c_void_p * world)(*[s.stream.value for s in sessions])
    descs = (abi.TensorDesc * world)(*[t.desc for t in outs])
    for rep in range(3):      # the receive areas alternate: several calls in a row
        if rep:
            for r, s in enumerate(sessions):
                kl = k // world
                s.execute(abi.OP_MUL_MAT, [s.tensors[-3], s.tensors[-2]], [outs[r]], abi.MulMatParams(0, 0))
        assert P.scrapgpu_cuda_sm100_group_all_reduce(group, streams, descs) == abi.OK, refapi.last_error()
        got = []
        for s, t in zip(sessions, outs):
            s.sync()
            got.append(t.download(np.float32, n))
        assert P.scrapgpu_cuda_sm100_group_status(group) == abi.OK
        for g in got:
            assert np.array_equal(g.view(np.uint32), got[0].view(np.uint32))
            assert sgref.nmse(g, want) <= 1e-6
    assert P.scrapgpu_cuda_sm100_group_free(group) == abi.OK
    assert P.scrapgpu_cuda_sm100_group_free(group) == abi.INVALID_ARGUMENT


@pytest.mark.parametrize("n", [256, 272])
def test_group_mul_mat_all_reduce(env, n):
    """scrapgpu_cuda_sm100_group_mul_mat_all_reduce: the K-sharded product and its all-reduce as one call.  N = 256 (whole
    16-row tiles of packed Q4_K) takes the launch with the exchange inside on every device, N = 272 with a Q6_K weight the
    separate launches; either way every device holds the full product, the same bits everywhere, NMSE 1e-6 of the oracle,
    over several calls in a row.  With one device the call is a plain MUL_MAT."""
    P, sessions = env
    world = len(sessions)
    dtype = abi.Q4_K if n == 256 else abi.Q6_K
    udt = U.Q4_K if n == 256 else U.Q6_K
    k = 2048
    wq = U.quantize(udt, U.seeded_weights(27 + n, n, k))
    image = np.ascontiguousarray(wq).ravel()
    x = U.seeded_acts(28, 1, k)
    want = sgref.mul_mat(udt, wq, k, x)[0]
    full = abi.tensor_desc(dtype, [k, n])
    devs = (C.c_void_p * world)(*[s.device.value for s in sessions])
    group = C.c_void_p()
    assert P.scrapgpu_cuda_sm100_group_create(devs, world, 4096, C.byref(group)) == abi.OK, refapi.last_error()
    P.scrapgpu_cuda_sm100_group_mul_mat_all_reduce.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    ws, xs, ys = [], [], []
    kl = k // world
    for r, s in enumerate(sessions):
        view = abi.TensorDesc()
        assert P.scrapgpu_cuda_sm100_shard(C.byref(full), 0, r, world, C.byref(view)) == abi.OK
        wt = s.tensor(dtype, [kl, n], layout=abi.LAYOUT_R32)
        assert P.scrapgpu_cuda_sm100_upload_view(s.stream, C.byref(wt.desc), image.ctypes.data_as(C.c_void_p), C.byref(view)) == abi.OK, refapi.last_error()
        ws.append(wt)
        xs.append(s.tensor(abi.F32, [kl]).upload(x[0, r * kl:(r + 1) * kl]))
        ys.append(s.tensor(abi.F32, [n]).upload(np.zeros(n, np.float32)))
        s.sync()
    streams = (C.c_void_p * world)(*[s.stream.value for s in sessions])
    wd = (abi.TensorDesc * world)(*[t.desc for t in ws])
    xd = (abi.TensorDesc * world)(*[t.desc for t in xs])
    yd = (abi.TensorDesc * world)(*[t.desc for t in ys])
    for rep in range(3):
        assert P.scrapgpu_cuda_sm100_group_mul_mat_all_reduce(group, streams, wd, xd, yd) == abi.OK, refapi.last_error()
    got = []
    for s, t in zip(sessions, ys):
        s.sync()
        got.append(t.download(np.float32, n))
    assert P.scrapgpu_cuda_sm100_group_status(group) == abi.OK
    for g in got:
        assert np.array_equal(g.view(np.uint32), got[0].view(np.uint32))
        assert sgref.nmse(g, want) <= 1e-6
    assert P.scrapgpu_cuda_sm100_group_free(group) == abi.OK
