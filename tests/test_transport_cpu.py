"""Tensor-parallel shard arithmetic of the plugin (scrapgpu_cuda_sm100_shard): descriptors only, no GPU.  The rules
are those of scrapgpulibrary_b200/tp.py: column-parallel weights are split by rows (ceil-sized shards, the last may
be short), row-parallel weights by K in whole quantization blocks, and the pieces put together again give the full
tensor.  Also: the multi-GPU entry points answer objects of other backends with INVALID_ARGUMENT without touching
them (tests/cpu/cpu_tests.cpp:279-338 states that rule for the vtable)."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import refapi
from scrapgpulibrary_b200 import _build, abi, tp

pytestmark = pytest.mark.skipif(not (refapi.available() and os.path.exists(_build.PLUGIN_SO)),
                                reason="needs oracle/_ref and the prebuilt plugin (built where the reference headers are present)")


@pytest.fixture(scope="module")
def plugin():
    from tests import refsession
    P = refsession.plugin()
    P.scrapgpu_cuda_sm100_shard.argtypes = [C.POINTER(abi.TensorDesc), C.c_int, C.c_size_t, C.c_size_t, C.POINTER(abi.TensorDesc)]
    return P


def view_bytes(image: np.ndarray, d: abi.TensorDesc) -> np.ndarray:
    """The rows a view descriptor selects from the flat host image of the full tensor."""
    be, bb = abi.BLOCK[d.dtype]
    row = d.ne[0] // be * bb
    return np.stack([image[d.offset + r * d.nb[1]: d.offset + r * d.nb[1] + row] for r in range(d.ne[1])]) if d.ne[1] > 0 else np.zeros((0, row), np.uint8)


@pytest.mark.parametrize("dtype", [abi.Q4_K, abi.Q6_K, abi.Q8_0, abi.F32])
@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_shards_tile_the_tensor(plugin, dtype, world):
    k, n = 1536, 37
    be, bb = abi.BLOCK[dtype]
    row = k // be * bb
    image = np.random.default_rng(dtype + world).integers(0, 256, n * row, dtype=np.uint8)
    full = abi.tensor_desc(dtype, [k, n])
    nat = image.reshape(n, row)
    # rows: ceil-sized shards in order
    got_rows = []
    for r in range(world):
        v = abi.TensorDesc()
        assert plugin.scrapgpu_cuda_sm100_shard(C.byref(full), 1, r, world, C.byref(v)) == abi.OK
        lo, cnt = tp.vocab_shard(n, r, world)
        assert v.ne[1] == cnt and v.ne[0] == k and v.nb[1] == full.nb[1]
        got_rows.append(view_bytes(image, v))
        assert np.array_equal(got_rows[-1], tp.shard_rows(nat, lo, cnt))
    assert np.array_equal(np.concatenate(got_rows), nat)
    # K: whole blocks, refused otherwise
    v = abi.TensorDesc()
    st = plugin.scrapgpu_cuda_sm100_shard(C.byref(full), 0, 0, world, C.byref(v))
    if k % world != 0 or (k // world) % be != 0:
        assert st == abi.UNSUPPORTED
    else:
        pieces = []
        for r in range(world):
            assert plugin.scrapgpu_cuda_sm100_shard(C.byref(full), 0, r, world, C.byref(v)) == abi.OK
            assert v.ne[0] == k // world and v.ne[1] == n and v.nb[1] == full.nb[1]
            pieces.append(view_bytes(image, v))
            if be > 1:
                assert np.array_equal(pieces[-1], tp.shard_cols(nat, dtype, k, r, k // world))
        assert np.array_equal(np.concatenate(pieces, axis=1), nat)


def test_shard_argument_errors(plugin):
    full = abi.tensor_desc(abi.Q4_K, [512, 8])
    v = abi.TensorDesc()
    assert plugin.scrapgpu_cuda_sm100_shard(C.byref(full), 1, 2, 2, C.byref(v)) == abi.INVALID_ARGUMENT      # rank >= world
    assert plugin.scrapgpu_cuda_sm100_shard(C.byref(full), 2, 0, 2, C.byref(v)) == abi.INVALID_ARGUMENT      # unknown split
    assert plugin.scrapgpu_cuda_sm100_shard(C.byref(full), 0, 0, 4, C.byref(v)) == abi.UNSUPPORTED           # 128 elements: not a whole block
    packed = abi.tensor_desc(abi.Q4_K, [512, 8], layout=abi.LAYOUT_R32)
    assert plugin.scrapgpu_cuda_sm100_shard(C.byref(packed), 1, 0, 2, C.byref(v)) == abi.UNSUPPORTED         # shards are cut from natural bytes
    assert plugin.scrapgpu_cuda_sm100_shard(None, 1, 0, 2, C.byref(v)) == abi.INVALID_ARGUMENT


def test_transport_entries_reject_foreign_objects(plugin):
    L = refapi.lib()
    assert L.scrapgpu_cpu_register() == abi.OK
    cpu = C.c_void_p()
    for i in range(L.scrapgpu_get_device_count()):
        L.scrapgpu_get_device(i, C.byref(cpu))
        info = abi.DeviceInfo()
        L.scrapgpu_device_info_init(C.byref(info), C.sizeof(info))
        L.scrapgpu_device_get_info(cpu, C.byref(info))
        if info.backend_name == b"cpu":
            break
    stream, buf = C.c_void_p(), C.c_void_p()
    assert L.scrapgpu_stream_create(cpu, C.byref(stream)) == abi.OK
    assert L.scrapgpu_buffer_alloc(cpu, 256, C.byref(buf)) == abi.OK
    t = abi.tensor_desc(abi.F32, [16], buffer=buf.value)
    plugin.scrapgpu_cuda_sm100_tensor_copy.argtypes = [C.c_void_p, C.POINTER(abi.TensorDesc), C.c_void_p, C.POINTER(abi.TensorDesc)]
    assert plugin.scrapgpu_cuda_sm100_tensor_copy(stream, C.byref(t), stream, C.byref(t)) == abi.INVALID_ARGUMENT
    group = C.c_void_p()
    devs = (C.c_void_p * 1)(cpu.value)
    plugin.scrapgpu_cuda_sm100_group_create.argtypes = [C.POINTER(C.c_void_p), C.c_size_t, C.c_size_t, C.POINTER(C.c_void_p)]
    assert plugin.scrapgpu_cuda_sm100_group_create(devs, 1, 64, C.byref(group)) == abi.INVALID_ARGUMENT
    assert plugin.scrapgpu_cuda_sm100_group_create(devs, 0, 64, C.byref(group)) == abi.UNSUPPORTED
    plugin.scrapgpu_cuda_sm100_group_free.argtypes = [C.c_void_p]
    assert plugin.scrapgpu_cuda_sm100_group_free(buf) == abi.INVALID_ARGUMENT
    L.scrapgpu_buffer_free(buf)
    L.scrapgpu_stream_free(stream)
