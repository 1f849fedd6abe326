"""The allocation-free attention entry (sm100_attention_static) against the regular one.

Who needs it: callers that cannot allocate device memory when they call -- a serving loop that has already given
all HBM to its own pools, a thread that must not wait on the driver's allocator, a process under an outside memory
budget.  For them the split-key partials live in a fixed array inside the library instead of a scratch buffer
allocated on first use.  The test drives both entries through the C ABI on the same inputs, twice in a row (the
array keeps the previous call's contents, which must not leak into the next result), and checks the refusal of a
shape that does not fit.  Collected last on purpose: a run that stops at the first failure has then run every other
test already."""
import ctypes as C

import numpy as np
import pytest

from oracle import sgref
from tests import util as U

pytestmark = pytest.mark.gpu
TOL = 1e-6   # NMSE, the bar of the other attention tests


def call(capi, stream, entry, q, k, v, causal, offset, scale):
    hq, nq, d = q.shape
    hkv, nk, _ = k.shape
    dv = v.shape[2]
    qb, kb, vb = (U.to_device(capi, stream, a) for a in (q, k, v))
    ob, optr = U.guarded_output(capi, stream, hq * nq * dv)
    capi.check(entry(stream.handle, qb.at(), kb.at(), vb.at(), None, 1, C.c_void_p(optr), d, dv, nq, nk, hq, hkv, int(causal), offset, None, scale), "attention")
    stream.sync()
    out = U.read_guarded(capi, stream, ob, hq * nq * dv).reshape(hq, nq, dv).copy()
    for b in (qb, kb, vb, ob):
        b.free()
    return out


def test_static_scratch_attention_matches_regular_entry(sm100, stream):
    lib = sm100.lib()
    assert lib.sm100_attention_static_capacity() == 4 << 20
    rng = np.random.default_rng(21)
    # first a decode-shaped call, then a different shape that reuses (and only partly overwrites) the array
    cases = [(32, 8, 128, 1152, 1, True, 1100), (8, 2, 64, 300, 3, True, 5)]
    for rep in range(2):
        for hq, hkv, d, nk, nq, causal, off in cases:
            q = rng.standard_normal((hq, nq, d)).astype(np.float32)
            k = rng.standard_normal((hkv, nk, d)).astype(np.float32)
            v = rng.standard_normal((hkv, nk, d)).astype(np.float32)
            scale = float(1.0 / np.sqrt(d))
            want = call(sm100, stream, lib.sm100_attention, q, k, v, causal, off, scale)
            got = call(sm100, stream, lib.sm100_attention_static, q, k, v, causal, off, scale)
            assert sgref.nmse(got, want) <= TOL, (rep, hq, nk)
            assert sgref.nmse(got, sgref.attention(q, k, v, causal, off, scale)) <= TOL


def test_static_scratch_survives_dirty_ticket_counters(sm100, stream):
    """The first 64 KiB of the built-in array are the ticket counters of the single-launch merge.  A call that raced
    with another one could leave them non-zero; the entry clears the ones it uses before every launch, so a later call
    must be right whatever they hold.  Here they are overwritten with ones on purpose."""
    lib = sm100.lib()
    p = C.c_void_p()
    sm100.check(lib.sm100_attention_static_prepare(C.byref(p)), "static_prepare")
    assert p.value
    rng = np.random.default_rng(22)
    hq, hkv, d, nk, nq, off = 32, 8, 128, 1152, 1, 1100
    q = rng.standard_normal((hq, nq, d)).astype(np.float32)
    k = rng.standard_normal((hkv, nk, d)).astype(np.float32)
    v = rng.standard_normal((hkv, nk, d)).astype(np.float32)
    scale = float(1.0 / np.sqrt(d))
    want = sgref.attention(q, k, v, True, off, scale)
    for rep in range(2):
        sm100.check(lib.sm100_memset(stream.handle, p, 1, 64 << 10, 1), "memset")
        got = call(sm100, stream, lib.sm100_attention_static, q, k, v, True, off, scale)
        assert sgref.nmse(got, want) <= TOL, rep


def test_static_scratch_refuses_oversized_shapes(sm100, stream):
    lib = sm100.lib()
    b = sm100.Buffer(1 << 16)
    # 4096 queries x 32 heads x >= 1 split x 130 floats is far beyond 4 MiB: refused before anything is launched
    st = lib.sm100_attention_static(stream.handle, b.at(), b.at(), b.at(), None, 1, b.at(), 128, 128, 4096, 64, 32, 8, 1, 0, None, 1.0)
    assert st == 1
    assert b"built-in array" in lib.sm100_last_error()
    b.free()
