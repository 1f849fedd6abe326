"""Generates the committed golden fixtures of tests/golden/.

Run where the reference checkout is present (it compiles the unmodified reference into oracle/_ref/ and
drives it through its public C API):

    python tests/golden/make_golden.py

  ref_known_answers.json  hand-built blocks, fp16 bit patterns and MUL_MAT known answers restated from the
                          reference's own unit tests (tests/ref/ref_quant_tests.cpp:23-105,179-223,
                          tests/ref/ref_ops_tests.cpp:586-602,756-772), each re-checked here against the
                          compiled reference before it is written
  ref_seeded.npz          seeded inputs and the outputs the compiled reference gives for them: quantize
                          bytes, dequantized values, MUL_MAT for M in {1, 3, 4, 8}, RMS_NORM(+MUL, +ADD),
                          ROPE, SOFT_MAX, SwiGLU, and scaled-dot-product attention through the core's own
                          composition on the reference's CPU backend

The GPU box has no reference checkout: tests read only these files there.
"""
import ctypes as C
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import refapi  # noqa: E402
from scrapgpulibrary_b200 import abi  # noqa: E402


def known_answers():
    out = {"dequant_blocks": [], "f16_bits": [], "mul_mat": []}
    # Q4_0: d = 1.0, qs[j] = j  ->  y[j] = j - 8, y[16 + j] = -8          (ref_quant_tests.cpp:23-37)
    blk = np.zeros(18, np.uint8); blk[1] = 0x3C; blk[2:18] = np.arange(16)
    out["dequant_blocks"].append({"name": "q4_0 hand built", "dtype": abi.Q4_0, "block": blk.tolist(),
                                  "values": [float(j - 8) for j in range(16)] + [-8.0] * 16})
    # Q8_0: d = 0.5, qs[j] = j - 16  ->  y[j] = (j - 16) * 0.5                (:39-52)
    blk = np.zeros(34, np.uint8); blk[1] = 0x38; blk[2:34] = (np.arange(32) - 16).astype(np.int8).view(np.uint8)
    out["dequant_blocks"].append({"name": "q8_0 hand built", "dtype": abi.Q8_0, "block": blk.tolist(),
                                  "values": [(j - 16) * 0.5 for j in range(32)]})
    # Q4_K: d = 1, dmin = 0, scales[0..3] = 32, both nibbles l & 15  ->  32 * (j & 15) in the first half, 0 after  (:54-78)
    blk = np.zeros(144, np.uint8); blk[1] = 0x3C; blk[4:8] = 32
    l = np.arange(128); blk[16:144] = (l & 15) | ((l & 15) << 4)
    out["dequant_blocks"].append({"name": "q4_k hand built", "dtype": abi.Q4_K, "block": blk.tolist(),
                                  "values": [32.0 * (j & 15) for j in range(128)] + [0.0] * 128})
    # Q6_K: d = 1, all scales 8, qh = 0, ql[i] = (i % 16) | ((i + 3) % 16) << 4     (:80-105)
    blk = np.zeros(210, np.uint8); blk[209] = 0x3C; blk[192:208] = 8
    for half in range(2):
        for ll in range(64):
            i = half * 64 + ll
            blk[i] = (i % 16) | (((i + 3) % 16) << 4)
    vals = np.zeros(256, np.float32)
    for n in (0, 128):
        for ll in range(32):
            vals[n + ll] = 8.0 * ((ll % 16) - 32)
            vals[n + ll + 32] = 8.0 * (((ll + 32) % 16) - 32)
            vals[n + ll + 64] = 8.0 * (((ll + 3) % 16) - 32)
            vals[n + ll + 96] = 8.0 * (((ll + 35) % 16) - 32)
    out["dequant_blocks"].append({"name": "q6_k hand built", "dtype": abi.Q6_K, "block": blk.tolist(), "values": vals.tolist()})
    for c in out["dequant_blocks"]:
        got = refapi.dequantize(c["dtype"], np.array(c["block"], np.uint8)[None, :], len(c["values"]))[0]
        assert np.array_equal(got, np.array(c["values"], np.float32)), c["name"]

    # fp16 conversion bits (ref_quant_tests.cpp:179-223)
    f_in = [1.0, -2.0, 0.5, 65504.0, 65520.0, 65512.0, -0.0, 5.960464477539063e-08, 2.9802322387695312e-08, 8.940696716308594e-08]
    f_bits = [0x3C00, 0xC000, 0x3800, 0x7BFF, 0x7C00, 0x7BFF, 0x8000, 0x0001, 0x0000, 0x0002]
    src = np.array(f_in, np.float32); dst = np.zeros(len(f_in), np.uint16)
    refapi.execute(abi.OP_CPY, [(abi.tensor_desc(abi.F32, [len(f_in)]), src)], [(abi.tensor_desc(abi.F16, [len(f_in)]), dst)], abi.CpyParams())
    assert dst.tolist() == f_bits
    out["f16_bits"] = [{"value": v, "bits": b} for v, b in zip(f_in, f_bits)]

    # MUL_MAT known answers (ref_ops_tests.cpp:586-602) and the K-order cancellation row (:756-772)
    out["mul_mat"].append({"name": "f32 3x2", "k": 3, "w": [[1, 2, 3], [4, 5, 6]], "x": [[7, 9, 11], [8, 10, 12]], "y": [[58, 139], [64, 154]]})
    out["mul_mat"].append({"name": "k order", "k": 5, "w": [[1e20, 1.0, -1e20, 3.0, 4.0]] * 5, "x": [[1.0] * 5] * 4, "y": [[7.0] * 5] * 4})
    for c in out["mul_mat"]:
        w = np.array(c["w"], np.float32)
        got = refapi.mul_mat(abi.F32, w.view(np.uint8).reshape(w.shape[0], -1), c["k"], np.array(c["x"], np.float32))
        assert np.array_equal(got, np.array(c["y"], np.float32)), c["name"]
    return out


def cpu_device():
    L = refapi.lib()
    refapi.check(L.scrapgpu_cpu_register(), "cpu_register")
    dev = C.c_void_p()
    for i in range(L.scrapgpu_get_device_count()):
        refapi.check(L.scrapgpu_get_device(i, C.byref(dev)), "get_device")
        info = abi.DeviceInfo()
        L.scrapgpu_device_info_init(C.byref(info), C.sizeof(info))
        L.scrapgpu_device_get_info(dev, C.byref(info))
        if info.backend_name == b"cpu":
            return dev
    raise RuntimeError("the reference's cpu backend did not register")


def ref_attention(q, k, v, causal, offset, scale):
    """scrapgpu_scaled_dot_product_attention on the reference's CPU backend.  q [Hq, nq, D] etc. (C order)."""
    L = refapi.lib()
    dev = cpu_device()
    stream = C.c_void_p()
    refapi.check(L.scrapgpu_stream_create(dev, C.byref(stream)), "stream_create")
    hq, nq, d = q.shape
    hkv, nk, _ = k.shape
    dv = v.shape[2]
    out = np.zeros((hq, nq, dv), np.float32)
    bufs = []

    def dev_tensor(a, ne):
        b = C.c_void_p()
        refapi.check(L.scrapgpu_buffer_alloc(dev, a.nbytes, C.byref(b)), "buffer_alloc")
        bufs.append(b)
        t = abi.tensor_desc(abi.F32, ne, buffer=b.value)
        refapi.check(L.scrapgpu_tensor_upload(stream, C.byref(t), a.ctypes.data_as(C.c_void_p), a.nbytes), "upload")
        return t

    tq, tk, tv = dev_tensor(q, [d, nq, hq, 1]), dev_tensor(k, [d, nk, hkv, 1]), dev_tensor(v, [dv, nk, hkv, 1])
    to = dev_tensor(out, [dv, nq, hq, 1])
    p = abi.AttentionParams()
    p.struct_size = C.sizeof(p)
    p.query, p.key, p.value, p.output = C.pointer(tq), C.pointer(tk), C.pointer(tv), C.pointer(to)
    p.query_position_offset = offset
    p.max_workspace_bytes = 64 << 20
    p.causal = int(causal)
    p.scale = scale
    refapi.check(L.scrapgpu_scaled_dot_product_attention(dev, stream, C.byref(p)), "sdpa")
    refapi.check(L.scrapgpu_tensor_download(stream, C.byref(to), out.ctypes.data_as(C.c_void_p), out.nbytes), "download")
    for b in bufs:
        L.scrapgpu_buffer_free(b)
    L.scrapgpu_stream_free(stream)
    return out


def seeded():
    rng = np.random.default_rng(20261125)
    z = {}
    k, n = 512, 12
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    w[2, :256] = 0.0
    w[4, :256] = -1.0 - 0.5 * np.abs(w[4, :256])
    z["w"] = w
    x = rng.standard_normal((8, k)).astype(np.float32)
    z["x"] = x
    for dt in (abi.Q4_0, abi.Q8_0, abi.Q4_K, abi.Q6_K):
        nm = abi.DTYPE_NAMES[dt]
        q = refapi.quantize(dt, w, threads=1)
        z[f"{nm}_blocks"] = q
        z[f"{nm}_dequant"] = refapi.dequantize(dt, q, k)
        for m in (1, 3, 4, 8):
            z[f"{nm}_mul_mat_m{m}"] = refapi.mul_mat(dt, q, k, x[:m])

    # RMS_NORM family: rows of 96
    ne0, rows = 96, 5
    a = rng.standard_normal((rows, ne0)).astype(np.float32) * 3
    b = rng.standard_normal((rows, ne0)).astype(np.float32)
    g = rng.standard_normal(ne0).astype(np.float32)
    z["norm_a"], z["norm_b"], z["norm_w"] = a, b, g
    ta, tw = abi.tensor_desc(abi.F32, [ne0, rows]), abi.tensor_desc(abi.F32, [ne0])
    eps = abi.RmsNormParams(); eps.eps = 1e-6
    y = np.zeros_like(a); refapi.execute(abi.OP_RMS_NORM, [(ta, a)], [(ta, y)], eps); z["rms_norm"] = y.copy()
    y = np.zeros_like(a); refapi.execute(abi.OP_RMS_NORM_MUL, [(ta, a), (tw, g)], [(ta, y)], eps); z["rms_norm_mul"] = y.copy()
    s = np.zeros_like(a); y = np.zeros_like(a)
    refapi.execute(abi.OP_ADD_RMS_NORM_MUL, [(ta, a), (ta, b), (tw, g)], [(ta, s), (ta, y)], eps)
    z["add_rms_norm_mul_sum"], z["add_rms_norm_mul"] = s.copy(), y.copy()

    # ROPE: [ne0 = 64, heads = 3, tokens = 4], NEOX and NORMAL, theta 1e6, n_dims 64 and 32
    xr = rng.standard_normal((4, 3, 64)).astype(np.float32)
    pos = np.array([0, 1, 1024, 1151], np.int32)
    z["rope_x"], z["rope_pos"] = xr, pos
    tx, tp = abi.tensor_desc(abi.F32, [64, 3, 4]), abi.tensor_desc(abi.I32, [4])
    for mode, nd in ((abi.ROPE_NEOX, 64), (abi.ROPE_NORMAL, 64), (abi.ROPE_NEOX, 32)):
        rp = abi.RopeParams(); rp.mode = mode; rp.n_dims = nd; rp.n_ctx_orig = 4096; rp.freq_base = 1e6
        rp.freq_scale = 1.0; rp.ext_factor = 0.0; rp.attn_factor = 1.0; rp.beta_fast = 32.0; rp.beta_slow = 1.0
        y = np.zeros_like(xr); refapi.execute(abi.OP_ROPE, [(tx, xr), (tp, pos)], [(tx, y)], rp)
        z[f"rope_mode{mode}_nd{nd}"] = y.copy()

    # SOFT_MAX with scale and an additive mask holding -inf
    sx = rng.standard_normal((6, 77)).astype(np.float32) * 4
    mk = np.zeros((6, 77), np.float32); mk[:, 50:] = -np.inf; mk[2, :] = rng.standard_normal(77)
    z["softmax_x"], z["softmax_mask"] = sx, mk
    ts = abi.tensor_desc(abi.F32, [77, 6])
    sp = abi.SoftMaxParams(); sp.scale = 0.125
    y = np.zeros_like(sx); refapi.execute(abi.OP_SOFT_MAX, [(ts, sx), (ts, mk)], [(ts, y)], sp); z["softmax_masked"] = y.copy()
    y = np.zeros_like(sx); refapi.execute(abi.OP_SOFT_MAX, [(ts, sx)], [(ts, y)], sp); z["softmax_plain"] = y.copy()

    # SwiGLU split inputs
    gx, gg = rng.standard_normal(200).astype(np.float32) * 3, rng.standard_normal(200).astype(np.float32)
    z["glu_x"], z["glu_g"] = gx, gg
    tg = abi.tensor_desc(abi.F32, [200])
    gp = abi.GluParams(); gp.kind = abi.GLU_SWIGLU; gp.split_inputs = 1
    y = np.zeros_like(gx); refapi.execute(abi.OP_GLU, [(tg, gx), (tg, gg)], [(tg, y)], gp); z["swiglu"] = y.copy()

    # attention through the core's composition on the reference's CPU backend: GQA 4 query heads on 2 KV heads
    aq = rng.standard_normal((4, 1, 32)).astype(np.float32)
    ak = rng.standard_normal((2, 40, 32)).astype(np.float32)
    av = rng.standard_normal((2, 40, 32)).astype(np.float32)
    z["att_q"], z["att_k"], z["att_v"] = aq, ak, av
    z["att_causal_off29"] = ref_attention(aq, ak, av, True, 29, 1.0 / np.sqrt(32.0))
    z["att_full"] = ref_attention(aq, ak, av, False, 0, 1.0 / np.sqrt(32.0))
    aq3 = rng.standard_normal((4, 3, 32)).astype(np.float32)
    z["att_q3"] = aq3
    z["att_causal_q3_off2"] = ref_attention(aq3, ak, av, True, 2, 0.2)
    return z


if __name__ == "__main__":
    if not refapi.build():
        raise SystemExit("the reference checkout is not available: cannot regenerate the fixtures")
    with open(os.path.join(HERE, "ref_known_answers.json"), "w") as f:
        json.dump(known_answers(), f, indent=1)
    np.savez_compressed(os.path.join(HERE, "ref_seeded.npz"), **seeded())
    print("wrote", os.listdir(HERE))
