"""CPU restatement of the decode step of scrapgpulibrary_b200/decode.py with the oracle's ops (sgref.c): the same
op list the reference's CPU backend would run (GET_ROWS, RMS_NORM_MUL, MUL_MAT, ROPE, SET_ROWS, attention as the
core composes it, ADD, GLU, TOP_K).  Test infrastructure only."""
from __future__ import annotations

import numpy as np

from . import sgref


def decode_reference(cfg, weights: dict, first_token: int, steps: int, k_prefill=None, v_prefill=None, threads=None):
    """weights: name -> (dtype, natural blocks, K) for matrices, name -> float32 vector for norms (global, unsharded).
    Returns (tokens [steps], logits of the last step)."""
    c = cfg
    kc = [np.zeros((c.kv_heads, c.n_ctx, c.head_dim), np.float32) for _ in range(c.layers)]
    vc = [np.zeros((c.kv_heads, c.n_ctx, c.head_dim), np.float32) for _ in range(c.layers)]
    if k_prefill is not None:
        for i in range(c.layers):
            kc[i][:, :c.start_pos] = k_prefill[i]
            vc[i][:, :c.start_pos] = v_prefill[i]

    def mm(name, x):
        dt, nat, k = weights[name]
        return sgref.mul_mat(dt, nat, k, x[None, :], threads=threads)[0]

    token, out, logits = first_token, [], None
    scale = np.float32(1.0 / np.sqrt(np.float32(c.head_dim)))
    for step in range(steps):
        pos = c.start_pos + step
        dt, nat, k = weights["embed"]
        x = sgref.get_rows(dt, nat, k, np.array([token], np.int32))[0]
        proj = None
        for i in range(c.layers):
            if proj is None:
                xn = sgref.rms_norm(x[None, :], weights[f"l{i}.attn_norm"], eps=c.eps)[0]
            else:
                s, y = sgref.rms_norm(x[None, :], weights[f"l{i}.attn_norm"], add=proj[None, :], eps=c.eps)
                x, xn = s[0], y[0]
            q, kk, v = mm(f"l{i}.wq", xn), mm(f"l{i}.wk", xn), mm(f"l{i}.wv", xn)
            q, kk = q.reshape(c.heads, c.head_dim), kk.reshape(c.kv_heads, c.head_dim)
            if c.qk_norm:
                q = sgref.rms_norm(q, weights[f"l{i}.q_norm"], eps=c.eps)
                kk = sgref.rms_norm(kk, weights[f"l{i}.k_norm"], eps=c.eps)
            p = np.array([pos], np.int32)
            q = sgref.rope(q[None], p, c.head_dim, True, c.rope_base)[0]
            kk = sgref.rope(kk[None], p, c.head_dim, True, c.rope_base)[0]
            kc[i][:, pos] = kk
            vc[i][:, pos] = v.reshape(c.kv_heads, c.head_dim)
            att = sgref.attention(q[:, None, :], kc[i], vc[i], True, pos, scale)[:, 0, :].reshape(-1)
            proj = mm(f"l{i}.wo", att)
            s, y = sgref.rms_norm(x[None, :], weights[f"l{i}.ffn_norm"], add=proj[None, :], eps=c.eps)
            x, xn = s[0], y[0]
            act = sgref.swiglu(mm(f"l{i}.wgate", xn), mm(f"l{i}.wup", xn))
            proj = mm(f"l{i}.wdown", act)
        s, y = sgref.rms_norm(x[None, :], weights["out_norm"], add=proj[None, :], eps=c.eps)
        logits = mm("head", y[0])
        token = sgref.argmax(logits)
        out.append(token)
    return np.array(out, np.int32), logits


def random_weights(cfg, seed: int):
    """Seeded global weights for a (small) config: N(0, 0.02) matrices quantized by the oracle, norm gains near 1."""
    c = cfg
    rng = np.random.default_rng(seed)
    w = {}

    def mat(name, dtype, n, k, std=0.02):
        w[name] = (dtype, sgref.quantize(dtype, (rng.standard_normal((n, k)) * std).astype(np.float32)), k)

    mat("embed", 32, c.vocab, c.hidden, 1.0)
    for i in range(c.layers):
        vdt = 33 if c.more_bits(i) else 32
        for nm, n in (("attn_norm", c.hidden), ("ffn_norm", c.hidden), ("q_norm", c.head_dim), ("k_norm", c.head_dim)):
            w[f"l{i}.{nm}"] = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        mat(f"l{i}.wq", 32, c.heads * c.head_dim, c.hidden, 0.05)
        mat(f"l{i}.wk", 32, c.kv_heads * c.head_dim, c.hidden, 0.05)
        mat(f"l{i}.wv", vdt, c.kv_heads * c.head_dim, c.hidden, 0.05)
        mat(f"l{i}.wo", 32, c.hidden, c.heads * c.head_dim, 0.05)
        mat(f"l{i}.wgate", 32, c.ffn, c.hidden, 0.05)
        mat(f"l{i}.wup", 32, c.ffn, c.hidden, 0.05)
        mat(f"l{i}.wdown", vdt, c.hidden, c.ffn, 0.05)
    w["out_norm"] = (1.0 + 0.1 * rng.standard_normal(c.hidden)).astype(np.float32)
    mat("head", 33, c.vocab, c.hidden, 0.05)
    return w
