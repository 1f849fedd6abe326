"""Layer-stack decode harness: a Qwen3-8B-shaped transformer decode step built from the backend's ops, one
process per GPU, tensor-parallel over `torch.distributed`.

The reference has no model runner of its own (models run through llama.cpp on top of its ggml adapter); the
closest thing is examples/pipeline_mlp.c:124-300, which builds per-layer descriptors once and then issues one
scrapgpu_op_execute per op and token.  This harness does the same for the decode step the benchmark names --
GET_ROWS -> per layer { RMS_NORM_MUL -> Q/K/V MUL_MAT -> per-head q/k RMS_NORM_MUL -> ROPE -> SET_ROWS into the
f32 KV cache -> causal GQA attention -> o MUL_MAT -> ADD_RMS_NORM_MUL -> gate/up MUL_MAT -> SwiGLU -> down
MUL_MAT } -> ADD_RMS_NORM_MUL -> head MUL_MAT -> TOP_K(1) -- straight on the C ABI of libscrapgpu_sm100, with the
whole step recorded once in a CUDA graph (the plan seat of the reference API) and replayed per token: position,
token id and KV write index all live on the device.

Tensor parallelism (new: the reference only splits layers across devices, docs/MULTI_GPU.md): weight rows are
sharded column-parallel for Q/K/V/gate/up and the vocabulary head, row-parallel (K shards) for o and down with
an all-reduce of the 4096-float partial after each, attention by KV head.  PyTorch supplies device memory, the
stream, graph capture and the NCCL process group; every kernel on the path is this repository's.
"""
from __future__ import annotations

import ctypes as C
import os
import zlib
from dataclasses import dataclass

import numpy as np
import torch

from . import capi, synth, tp

Q4_K, Q6_K = 32, 33


@dataclass
class DecodeConfig:
    """Defaults: Qwen3-8B shapes (36 layers, hidden 4096, 32 query / 8 KV heads of 128, FFN 12288, vocab 151936)."""
    layers: int = 36
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 12288
    vocab: int = 151936
    n_ctx: int = 1152
    start_pos: int = 1024
    rope_base: float = 1e6
    eps: float = 1e-6
    qk_norm: bool = True

    def more_bits(self, layer: int) -> bool:
        """Which layers keep attn_v and ffn_down in Q6_K in a Q4_K_M mix: the published rule of llama.cpp's
        quantizer (first and last eighth, and every third layer in between)."""
        n = self.layers
        return layer < n // 8 or layer >= 7 * n // 8 or (layer - n // 8) % 3 == 2


class SyntheticWeights:
    """A seeded synthetic model of a DecodeConfig's shapes, defined GLOBALLY (unsharded) and independent of rank
    and world size, so that every tensor-parallel layout shards the same model and the CPU oracle can run it too.

    Behaves like the `weights` mapping of DecodeModel / oracle.decode_ref: name -> (dtype, natural blocks [N, row_bytes],
    K) for matrices, name -> float32 vector for norm gains.  Real GGUF files are not available offline; generating
    8 G distinct weights per rank would take minutes, so a matrix is built from one base matrix per (dtype, shape) --
    valid blocks of seeded N(0, 0.02) weights (synth.py) -- whose rows are rotated by a per-name amount; where a matrix
    has more rows than its base (embedding, vocabulary head), each repetition of the base gets its own low bits in the
    blocks' f16 scale, so no two rows of the matrix are equal (equal rows would tie in the greedy arg-max)."""

    BASE_ROWS = 16384

    def __init__(self, cfg: DecodeConfig, seed: int = 0x5CA9):
        self.cfg, self.seed = cfg, seed
        self._base = {}
        c = cfg
        self.shapes = {"embed": (Q4_K, c.vocab, c.hidden), "head": (Q6_K, c.vocab, c.hidden)}
        rng = np.random.default_rng(seed + 17)
        self.vectors = {}
        for i in range(c.layers):
            vdt = Q6_K if c.more_bits(i) else Q4_K
            for nm, n in (("attn_norm", c.hidden), ("ffn_norm", c.hidden), ("q_norm", c.head_dim), ("k_norm", c.head_dim)):
                self.vectors[f"l{i}.{nm}"] = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
            self.shapes[f"l{i}.wq"] = (Q4_K, c.heads * c.head_dim, c.hidden)
            self.shapes[f"l{i}.wk"] = (Q4_K, c.kv_heads * c.head_dim, c.hidden)
            self.shapes[f"l{i}.wv"] = (vdt, c.kv_heads * c.head_dim, c.hidden)
            self.shapes[f"l{i}.wo"] = (Q4_K, c.hidden, c.heads * c.head_dim)
            self.shapes[f"l{i}.wgate"] = (Q4_K, c.ffn, c.hidden)
            self.shapes[f"l{i}.wup"] = (Q4_K, c.ffn, c.hidden)
            self.shapes[f"l{i}.wdown"] = (vdt, c.hidden, c.ffn)
        self.vectors["out_norm"] = (1.0 + 0.1 * rng.standard_normal(c.hidden)).astype(np.float32)

    def __contains__(self, name) -> bool:
        return name in self.shapes or name in self.vectors

    def _base_matrix(self, dtype: int, n: int, k: int) -> np.ndarray:
        key = (dtype, min(n, self.BASE_ROWS), k)
        if key not in self._base:
            self._base[key] = synth.quantized_matrix(dtype, (self.seed * 31 + dtype * 7 + key[1] * 3 + k) % (1 << 31), key[1], k)
        return self._base[key]

    def rows(self, name: str, lo: int, count: int) -> np.ndarray:
        """Rows [lo, lo + count) of the global matrix `name` (natural blocks)."""
        dtype, n, k = self.shapes[name]
        base = self._base_matrix(dtype, n, k)
        rot = (zlib.crc32(name.encode()) % 977) * 3
        src = (np.arange(lo, lo + count, dtype=np.int64) - rot) % n      # row of the unrotated tiling
        out = base[src % base.shape[0]]                                    # a copy (fancy indexing)
        if n > base.shape[0]:
            be, bb = tp.BLOCK[dtype]
            d_at = 0 if dtype == Q4_K else bb - 2                          # byte offset of the block's f16 scale d
            blocks = out.reshape(count, k // be, bb)
            rep = (src // base.shape[0]).astype(np.uint8)                  # < 16 for every shape in use
            blocks[:, :, d_at] = (blocks[:, :, d_at] & 0xF0) | rep[:, None]
        return out

    def __getitem__(self, name):
        if name in self.vectors:
            return self.vectors[name]
        dtype, n, k = self.shapes[name]
        return dtype, self.rows(name, 0, n), k


def _dev(t: torch.Tensor) -> C.c_void_p:
    return C.c_void_p(t.data_ptr())


class Weight:
    """A quantized weight matrix [K, N] resident on the device in the backend-packed layout."""

    def __init__(self, model: "DecodeModel", dtype: int, natural: np.ndarray, k: int):
        self.dtype, self.k, self.n = dtype, k, natural.shape[0]
        nat = torch.from_numpy(np.ascontiguousarray(natural)).to(model.device)
        self.data = torch.empty(nat.numel(), dtype=torch.uint8, device=model.device)
        capi.check(model.L.sm100_pack_device(model.stream, dtype, k, self.n, _dev(nat), _dev(self.data)), "pack_device")
        torch.cuda.synchronize(model.device)
        self.nbytes = nat.numel()


class DecodeModel:
    def __init__(self, cfg: DecodeConfig, rank: int = 0, world: int = 1, device_index: int = 0, seed: int = 0x5CA9,
                 weights: dict | None = None, allreduce=None, fuse: bool = True):
        """weights: mapping name -> (dtype, natural uint8 [N_global, row_bytes], K_global) with GLOBAL matrices (sharded
        here) and name -> f32 vector for the norm gains; default: SyntheticWeights(cfg, seed), the same global model
        for every rank and world size.  allreduce: callable on a torch tensor (default: torch.distributed when
        world > 1)."""
        if weights is None:
            weights = SyntheticWeights(cfg, seed)
        assert cfg.heads % cfg.kv_heads == 0 and cfg.kv_heads % world == 0 and cfg.ffn % (256 * world) == 0
        self.cfg, self.rank, self.world = cfg, rank, world
        self.device = torch.device("cuda", device_index)
        torch.cuda.set_device(self.device)
        self.L = capi.lib()
        capi.check(self.L.sm100_set_device(device_index), "set_device")
        self.tstream = torch.cuda.Stream(self.device)
        self.stream = C.c_void_p(self.tstream.cuda_stream)
        self.allreduce = allreduce
        self.fuse = fuse   # fold RMS norm / SwiGLU into the Q4_K projections that consume them (one launch each)
        self.fuse_swiglu = fuse and os.environ.get("SM100_FUSE_SWIGLU", "1") != "0"
        # the all-reduce of the row-parallel projections inside their matvec launch (sm100_mul_mat_allreduce)
        self.fuse_exchange = fuse and os.environ.get("SM100_TP_FUSED", "1") != "0"
        # SwiGLU in the epilogue of the gate / up launch (sm100_mul_mat_glu) instead of in front of the down projection
        self.fuse_glu = fuse and os.environ.get("SM100_FUSE_GLU", "1") != "0"
        c = cfg
        self.hq, self.hkv = c.heads // world, c.kv_heads // world
        self.q_dim, self.kv_dim, self.ffn = self.hq * c.head_dim, self.hkv * c.head_dim, c.ffn // world
        self.vocab_lo, self.vocab_n = tp.vocab_shard(c.vocab, rank, world)
        self.weight_bytes = 0
        f32 = dict(dtype=torch.float32, device=self.device)
        with torch.cuda.stream(self.tstream):
            self.embed = self._weight("embed", Q4_K, c.vocab, c.hidden, weights, seed, shard=None)
            self.layers = []
            rng = np.random.default_rng(seed + 17)
            for i in range(c.layers):
                vdt = Q6_K if c.more_bits(i) else Q4_K
                lw = {
                    "attn_norm": torch.from_numpy(self._norm_w(weights, f"l{i}.attn_norm", c.hidden, rng)).to(self.device),
                    "ffn_norm": torch.from_numpy(self._norm_w(weights, f"l{i}.ffn_norm", c.hidden, rng)).to(self.device),
                    "q_norm": torch.from_numpy(self._norm_w(weights, f"l{i}.q_norm", c.head_dim, rng)).to(self.device),
                    "k_norm": torch.from_numpy(self._norm_w(weights, f"l{i}.k_norm", c.head_dim, rng)).to(self.device),
                    "wq": self._weight(f"l{i}.wq", Q4_K, c.heads * c.head_dim, c.hidden, weights, seed + i, shard=("rows", self.hq * c.head_dim)),
                    "wk": self._weight(f"l{i}.wk", Q4_K, c.kv_heads * c.head_dim, c.hidden, weights, seed + i, shard=("rows", self.hkv * c.head_dim)),
                    "wv": self._weight(f"l{i}.wv", vdt, c.kv_heads * c.head_dim, c.hidden, weights, seed + i, shard=("rows", self.hkv * c.head_dim)),
                    "wo": self._weight(f"l{i}.wo", Q4_K, c.hidden, c.heads * c.head_dim, weights, seed + i, shard=("cols", self.q_dim)),
                    "wgate": self._weight(f"l{i}.wgate", Q4_K, c.ffn, c.hidden, weights, seed + i, shard=("rows", self.ffn)),
                    "wup": self._weight(f"l{i}.wup", Q4_K, c.ffn, c.hidden, weights, seed + i, shard=("rows", self.ffn)),
                    "wdown": self._weight(f"l{i}.wdown", vdt, c.hidden, c.ffn, weights, seed + i, shard=("cols", self.ffn)),
                    "k_cache": torch.zeros(self.hkv, c.n_ctx, c.head_dim, **f32),
                    "v_cache": torch.zeros(self.hkv, c.n_ctx, c.head_dim, **f32),
                }
                self.layers.append(lw)
            self.out_norm = torch.from_numpy(self._norm_w(weights, "out_norm", c.hidden, rng)).to(self.device)
            self.head = self._weight("head", Q6_K, c.vocab, c.hidden, weights, seed + 999, shard=("rows", self.vocab_n, self.vocab_lo))
            # activations
            self.token = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.pos = torch.full((1,), c.start_pos, dtype=torch.int32, device=self.device)
            self.x = torch.zeros(c.hidden, **f32)          # residual stream
            self.x2 = torch.zeros(c.hidden, **f32)         # its alternate buffer (fused launches do not update in place)
            self.xn = torch.zeros(c.hidden, **f32)         # normalised
            self.q = torch.zeros(self.q_dim, **f32)
            self.k = torch.zeros(self.kv_dim, **f32)
            self.v = torch.zeros(self.kv_dim, **f32)
            self.att = torch.zeros(self.q_dim, **f32)
            self.proj = torch.zeros(c.hidden, **f32)       # o / down output (partial under TP)
            self.gate = torch.zeros(self.ffn, **f32)
            self.up = torch.zeros(self.ffn, **f32)
            self.act = torch.zeros(self.ffn, **f32)
            self.logits = torch.zeros(max(1, self.vocab_n), **f32)
            self.best = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.cand = torch.zeros(2, **f32)              # (best logit, global index) of this rank
            self.cands = torch.zeros(world, 2, **f32)
            positions = np.arange(c.n_ctx)
            self.rope = torch.from_numpy(self._rope_table(positions)).to(self.device)
            self.tokens_out = torch.zeros(4096, dtype=torch.int32, device=self.device)
            self.step_index = torch.zeros(1, dtype=torch.int64, device=self.device)
        torch.cuda.synchronize(self.device)
        self.graph = None
        self.kv_bytes_per_pos = 2 * 4 * c.head_dim * self.hkv * c.layers

    # ---- construction helpers -------------------------------------------------------------------------
    def _norm_w(self, weights, name, n, rng):
        if weights is not None and name in weights:
            return np.ascontiguousarray(weights[name], dtype=np.float32)
        return (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)

    def _rope_table(self, positions) -> np.ndarray:
        """(cos, sin) with the reference's recipe (src/core/ref/ops.cpp:559-601): sequential f32 products, libm."""
        c = self.cfg
        half = c.head_dim // 2
        out = np.empty((len(positions), half, 2), np.float32)
        ts = np.float32(np.power(np.float32(c.rope_base), np.float32(-2.0) / np.float32(c.head_dim), dtype=np.float32))
        theta = positions.astype(np.float32)
        import math
        for j in range(half):
            for i in range(len(positions)):
                out[i, j, 0] = np.float32(math.cos(float(theta[i])))
                out[i, j, 1] = np.float32(math.sin(float(theta[i])))
            theta = (theta * ts).astype(np.float32)
        return out

    def _weight(self, name, dtype, n_global, k_global, weights, seed, shard):
        """shard: None (replicated), ("rows", n_local[, lo]) or ("cols", k_local)."""
        if isinstance(weights, SyntheticWeights):
            dt, n_all, kg = weights.shapes[name]
            assert dt == dtype and kg == k_global and n_all == n_global
            if shard is not None and shard[0] == "rows":
                lo = shard[2] if len(shard) > 2 else self.rank * shard[1]
                loc, k = weights.rows(name, lo, shard[1]), k_global      # only this rank's rows are materialised
            elif shard is None:
                loc, k = weights.rows(name, 0, n_global), k_global
            else:
                loc, k = tp.shard_cols(weights.rows(name, 0, n_global), dtype, k_global, self.rank, shard[1]), shard[1]
        else:
            dt, nat, kg = weights[name]
            assert dt == dtype and kg == k_global
            nat = np.asarray(nat)
            if shard is None:
                loc, k = nat, k_global
            elif shard[0] == "rows":
                lo = shard[2] if len(shard) > 2 else self.rank * shard[1]
                loc, k = tp.shard_rows(nat, lo, shard[1]), k_global
            else:
                loc, k = tp.shard_cols(nat, dtype, k_global, self.rank, shard[1]), shard[1]
        if loc.shape[0] == 0:
            return None
        w = Weight(self, dtype, loc, k)
        self.weight_bytes += w.nbytes
        return w

    # ---- one decode step ------------------------------------------------------------------------------
    def _mm(self, w: Weight, x: torch.Tensor, y: torch.Tensor):
        capi.check(self.L.sm100_mul_mat(self.stream, w.dtype, 1, _dev(w.data), 0, w.k, w.n, _dev(x), w.k, 1, _dev(y), w.n), "mul_mat")

    def _mm_multi(self, ws, x: torch.Tensor, ys):
        """MUL_MAT_MULTI: weight tensors that share the activation column go out in one launch where the library can."""
        n = len(ws)
        k = ws[0].k
        assert all(w.k == k for w in ws)
        dts = (C.c_int * n)(*[w.dtype for w in ws])
        lays = (C.c_int * n)(*([1] * n))
        wp = (C.c_void_p * n)(*[w.data.data_ptr() for w in ws])
        yp = (C.c_void_p * n)(*[y.data_ptr() for y in ys])
        ns = (C.c_int64 * n)(*[w.n for w in ws])
        capi.check(self.L.sm100_mul_mat_multi(self.stream, n, dts, lays, wp, k, ns, _dev(x), yp), "mul_mat_multi")

    def _mm_fused(self, prologue: int, a, b, norm_w, sum_out, x_out, ws, ys):
        """MUL_MAT_MULTI with the producer of the activation column (1 = SwiGLU(a, b), 2 = (ADD_)RMS_NORM_MUL) in the
        same launch; packed Q4_K tensors only."""
        n = len(ws)
        k = ws[0].k
        dts = (C.c_int * n)(*[w.dtype for w in ws])
        lays = (C.c_int * n)(*([1] * n))
        wp = (C.c_void_p * n)(*[w.data.data_ptr() for w in ws])
        yp = (C.c_void_p * n)(*[y.data_ptr() for y in ys])
        ns = (C.c_int64 * n)(*[w.n for w in ws])
        opt = lambda t: _dev(t) if t is not None else None
        capi.check(self.L.sm100_mul_mat_fused(self.stream, prologue, _dev(a), opt(b), opt(norm_w), self.cfg.eps, opt(sum_out), opt(x_out), n,
                                              dts, lays, wp, k, ns, yp), "mul_mat_fused")

    def _mm_reduce(self, w: Weight, prologue: int, a: torch.Tensor, b, y: torch.Tensor) -> bool:
        """A row-parallel projection with its all-reduce in one launch (sm100_mul_mat_allreduce) where the exchange is the
        library's own (PeerAllReduce) and the tensor is packed Q4_K; False: the caller runs the separate launches."""
        ctx = getattr(self.allreduce, "ctx", None)
        if self.world == 1 or ctx is None or not self.fuse_exchange or w.dtype != Q4_K or w.n % 16 != 0:
            return False
        capi.check(self.L.sm100_mul_mat_allreduce(ctx, self.stream, prologue, _dev(a), _dev(b) if b is not None else None, w.dtype, 1, _dev(w.data),
                                                  w.k, w.n, _dev(y)), "mul_mat_allreduce")
        return True

    def _reduce(self, t: torch.Tensor):
        if self.world > 1:
            if self.allreduce is not None:
                self.allreduce(t)
            else:
                torch.distributed.all_reduce(t)

    def enqueue_step(self):
        """Enqueues one token on self.tstream (must be the current torch stream)."""
        c, L, s = self.cfg, self.L, self.stream
        chk = capi.check
        chk(L.sm100_get_rows(s, self.embed.dtype, 1, _dev(self.embed.data), 0, c.hidden, c.vocab, _dev(self.token), 1, _dev(self.x), c.hidden), "get_rows")
        scale = float(1.0 / np.sqrt(c.head_dim))
        # the residual stream alternates between two buffers: the fused launches read the old one in every CTA
        # while one CTA writes the updated one
        x_cur, x_alt = self.x, self.x2
        for i, lw in enumerate(self.layers):
            add = self.proj if i > 0 else None     # the previous layer's FFN output joins the residual here
            qkv = [lw["wq"], lw["wk"], lw["wv"]]
            q4 = [w for w in qkv if w.dtype == Q4_K]
            if self.fuse and len(q4) >= 2:
                # ADD_RMS_NORM_MUL folded into the Q4_K projections; a Q6_K value projection reads the normalised row
                outs = {id(lw["wq"]): self.q, id(lw["wk"]): self.k, id(lw["wv"]): self.v}
                need_xn = len(q4) < 3
                self._mm_fused(2, x_cur, add, lw["attn_norm"], x_alt if add is not None else None, self.xn if need_xn else None,
                               q4, [outs[id(w)] for w in q4])
                if add is not None:
                    x_cur, x_alt = x_alt, x_cur
                if need_xn:
                    self._mm(lw["wv"], self.xn, self.v)
            else:
                if add is None:
                    chk(L.sm100_rms_norm(s, _dev(x_cur), None, _dev(lw["attn_norm"]), None, _dev(self.xn), c.hidden, 1, c.eps), "rms_norm")
                else:
                    chk(L.sm100_rms_norm(s, _dev(x_cur), _dev(add), _dev(lw["attn_norm"]), _dev(x_cur), _dev(self.xn), c.hidden, 1, c.eps), "add_rms_norm")
                self._mm_multi(qkv, self.xn, [self.q, self.k, self.v])
            # per-head norm + rotation + KV store + attention over the cache: one launch (two where the shapes do not allow it)
            chk(L.sm100_attention_decode(s, _dev(self.q), _dev(self.k), _dev(self.v), _dev(lw["q_norm"]) if c.qk_norm else None,
                                         _dev(lw["k_norm"]) if c.qk_norm else None, _dev(self.pos), _dev(self.rope), 0, c.n_ctx, _dev(lw["k_cache"]),
                                         _dev(lw["v_cache"]), _dev(self.att), c.head_dim, self.hq, self.hkv, c.n_ctx, c.eps, c.rope_base, 1, scale),
                "attention_decode")
            if not self._mm_reduce(lw["wo"], 0, self.att, None, self.proj):
                self._mm(lw["wo"], self.att, self.proj)
                self._reduce(self.proj)
            glu_done = False
            if self.fuse and self.fuse_glu and lw["wgate"].dtype == Q4_K and lw["wup"].dtype == Q4_K and lw["wgate"].n == lw["wup"].n:
                # ADD_RMS_NORM_MUL in the prologue, gate and up in one launch, SwiGLU in its epilogue: act comes out directly
                st = L.sm100_mul_mat_glu(s, 2, _dev(x_cur), _dev(self.proj), _dev(lw["ffn_norm"]), c.eps, _dev(x_alt), None, Q4_K, 1,
                                         _dev(lw["wgate"].data), _dev(lw["wup"].data), lw["wgate"].k, lw["wgate"].n, None, None, _dev(self.act))
                if st != 1:    # 1 = UNSUPPORTED: the separate launches below
                    chk(st, "mul_mat_glu")
                    glu_done = True
                    x_cur, x_alt = x_alt, x_cur
            if glu_done:
                if not self._mm_reduce(lw["wdown"], 0, self.act, None, self.proj):
                    self._mm(lw["wdown"], self.act, self.proj)
                    self._reduce(self.proj)
                continue
            if self.fuse:
                self._mm_fused(2, x_cur, self.proj, lw["ffn_norm"], x_alt, None, [lw["wgate"], lw["wup"]], [self.gate, self.up])
                x_cur, x_alt = x_alt, x_cur
            else:
                chk(L.sm100_rms_norm(s, _dev(x_cur), _dev(self.proj), _dev(lw["ffn_norm"]), _dev(x_cur), _dev(self.xn), c.hidden, 1, c.eps), "add_rms_norm")
                self._mm_multi([lw["wgate"], lw["wup"]], self.xn, [self.gate, self.up])
            if self.fuse_swiglu and self._mm_reduce(lw["wdown"], 1, self.gate, self.up, self.proj):
                pass
            elif self.fuse_swiglu and lw["wdown"].dtype == Q4_K:
                self._mm_fused(1, self.gate, self.up, None, None, None, [lw["wdown"]], [self.proj])
                self._reduce(self.proj)
            else:
                chk(L.sm100_swiglu(s, _dev(self.gate), _dev(self.up), _dev(self.act), self.ffn), "swiglu")
                self._mm(lw["wdown"], self.act, self.proj)
                self._reduce(self.proj)
        # (the next token starts by overwriting self.x with its embedding, so it does not matter where the stream ended)
        chk(L.sm100_rms_norm(s, _dev(x_cur), _dev(self.proj), _dev(self.out_norm), _dev(x_cur), _dev(self.xn), c.hidden, 1, c.eps), "out_norm")
        ctx = getattr(self.allreduce, "ctx", None)
        if self.world > 1 and ctx is not None and self.fuse_exchange:
            # row-sharded head: local arg-max and the exchange of the ranks' (logit, global index) candidates in one kernel
            if self.head is not None:
                self._mm(self.head, self.xn, self.logits)
            chk(L.sm100_argmax_allreduce(ctx, s, _dev(self.logits) if self.head is not None else None, self.vocab_n if self.head is not None else 0,
                                         self.vocab_lo, _dev(self.token)), "argmax_allreduce")
        else:
            if self.head is not None:
                self._mm(self.head, self.xn, self.logits)
                chk(L.sm100_argmax(s, _dev(self.logits), self.vocab_n, _dev(self.best)), "argmax")
            if self.world == 1:
                self.token.copy_(self.best)
            else:
                # (best logit, global index) per rank; highest logit wins, lowest index on ties
                self.cand[0] = self.logits[self.best.long()][0] if self.head is not None else float("-inf")
                self.cand[1] = (self.best + self.vocab_lo).float()[0]
                torch.distributed.all_gather_into_tensor(self.cands.view(-1), self.cand)
                top = self.cands[:, 0].max()
                idx = torch.where(self.cands[:, 0] == top, self.cands[:, 1], torch.full_like(self.cands[:, 1], 3e9)).min()
                self.token.copy_(idx.to(torch.int32).view(1))
        self.tokens_out.index_copy_(0, self.step_index, self.token)
        self.step_index.add_(1)
        self.pos.add_(1)

    # ---- driving --------------------------------------------------------------------------------------
    def reset(self, token: int, prefill_seed: int | None = None):
        c = self.cfg
        with torch.cuda.stream(self.tstream):
            self.token.fill_(token)
            self.pos.fill_(c.start_pos)
            self.step_index.zero_()
            if prefill_seed is not None:
                g = torch.Generator(device="cpu").manual_seed(prefill_seed)
                for i, lw in enumerate(self.layers):
                    for name in ("k_cache", "v_cache"):
                        full = torch.randn(c.kv_heads, c.start_pos, c.head_dim, generator=g)
                        lw[name].zero_()
                        lw[name][:, :c.start_pos] = full[self.rank * self.hkv:(self.rank + 1) * self.hkv].to(self.device)
        torch.cuda.synchronize(self.device)

    def capture(self):
        """Records one step in a CUDA graph (the first eager step also creates the library's attention scratch)."""
        with torch.cuda.stream(self.tstream):
            self.enqueue_step()
        torch.cuda.synchronize(self.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=self.tstream):
            self.enqueue_step()
        torch.cuda.synchronize(self.device)

    def run(self, steps: int):
        with torch.cuda.stream(self.tstream):
            for _ in range(steps):
                if self.graph is not None:
                    self.graph.replay()
                else:
                    self.enqueue_step()

    def tokens(self, n: int) -> np.ndarray:
        torch.cuda.synchronize(self.device)
        return self.tokens_out[:n].cpu().numpy()

    def bytes_per_token(self, pos: int) -> float:
        """Algorithmic bytes one decode step must move on this rank: every weight once, the visible KV cache, the
        embedding row."""
        return float(self.weight_bytes - (self.embed.nbytes if self.embed is not None else 0) + self.kv_bytes_per_pos * (pos + 1) + self.cfg.hidden * 0.5625)
