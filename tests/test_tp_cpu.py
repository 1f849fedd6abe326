"""Tensor-parallel sharding rules on CPU ranks (gloo, world size 2): each rank runs the CPU oracle on its shard of
seeded quantized weights, partial results meet through real collectives, and the combination must equal the
unsharded oracle -- column-parallel slices gathered, row-parallel partials all-reduced (NMSE <= 1e-6: the f32 sum
order differs from the single-device order), greedy token merged from per-rank (logit, index) pairs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import sgref
from scrapgpulibrary_b200 import tp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)          # every rank builds the same global tensors
        k, n, ffn, vocab = 512, 96, 1024, 1000
        x = rng.standard_normal((1, k)).astype(np.float32)
        for dtype in (32, 33):
            w_col = sgref.quantize(dtype, (rng.standard_normal((n, k)) * 0.05).astype(np.float32))
            w_row = sgref.quantize(dtype, (rng.standard_normal((k, ffn)) * 0.05).astype(np.float32))     # [N = k, K = ffn]
            act = rng.standard_normal((1, ffn)).astype(np.float32)
            # column-parallel: my rows, gathered
            n_local = n // world
            mine = sgref.mul_mat(dtype, tp.shard_rows(w_col, rank * n_local, n_local), k, x, threads=1)[0]
            parts = [torch.zeros(n_local) for _ in range(world)]
            dist.all_gather(parts, torch.from_numpy(mine))
            full = torch.cat(parts).numpy()
            want = sgref.mul_mat(dtype, w_col, k, x, threads=1)[0]
            assert np.array_equal(full, want), "column-parallel slices must reproduce the unsharded rows exactly"
            # row-parallel: my K slice, all-reduced
            k_local = ffn // world
            partial = sgref.mul_mat(dtype, tp.shard_cols(w_row, dtype, ffn, rank, k_local), k_local,
                                    np.ascontiguousarray(act[:, rank * k_local:(rank + 1) * k_local]), threads=1)[0]
            t = torch.from_numpy(partial.copy())
            dist.all_reduce(t)
            want = sgref.mul_mat(dtype, w_row, ffn, act, threads=1)[0]
            assert sgref.nmse(t.numpy(), want) <= 1e-6
        # greedy token over a sharded vocabulary, with a tie across ranks
        logits = rng.standard_normal(vocab).astype(np.float32)
        logits[17] = logits[777] = 9.5
        lo, cnt = tp.vocab_shard(vocab, rank, world)
        best = sgref.argmax(logits[lo:lo + cnt])
        cand = torch.tensor([float(logits[lo + best]), float(lo + best)], dtype=torch.float64)
        cands = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(cands, cand)
        assert tp.merge_argmax(torch.stack(cands).numpy()) == sgref.argmax(logits) == 17
        with open(os.path.join(out_dir, f"ok{rank}"), "w") as f:
            f.write("ok")
    finally:
        dist.destroy_process_group()


def test_tp_sharding_rules_with_gloo_ranks(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_shard_helpers():
    assert tp.vocab_shard(151936, 7, 8) == (7 * 18992, 18992)
    assert tp.vocab_shard(10, 3, 4) == (9, 1) and tp.vocab_shard(10, 2, 8) == (4, 2)
    assert tp.merge_argmax(np.array([[1.0, 5], [3.0, 9], [3.0, 2]])) == 2
    nat = np.arange(4 * 2 * 144, dtype=np.uint8).reshape(4, 288) if False else np.zeros((4, 288), np.uint8)
    assert tp.shard_cols(nat, 32, 512, 1, 256).shape == (4, 144)
    with pytest.raises(ValueError):
        tp.shard_cols(nat, 32, 512, 0, 100)
