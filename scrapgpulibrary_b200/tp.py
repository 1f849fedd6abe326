"""Tensor-parallel sharding rules of the decode stack (host-side, no CUDA): which slice of each weight a rank owns
and how per-rank results combine.  The reference splits models by layer only (docs/MULTI_GPU.md); sharding weight
rows across GPUs is this backend's addition, so the rules live in one small, CPU-testable place.

  column-parallel (Q, K, V, gate, up, vocabulary head): rank r owns rows [r * n_local, (r + 1) * n_local) of W
      [K, N]; every rank reads the full activation and writes its slice of the output.
  row-parallel (o, down): rank r owns the K-slice [r * k_local, (r + 1) * k_local) of every row (whole quantization
      blocks, so k_local must be a multiple of the block size); each rank produces a full-length partial output and
      the partials are summed (all-reduce).
  greedy token: every rank reports (best logit, global index) of its vocabulary shard; the highest logit wins, the
      lowest index on ties (src/core/ref/ops.cpp:1189-1228 semantics for TOP_K with k = 1).
"""
from __future__ import annotations

import numpy as np

BLOCK = {16: (32, 18), 17: (32, 34), 32: (256, 144), 33: (256, 210)}   # dtype -> (elements, bytes) per block


def shard_rows(natural: np.ndarray, lo: int, n_local: int) -> np.ndarray:
    """Rows [lo, lo + n_local) of a natural-layout matrix [N, row_bytes]."""
    return natural[lo:lo + n_local]


def shard_cols(natural: np.ndarray, dtype: int, k_global: int, rank: int, k_local: int) -> np.ndarray:
    """The K-slice of rank `rank` of every row: whole blocks [rank * k_local / be, (rank + 1) * k_local / be)."""
    be, bb = BLOCK[dtype]
    if k_local % be != 0 or k_global % be != 0:
        raise ValueError("a K shard must consist of whole quantization blocks")
    n = natural.shape[0]
    b0 = rank * k_local // be
    return np.ascontiguousarray(natural.reshape(n, k_global // be, bb)[:, b0:b0 + k_local // be].reshape(n, -1))


def vocab_shard(vocab: int, rank: int, world: int) -> tuple[int, int]:
    """(first row, row count) of the vocabulary head owned by a rank: equal ceil-sized shards, the last may be short."""
    per = -(-vocab // world)
    lo = min(vocab, rank * per)
    return lo, max(0, min(vocab, lo + per) - lo)


def merge_argmax(candidates: np.ndarray) -> int:
    """candidates [world, 2] of (best logit, global index): highest logit, lowest index on ties."""
    c = np.asarray(candidates, dtype=np.float64)
    top = c[:, 0].max()
    return int(c[c[:, 0] == top, 1].min())
