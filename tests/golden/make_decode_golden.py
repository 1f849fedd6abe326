"""Generates tests/golden/decode_qwen3_8b_shape.json: the greedy tokens of the CPU oracle (oracle/decode_ref.py, the
reference's op list restated on oracle/sgref.c) for the benchmark's decode configuration at FULL shape -- 36 layers,
hidden 4096, 32 query / 8 KV heads of 128, FFN 12288, vocabulary 151936, f32 KV cache pre-filled to position 1024 --
on the rank-independent synthetic model scrapgpulibrary_b200.decode.SyntheticWeights(cfg, seed).

    python tests/golden/make_decode_golden.py [steps]

One token takes the oracle several seconds on all host cores (5.6 GB of quantized weights per token), which is why
the GPU tests and the benchmark compare with this committed list instead of running the oracle on the GPU box.
The KV prefill is the one DecodeModel.reset(token, prefill_seed) draws (torch CPU generator)."""
import json
import os
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import decode_ref  # noqa: E402
from scrapgpulibrary_b200.decode import DecodeConfig, SyntheticWeights  # noqa: E402

SEED, FIRST_TOKEN, PREFILL_SEED = 0x5CA9, 1234, 7


class Cached:
    """Materialises each global matrix once (5.6 GB of host memory for the full model)."""

    def __init__(self, sw):
        self.sw, self.cache = sw, {}

    def __getitem__(self, name):
        if name not in self.cache:
            self.cache[name] = self.sw[name]
        return self.cache[name]


def prefill(cfg):
    g = torch.Generator(device="cpu").manual_seed(PREFILL_SEED)
    kp, vp = [], []
    for _ in range(cfg.layers):
        kp.append(torch.randn(cfg.kv_heads, cfg.start_pos, cfg.head_dim, generator=g).numpy())
        vp.append(torch.randn(cfg.kv_heads, cfg.start_pos, cfg.head_dim, generator=g).numpy())
    return kp, vp


def main():
    steps = int(sys.argv[1]) if len(sys.argv) > 1 else 6
    cfg = DecodeConfig()
    weights = Cached(SyntheticWeights(cfg, SEED))
    kp, vp = prefill(cfg)
    t0 = time.time()
    tokens, logits = decode_ref.decode_reference(cfg, weights, FIRST_TOKEN, steps, kp, vp, threads=os.cpu_count())
    order = np.argsort(-logits)[:4]
    out = {"config": "DecodeConfig() defaults (Qwen3-8B shape)", "seed": SEED, "first_token": FIRST_TOKEN, "prefill_seed": PREFILL_SEED,
           "steps": steps, "tokens": [int(t) for t in tokens],
           "last_step_top4": [[int(i), float(logits[i])] for i in order],
           "oracle_seconds": round(time.time() - t0, 1)}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "decode_qwen3_8b_shape.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print(out)


if __name__ == "__main__":
    main()
