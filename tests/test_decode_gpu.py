"""Layer-stack decode on the GPU against the CPU oracle: identical greedy tokens (the north star's bar for the
decode stack) and logits within NMSE 1e-6, on a reduced Qwen3-shaped configuration the oracle finishes in
seconds; eager launches and CUDA-graph replay must agree token for token."""
import numpy as np
import pytest

from oracle import decode_ref, sgref

pytestmark = pytest.mark.gpu


def small_cfg():
    from scrapgpulibrary_b200.decode import DecodeConfig
    return DecodeConfig(layers=3, hidden=1024, heads=8, kv_heads=2, head_dim=128, ffn=2048, vocab=4096, n_ctx=64, start_pos=8)


def test_decode_matches_oracle_tokens_and_logits(sm100):
    import torch
    from scrapgpulibrary_b200.decode import DecodeModel
    cfg = small_cfg()
    weights = decode_ref.random_weights(cfg, 7)
    rng = np.random.default_rng(11)
    kp = [rng.standard_normal((cfg.kv_heads, cfg.start_pos, cfg.head_dim)).astype(np.float32) for _ in range(cfg.layers)]
    vp = [rng.standard_normal((cfg.kv_heads, cfg.start_pos, cfg.head_dim)).astype(np.float32) for _ in range(cfg.layers)]
    steps = 10
    want_tokens, want_logits = decode_ref.decode_reference(cfg, weights, 123, steps, kp, vp)

    model = DecodeModel(cfg, weights=weights)

    def load_prefill():
        model.reset(123)
        for i, lw in enumerate(model.layers):
            lw["k_cache"].zero_()
            lw["v_cache"].zero_()
            lw["k_cache"][:, :cfg.start_pos] = torch.from_numpy(kp[i]).to(model.device)
            lw["v_cache"][:, :cfg.start_pos] = torch.from_numpy(vp[i]).to(model.device)
        torch.cuda.synchronize()

    load_prefill()
    model.run(steps)
    eager = model.tokens(steps)
    logits = model.logits.cpu().numpy()
    assert np.array_equal(eager, want_tokens)
    assert sgref.nmse(logits, want_logits) <= 1e-6

    model.capture()
    load_prefill()
    model.run(steps)
    assert np.array_equal(model.tokens(steps), want_tokens)


def test_full_shape_decode_tokens_match_oracle(sm100):
    """The benchmark's decode configuration at full shape (36 layers, hidden 4096, 32 / 8 heads of 128, FFN 12288,
    vocabulary 151936, KV cache pre-filled to 1024): the first greedy tokens of the GPU stack, eager and under graph
    replay, equal the CPU oracle's on the same rank-independent synthetic model.  The oracle's tokens are the
    committed list tests/golden/decode_qwen3_8b_shape.json (generator: tests/golden/make_decode_golden.py; one token
    costs the oracle seconds on all host cores)."""
    import json
    import os
    from scrapgpulibrary_b200.decode import DecodeConfig, DecodeModel
    gold = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "decode_qwen3_8b_shape.json")))
    want = gold["tokens"]
    assert len(want) >= 4
    model = DecodeModel(DecodeConfig(), seed=gold["seed"])
    model.reset(token=gold["first_token"], prefill_seed=gold["prefill_seed"])
    model.run(len(want))
    assert model.tokens(len(want)).tolist() == want
    model.reset(token=gold["first_token"], prefill_seed=gold["prefill_seed"])
    model.capture()     # runs one eager token, then records the step
    model.reset(token=gold["first_token"], prefill_seed=gold["prefill_seed"])
    model.run(len(want))
    assert model.tokens(len(want)).tolist() == want
