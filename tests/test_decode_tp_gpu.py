"""Tensor-parallel decode on 2 GPUs (one process per GPU; all-reduce by NCCL, or by the library's own one-shot kernel
over peer-mapped memory): greedy tokens identical to the CPU oracle's and to
the single-GPU run, eager and under CUDA-graph replay.  Needs two GPUs; on a single-GPU box the test is skipped."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from oracle import decode_ref

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("exchange", ["nccl", "peer"])
def test_tp2_decode_tokens_match_oracle(sm100, tmp_path, exchange):
    if sm100.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from scrapgpulibrary_b200.decode import DecodeConfig
    steps = 8
    cfg = DecodeConfig(layers=3, hidden=1024, heads=8, kv_heads=2, head_dim=128, ffn=2048, vocab=4096, n_ctx=64, start_pos=8)
    weights = decode_ref.random_weights(cfg, 7)
    rng = np.random.default_rng(11)
    kp = [rng.standard_normal((cfg.kv_heads, cfg.start_pos, cfg.head_dim)).astype(np.float32) for _ in range(cfg.layers)]
    vp = [rng.standard_normal((cfg.kv_heads, cfg.start_pos, cfg.head_dim)).astype(np.float32) for _ in range(cfg.layers)]
    want, _ = decode_ref.decode_reference(cfg, weights, 123, steps, kp, vp)
    out = tmp_path / "tokens.json"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29731" if exchange == "nccl" else "29733", os.path.join(ROOT, "tests", "tp_decode_worker.py"), str(out), str(steps), exchange],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    got = json.loads(out.read_text())
    assert got["world"] == 2 and got["fault"] == 0
    assert got["eager"] == want.tolist()
    assert got["replay"] == want.tolist()


def test_tp2_full_shape_tokens_match_oracle(sm100, tmp_path):
    """The benchmark's full decode configuration split over 2 GPUs (own peer all-reduce): the same greedy tokens as
    the CPU oracle's committed list, i.e. as the single-GPU run of test_decode_gpu.py -- one global model, sharded."""
    if sm100.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    gold = json.load(open(os.path.join(ROOT, "tests", "golden", "decode_qwen3_8b_shape.json")))
    steps = len(gold["tokens"])
    out = tmp_path / "tokens_full.json"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29735", os.path.join(ROOT, "tests", "tp_decode_worker.py"), str(out), str(steps), "peer", "full"],
                       capture_output=True, text=True, timeout=1200, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    got = json.loads(out.read_text())
    assert got["world"] == 2 and got["fault"] == 0
    assert got["eager"] == gold["tokens"]
    assert got["replay"] == gold["tokens"]
