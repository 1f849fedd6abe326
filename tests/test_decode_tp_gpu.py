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


def test_mul_mat_allreduce(sm100, tmp_path):
    """sm100_mul_mat_allreduce and sm100_argmax_allreduce on 2 GPUs: the K-sharded product with the exchange inside the matvec launch equals the CPU
    oracle's product over the full K (NMSE 1e-6), gives the same bits on both ranks, on repeated calls and under graph
    replay, never runs into its bounded wait; tensors the fused kernel does not serve take the separate launches."""
    if sm100.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = tmp_path / "fused.json"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29737", os.path.join(ROOT, "tests", "fused_exchange_worker.py"), str(out)],
                       capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    got = json.loads(out.read_text())
    assert got["world"] == 2 and got["fault"] == 0, got
    for c in got["cases"]:
        assert c["nmse"] <= 1e-6 and c["repeat_equal"] and c["replay_equal"] and c["ranks_equal"], c
    assert [c["kernel"] for c in got["cases"][:4]] == ["matvec_q4k_ring+allreduce"] * 4, got["cases"]
    assert "ring" not in got["cases"][4]["kernel"]
    assert got["interleaved_worst_nmse"] <= 1e-6, got
    assert got["argmax_ok"], got      # sm100_argmax_allreduce: global arg-max of a row-sharded vector, ties, an empty shard


@pytest.mark.parametrize("exchange", ["nccl", "peer", "peer-unfused"])
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
    if exchange == "peer-unfused":   # the own all-reduce as a launch of its own after the row-parallel projections
        env["SM100_TP_FUSED"] = "0"
        exchange = "peer"
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
