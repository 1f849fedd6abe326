"""Worker of tests/test_decode_tp_gpu.py: one tensor-parallel rank of the decode stack (run under torchrun).
Rank 0 writes the greedy tokens it produced (eager and graph replay) to the path given as argv[1].
argv: out_path steps exchange(nccl|peer) [config: small|full]; "full" is the benchmark's Qwen3-8B-shaped stack on the
rank-independent synthetic model, first token and KV prefill as in tests/golden/decode_qwen3_8b_shape.json."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import decode_ref  # noqa: E402
from scrapgpulibrary_b200.decode import DecodeConfig, DecodeModel  # noqa: E402


def main():
    out_path, steps = sys.argv[1], int(sys.argv[2])
    exchange = sys.argv[3] if len(sys.argv) > 3 else "nccl"
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    full = len(sys.argv) > 4 and sys.argv[4] == "full"
    if full:
        return run_full(out_path, steps, exchange, rank, world, local)
    cfg = DecodeConfig(layers=3, hidden=1024, heads=8, kv_heads=2, head_dim=128, ffn=2048, vocab=4096, n_ctx=64, start_pos=8)
    weights = decode_ref.random_weights(cfg, 7)      # the same global weights on every rank, sharded by the model
    rng = np.random.default_rng(11)
    kp = [rng.standard_normal((cfg.kv_heads, cfg.start_pos, cfg.head_dim)).astype(np.float32) for _ in range(cfg.layers)]
    vp = [rng.standard_normal((cfg.kv_heads, cfg.start_pos, cfg.head_dim)).astype(np.float32) for _ in range(cfg.layers)]
    allreduce = None
    if exchange == "peer":   # the library's one-shot all-reduce over peer-mapped memory instead of NCCL
        from scrapgpulibrary_b200.collective import PeerAllReduce
        allreduce = PeerAllReduce(rank, world, local, cfg.hidden, dist)
    model = DecodeModel(cfg, rank=rank, world=world, device_index=local, weights=weights, allreduce=allreduce)

    def load_prefill():
        model.reset(123)
        lo, hi = rank * model.hkv, (rank + 1) * model.hkv
        for i, lw in enumerate(model.layers):
            lw["k_cache"].zero_()
            lw["v_cache"].zero_()
            lw["k_cache"][:, :cfg.start_pos] = torch.from_numpy(kp[i][lo:hi]).to(model.device)
            lw["v_cache"][:, :cfg.start_pos] = torch.from_numpy(vp[i][lo:hi]).to(model.device)
        torch.cuda.synchronize()

    load_prefill()
    model.run(steps)
    eager = model.tokens(steps).tolist()
    model.capture()
    load_prefill()
    model.run(steps)
    replay = model.tokens(steps).tolist()
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump({"eager": eager, "replay": replay, "world": world, "fault": allreduce.fault() if allreduce is not None else 0}, f)
    dist.barrier()
    torch.cuda.synchronize()
    # no destroy_process_group(): it was seen to block for minutes here while captured graphs hold the communicator
    sys.stdout.flush()
    os._exit(0)


def run_full(out_path, steps, exchange, rank, world, local):
    gold = json.load(open(os.path.join(ROOT, "tests", "golden", "decode_qwen3_8b_shape.json")))
    cfg = DecodeConfig()
    allreduce = None
    if exchange == "peer":
        from scrapgpulibrary_b200.collective import PeerAllReduce
        allreduce = PeerAllReduce(rank, world, local, cfg.hidden, dist)
    model = DecodeModel(cfg, rank=rank, world=world, device_index=local, seed=gold["seed"], allreduce=allreduce)
    model.reset(token=gold["first_token"], prefill_seed=gold["prefill_seed"])
    model.run(steps)
    eager = model.tokens(steps).tolist()
    model.reset(token=gold["first_token"], prefill_seed=gold["prefill_seed"])
    model.capture()
    model.reset(token=gold["first_token"], prefill_seed=gold["prefill_seed"])
    model.run(steps)
    replay = model.tokens(steps).tolist()
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump({"eager": eager, "replay": replay, "world": world, "fault": allreduce.fault() if allreduce is not None else 0}, f)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
