"""Worker of tests/test_decode_tp_gpu.py::test_mul_mat_allreduce: one rank (run under torchrun) of K-sharded products
whose all-reduce happens inside the matvec launch (sm100_mul_mat_allreduce).  Every rank holds the K shard of the same
seeded global matrix; the result is compared with the CPU oracle's product over the full K, with the separate
matvec + sm100_allreduce_sum path, across ranks bit for bit, over several calls in a row and under CUDA-graph replay.
Rank 0 writes a JSON report to argv[1]."""
import ctypes as C
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import sgref  # noqa: E402
from scrapgpulibrary_b200 import capi, tp  # noqa: E402
from scrapgpulibrary_b200.collective import PeerAllReduce  # noqa: E402
from tests import util as U  # noqa: E402

Q4_K, Q6_K = 32, 33


def main():
    out_path = sys.argv[1]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    L = capi.lib()
    capi.check(L.sm100_set_device(local), "set_device")
    ar = PeerAllReduce(rank, world, local, 4096, dist)
    stream = capi.Stream(local)
    report = {"world": world, "cases": []}

    def to_device(array):      # (tests.util's helpers allocate on device 0)
        arr = np.ascontiguousarray(array)
        buf = capi.Buffer(arr.nbytes, local)
        buf.upload(stream, arr)
        return buf

    def guarded_output(count):
        buf = to_device(np.full(count + 2 * U.GUARD, U.CANARY, dtype=np.float32))
        return buf, buf.ptr + 4 * U.GUARD

    # (dtype, K global, N, prologue): benchmark's K-sharded shape, a small one, one with leftover-free odd tile count, a Q6_K one
    # (served by the separate launches), SwiGLU in front of the down projection
    cases = [(Q4_K, 12288, 4096, 0), (Q4_K, 1024, 1024, 0), (Q4_K, 2048, 48, 0), (Q4_K, 4096, 4096, 1), (Q6_K, 2048, 1024, 0)]
    for ci, (dtype, kg, n, prologue) in enumerate(cases):
        kl = kg // world
        wq = U.quantize(dtype, U.seeded_weights(500 + ci, n, kg))
        rng = np.random.default_rng(600 + ci)
        a = rng.standard_normal(kg).astype(np.float32)
        b = rng.standard_normal(kg).astype(np.float32)
        x = sgref.swiglu(a, b) if prologue == 1 else a
        want = sgref.mul_mat(dtype, wq, kg, x.reshape(1, kg)).reshape(n)
        loc = tp.shard_cols(wq, dtype, kg, rank, kl)
        wb = to_device(capi.pack(dtype, kl, loc))
        ab = to_device(a[rank * kl:(rank + 1) * kl])
        bb = to_device(b[rank * kl:(rank + 1) * kl])
        outs = [guarded_output(n) for _ in range(3)]
        stream.sync()
        dist.barrier()

        def call(yptr):
            capi.check(L.sm100_mul_mat_allreduce(ar.ctx, stream.handle, prologue, C.c_void_p(ab.ptr), C.c_void_p(bb.ptr) if prologue else None, dtype, 1,
                                                 C.c_void_p(wb.ptr), kl, n, C.c_void_p(yptr)), "mul_mat_allreduce")

        for _, yptr in outs:       # three calls in a row, no synchronisation in between: both receive buffers in use
            call(yptr)
        kernel = (L.sm100_matvec_last_kernel() or b"").decode()
        stream.sync()
        got = [U.read_guarded(capi, stream, yb, n).copy() for yb, _ in outs]
        # under graph replay
        with capi.Graph(stream) as g:
            call(outs[0][1])
            call(outs[1][1])
        for _ in range(3):
            g.launch()
        stream.sync()
        g.destroy()
        replay = [U.read_guarded(capi, stream, outs[i][0], n).copy() for i in range(2)]
        # every rank holds the same bits
        mine = torch.from_numpy(got[0].view(np.int32).copy()).cuda()
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        same_bits = all(bool(torch.equal(everyone[0], e)) for e in everyone)
        report["cases"].append({
            "dtype": dtype, "k": kg, "n": n, "prologue": prologue, "kernel": kernel,
            "nmse": float(sgref.nmse(got[0].reshape(1, n), want.reshape(1, n))),
            "repeat_equal": bool(all(np.array_equal(got[0], g_) for g_ in got[1:])),
            "replay_equal": bool(all(np.array_equal(got[0], r) for r in replay)),
            "ranks_equal": same_bits})
        for buf in [wb, ab, bb] + [o[0] for o in outs]:
            buf.free()
    # launches of different shapes (different grids, other CTAs owning a row tile) interleaved without synchronisation:
    # a value must never be taken for that of another launch
    shapes = [(1024, 1024), (4096, 2048), (2048, 48)]
    held = []
    for si, (kg, n) in enumerate(shapes):
        kl = kg // world
        wq = U.quantize(Q4_K, U.seeded_weights(700 + si, n, kg))
        x = np.random.default_rng(710 + si).standard_normal(kg).astype(np.float32)
        held.append((kl, n, to_device(capi.pack(Q4_K, kl, tp.shard_cols(wq, Q4_K, kg, rank, kl))), to_device(x[rank * kl:(rank + 1) * kl]),
                     sgref.mul_mat(Q4_K, wq, kg, x.reshape(1, kg)).reshape(n), [guarded_output(n) for _ in range(4)]))
    stream.sync()
    dist.barrier()
    for rep in range(4):
        for kl, n, wb, xb, want, outs in held:
            capi.check(L.sm100_mul_mat_allreduce(ar.ctx, stream.handle, 0, C.c_void_p(xb.ptr), None, Q4_K, 1, C.c_void_p(wb.ptr), kl, n,
                                                 C.c_void_p(outs[rep][1])), "mul_mat_allreduce")
    stream.sync()
    worst = 0.0
    for kl, n, wb, xb, want, outs in held:
        for yb, _ in outs:
            worst = max(worst, float(sgref.nmse(U.read_guarded(capi, stream, yb, n).reshape(1, n), want.reshape(1, n))))
    report["interleaved_worst_nmse"] = worst
    # greedy token over a row-sharded head: the global arg-max, lowest index on ties (also across ranks), an empty shard
    L.sm100_argmax_allreduce.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
    rngm = np.random.default_rng(900)
    total = 4099
    ok_argmax = True
    for trial in range(6):
        row = rngm.standard_normal(total).astype(np.float32)
        if trial == 1:                      # the same maximum on both ranks: the lower global index wins
            row[[7, 3000]] = 9.0
        if trial == 2:
            row[[3000, 3500]] = 9.0
        per = -(-total // world) if trial != 3 else total      # trial 3: everything on rank 0, the others hold no rows
        lo = min(total, rank * per)
        n_loc = max(0, min(total, lo + per) - lo)
        xb_ = to_device(row[lo:lo + n_loc]) if n_loc else None
        ob_ = to_device(np.full(1, -1, np.int32))
        capi.check(L.sm100_argmax_allreduce(ar.ctx, stream.handle, C.c_void_p(xb_.ptr) if xb_ else None, n_loc, lo, C.c_void_p(ob_.ptr)), "argmax_allreduce")
        stream.sync()
        got_tok = int(ob_.download(stream, np.int32, 1)[0])
        want_tok = int(np.flatnonzero(row == row.max())[0])
        ok_argmax = ok_argmax and got_tok == want_tok
    report["argmax_ok"] = bool(ok_argmax)
    report["fault"] = ar.fault()
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(report, f)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
