#!/usr/bin/env python
"""Benchmark of the cuda_sm100 hot path: the Q4_K decode matvec over Qwen3-8B-shaped projections.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the M = 1 matvec over a pool of distinct packed Q4_K weight matrices:
`layers` x {K=4096 N=4096, K=4096 N=12288, K=12288 N=4096} (Qwen3-8B's q/o, gate/up and down projection
shapes; 36 layers = 2.4 GB, far above the 126 MB L2, so every step streams its weights from HBM).
metric = algorithmic GB/s = sum over launches of (N*K*0.5625 + 4*K + 4*N) bytes / device time.

  value      launches replayed from one CUDA graph, inputs resident in HBM, CUDA-event timing on the
             launching stream
  e2e        the same pass through the backend plugin's vtable (what scrapgpu_buffer_write / scrapgpu_plan_execute /
             scrapgpu_buffer_read / scrapgpu_stream_sync of the reference's C API forward to) with HOST activations:
             per step one non-blocking write of the arena that holds every matvec's x from pinned host memory, one
             plan_execute of the step's MUL_MAT nodes, one non-blocking read of the results arena into pinned host
             memory, one sync (weights stay
             resident, as they do after scrapgpu_tensor_upload in the reference's usage); timed on the host clock
             around steps that each end in a sync
  roofline   achieved = algorithmic bytes per launch / mean launch duration (the same CUDA-event region),
             peak = measured HBM copy bandwidth of MEASURED_PEAKS.json (burst figure; fallback 6650 GB/s)
  cpu_baseline  the unmodified reference's CPU MUL_MAT (oracle/_ref, built from the reference's own sources) on
             one layer's three matrices, single thread (the reference is single-threaded)

`--impl reference` times that CPU reference with all host threads (rows sharded over threads, each slice an
unmodified scrapgpu_ref_execute call) on a bounded sample of the same workload.

With N > 1 ranks (torchrun) the SAME sweep is split over the ranks the way a tensor-parallel model splits its
projections: the q/o-shaped and the gate/up-shaped matrices by weight rows (N / P rows per rank, the whole activation
column, no collective), the down-shaped matrix by K (K / P columns of every row per rank) followed by an all-reduce of
the 4096-float partial results (the library's one-shot all-reduce over peer-mapped memory).  value = algorithmic
bytes of the whole (unsplit) sweep / max-over-ranks device time: strong scaling.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

Q4_0, Q8_0, Q4_K, Q6_K = 16, 17, 32, 33
BPW = {Q4_0: 0.5625, Q8_0: 1.0625, Q4_K: 0.5625, Q6_K: 0.8203125}
SHAPES = [(4096, 4096), (4096, 12288), (12288, 4096)]  # (K, N)
METRIC = "q4_k_matvec_algorithmic_gbps"
# what the timed kernel computes in (not a precision claim: results are within NMSE 1e-6 of the f32 reference, measured ~5e-9)
ARITHMETIC = "u8 weights x s16 activations (two s8 planes, one f32 scale per 32) -> s32 on mma.sync; f32 block scales and accumulation"


def algorithmic_bytes(dtype: int, k: int, n: int, m: int = 1) -> float:
    """Bytes a MUL_MAT must move: packed weights once, activations in, results out."""
    return n * k * BPW[dtype] + 4.0 * k * m + 4.0 * n * m


# the all-reduce of a K-sharded product inside the matvec launch (sm100_mul_mat_allreduce); 0: matvec, then sm100_allreduce_sum
FUSED_EXCHANGE = os.environ.get("SM100_TP_FUSED", "1") != "0"


def profiled_traffic(kernel_prefix: str):
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel from the ncu capture
    summarised under profiles/: profiles/roofline_traffic.json names the kernel it was taken from, so a figure that
    belongs to another kernel is not reported."""
    p = os.path.join(ROOT, "profiles", "roofline_traffic.json")
    try:
        rec = json.load(open(p))
        if str(rec.get("kernel", "")).startswith(kernel_prefix):
            return int(rec["dram_bytes_per_launch"]), rec.get("source")
    except Exception:
        pass
    return None, None


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, a B200 HBM3e copy bandwidth measured earlier; MEASURED_PEAKS.json absent)"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, device: int):
        self.device = device
        self.rows = []
        self.proc = None

    def start(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device}", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()
        # nvidia-smi needs a moment to attach: wait for its first sample so that the timed region is covered
        t0 = time.time()
        while not self.rows and time.time() - t0 < 5.0:
            time.sleep(0.02)
        self.rows.clear()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


SPLIT = ("rows", "rows", "k")   # how each sweep shape is split over tensor-parallel ranks (q/o-shaped, gate/up-shaped, down-shaped)


def build_pool(capi, stream, dtype: int, layers: int, seed: int, rank: int = 0, world: int = 1):
    """Packed weights on the device: `layers` distinct matrices per shape.  One matrix per shape is synthesised
    on the host; the others are row rotations of it (distinct HBM addresses, same value distribution),
    repacked on the device from the natural bytes.  With world > 1 every rank keeps its shard of every matrix
    (SPLIT): the same global matrices on every rank (the seed does not depend on the rank)."""
    from scrapgpulibrary_b200 import synth, tp
    pool = []
    L = capi.lib()
    for si, (k, n) in enumerate(SHAPES):
        base = synth.quantized_matrix(dtype, seed + si, n, k)
        kl, nl = (k, n // world) if SPLIT[si] == "rows" else (k // world, n)
        assert nl % 16 == 0 and kl % 256 == 0, "the sweep shapes split evenly over 1, 2, 4 and 8 ranks"
        staging = None
        mats = []
        for layer in range(layers):
            rot = np.roll(base, layer * 17, axis=0) if layer else base
            if world > 1:
                rot = tp.shard_rows(rot, rank * nl, nl) if SPLIT[si] == "rows" else tp.shard_cols(rot, dtype, k, rank, kl)
            rot = np.ascontiguousarray(rot)
            if staging is None:
                staging = capi.Buffer(rot.nbytes)
            staging.upload(stream, rot)
            dst = capi.Buffer(rot.nbytes)
            capi.check(L.sm100_pack_device(stream.handle, dtype, kl, nl, staging.at(), dst.at()), "pack_device")
            stream.sync()
            mats.append(dst)
        staging.free()
        pool.append({"k": kl, "n": nl, "k_full": k, "n_full": n, "mats": mats, "natural": base, "split": SPLIT[si] if world > 1 else None})
    return pool


def run_ours(args, rank: int, world: int, local_rank: int):
    from scrapgpulibrary_b200 import _build, capi
    _build.build_sm100()
    capi.require_device()
    L = capi.lib()
    capi.set_default_device(local_rank)
    stream = capi.Stream(local_rank)
    if args.no_pdl:
        L.sm100_set_pdl(0)
    if args.gemm_only:
        print(json.dumps({"gemm_only": True, **prefill_gemm(capi, stream, reps=5)}), flush=True)
        return None
    if args.decode_only:
        # profiler runs of the layer-stack decode alone (single GPU): a few tokens, one line
        d = run_decode(args, rank, world, local_rank, None, stream_sync=stream.sync)
        print(json.dumps({"decode_only": True, **d}), flush=True)
        return None
    dtype = Q4_K
    layers = args.layers
    dist, allreduce = None, None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        torch.cuda.set_device(local_rank)
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod
        from scrapgpulibrary_b200.collective import PeerAllReduce
        allreduce = PeerAllReduce(rank, world, local_rank, 4096 * 8, dist)   # rendezvous over torch.distributed, exchange by the library's own kernel
    t0 = time.time()
    pool = build_pool(capi, stream, dtype, layers, seed=0x5CA9, rank=rank, world=world)
    setup_s = time.time() - t0

    rng = np.random.default_rng(1234)
    xs, ys = {}, {}
    for k in sorted({p["k"] for p in pool} | {4096, 12288}):
        xs[k] = capi.Buffer(4 * k * 8)
        xs[k].upload(stream, rng.standard_normal(k * 8).astype(np.float32))
    for n in sorted({p["n"] for p in pool} | {4096, 12288}):
        ys[n] = capi.Buffer(4 * n * 8)

    # launch order of one step: layer by layer, q/o-shaped, gate/up-shaped, down-shaped
    order = [(s, layer) for layer in range(layers) for s in range(len(SHAPES))]
    # algorithmic bytes of the WHOLE sweep (all ranks together move every weight byte once)
    step_bytes = sum(algorithmic_bytes(dtype, pool[s]["k_full"], pool[s]["n_full"]) for s, _ in order)

    def enqueue_step(m: int = 1, only_shape=None):
        cnt = 0
        for s, layer in order:
            if only_shape is not None and s != only_shape:
                continue
            p = pool[s]
            if p["split"] == "k" and m == 1 and FUSED_EXCHANGE:
                # the K shards' partial sums are exchanged and added inside the matvec launch
                capi.check(L.sm100_mul_mat_allreduce(allreduce.ctx, stream.handle, 0, C.c_void_p(xs[p["k"]].ptr), None, dtype, 1, C.c_void_p(p["mats"][layer].ptr),
                                                     p["k"], p["n"], C.c_void_p(ys[p["n"]].ptr)), "mul_mat_allreduce")
                cnt += 1
                continue
            capi.mul_mat(stream, dtype, 1, p["mats"][layer], p["k"], p["n"], xs[p["k"]], m, ys[p["n"]])
            if p["split"] == "k":   # partial sums of the K shards -> the full result on every rank
                capi.check(L.sm100_allreduce_sum(allreduce.ctx, stream.handle, C.c_void_p(ys[p["n"]].ptr), p["n"] * m), "allreduce_sum")
            cnt += 1
        return cnt

    def timed_graph(m: int, only_shape, steps: int, warmup: int):
        if m > 2:   # the multi-column path keeps quantized activations in library scratch: create it outside the capture
            enqueue_step(m, only_shape if only_shape is not None else 0)
            stream.sync()
        launches0 = L.sm100_launch_count()
        with capi.Graph(stream) as g:
            matvecs = enqueue_step(m, only_shape)
        per_step = int(L.sm100_launch_count() - launches0)   # kernels of this library captured for one step
        assert per_step >= matvecs
        for _ in range(warmup):
            g.launch()
        stream.sync()
        e0, e1 = capi.Event(), capi.Event()
        e0.record(stream)
        for _ in range(steps):
            g.launch()
        e1.record(stream)
        e1.sync()
        ms = e0.elapsed_ms(e1)
        g.destroy()
        return ms, per_step, matvecs

    # ---- headline: whole sweep, M = 1, graph replay ----
    def barrier():
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()
        stream.sync()

    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()
    ms, per_step, matvecs_per_step = timed_graph(1, None, args.steps, args.warmup)
    headline_kernel = (L.sm100_matvec_last_kernel() or b"").decode()   # the kernel family that served the timed launches
    barrier()
    clocks = sampler.stop() if rank == 0 else {}
    if dist is not None:
        import torch
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    value = step_bytes / (ms_per_step * 1e-3) / 1e9
    launches_timed = per_step * args.steps

    # ---- the other half of the metric: Qwen3-8B-shaped decode tok/s, tensor-parallel over all ranks ----
    decode = None
    if not args.no_decode and not args.quick:
        try:
            decode = run_decode(args, rank, world, local_rank, dist, stream_sync=stream.sync)
        except Exception as e:  # the headline line must survive a failure of the secondary measurement
            decode = {"error": f"{type(e).__name__}: {e}"[:300]}

    # ---- the vocabulary head sharded by rows over the ranks, logits all-gathered (N > 1) ----
    head = None
    if dist is not None and not args.quick:
        try:
            head = sharded_head(capi, rank, world, local_rank, dist, allreduce)
        except Exception as e:
            head = {"error": f"{type(e).__name__}: {e}"[:300]}

    out = None
    if args.quick:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": round(value, 1), "unit": "GB/s", "quick": True, "n_gpus": world, "ms_per_step": round(ms_per_step, 4),
                              "launches_per_step": per_step}), flush=True)
        return None
    detail, cpu = {}, None
    if world == 1:
        h2d = sum(4 * pool[s]["k"] for s, _ in order)
        d2h = sum(4 * pool[s]["n"] for s, _ in order)
    else:   # one buffer per distinct K and per distinct N goes up / comes back per step and rank
        h2d = world * sum(4 * k for k in {pool[s]["k"] for s, _ in order})
        d2h = world * sum(4 * n for n in {pool[s]["n"] for s, _ in order})
    if world > 1:
        # every rank takes part (the K-split shape ends in an all-reduce): host activations in, host results out through the C ABI
        e2e = e2e_sharded(capi, stream, pool, order, enqueue_step, xs, ys, dist, max(3, args.warmup), max(3, args.steps // 2))
    if rank == 0 and world == 1:
        # per-shape and per-M figures (explanatory; the same graph-replay protocol, fewer steps)
        sub_steps = max(3, args.steps // 2)
        for s, (k, n) in enumerate(SHAPES):
            m_ms, _, cnt = timed_graph(1, s, sub_steps, 3)
            detail[f"q4_k_k{k}_n{n}_m1_gbps"] = round(cnt * algorithmic_bytes(dtype, k, n) * sub_steps / (m_ms * 1e-3) / 1e9, 1)
        for m in (2, 4, 8):
            m_ms, _, cnt = timed_graph(m, None, sub_steps, 3)
            b = sum(algorithmic_bytes(dtype, pool[s]["k"], pool[s]["n"], m) for s, _ in order)
            detail[f"q4_k_sweep_m{m}_gbps"] = round(b * sub_steps / (m_ms * 1e-3) / 1e9, 1)

        # ---- the other decode formats: Q6_K over the same shapes and batches, the Q4_0 case, the Q6_K vocabulary head ----
        detail.update(other_formats(capi, stream))

        # ---- prefill GEMM (tensor cores): Q8_0, M = 512 tokens, K = 4096, N in {4096, 12288} ----
        detail.update(prefill_gemm(capi, stream))

        # ---- e2e: host activations in, host results out, through the backend plugin's vtable ----
        e2e = e2e_through_plugin(capi, stream, pool, order, dtype, local_rank, rng, max(3, args.warmup), max(3, args.steps // 2))

        cpu = cpu_baseline(pool, threads=1, repeats=5)
    if rank == 0:
        peak, peak_src = measured_peak_gbs()
        per_launch_bytes = step_bytes / world / matvecs_per_step          # per GPU and matvec launch
        per_launch_us = ms_per_step * 1e3 / matvecs_per_step               # (at N > 1 this includes the all-reduce launches in between)
        achieved = per_launch_bytes / (per_launch_us * 1e-6) / 1e9
        kernel_name = (L.sm100_matvec_last_kernel() or b"").decode() if headline_kernel is None else headline_kernel
        # (the capture is of the unsharded launches: it says nothing about a rank's share)
        traffic, traffic_src = profiled_traffic(kernel_name) if world == 1 else (None, None)
        out = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": ARITHMETIC,
            "data": "synthetic: seeded N(0, 0.02) weights in Q4_K blocks, N(0, 1) activations",
            "config": {"workload": f"Q4_K matvec sweep, M=1, Qwen3-8B projection shapes (K,N) in {SHAPES} x {layers} layers"
                                   + ("" if world == 1 else f", split over {world} GPUs: (K,N) {SHAPES[0]} and {SHAPES[1]} by weight rows, {SHAPES[2]} by K with an "
                                      "all-reduce of the 4096-float partial results over peer-mapped memory ("
                                      + ("inside the matvec launch" if FUSED_EXCHANGE else "own one-shot kernel after the matvec") + ")"),
                       "launches_per_step": per_step, "matvecs_per_step": matvecs_per_step, "bytes_per_step": int(step_bytes), "bytes_per_step_per_gpu": int(step_bytes / world),
                       "weights_layout": "backend-packed planes", "all_reduce_fault": allreduce.fault() if allreduce is not None else 0,
                       "l2": "inputs larger than L2 (pool %.2f GB per GPU, L2 126 MB)" % (step_bytes / world / 1e9), "timing": "CUDA events on the launching stream, one graph replay per step",
                       "setup_s": round(setup_s, 1), "detail": detail, "decode": decode, "head_sharded": head},
            "gpu_launches": int(launches_timed),
            "e2e": {"value": round(step_bytes / (e2e["ms_per_step"] * 1e-3) / 1e9, 1), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": round(e2e["ms_per_step"], 4), "note": e2e["note"]} if world > 1 else
                   {"value": round(step_bytes / (e2e["ms_per_step"] * 1e-3) / 1e9, 1), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": round(e2e["ms_per_step"], 4), "form": e2e["form"], "one_stream_ms_per_step": round(e2e["one_stream_ms_per_step"], 4),
                    "pipelined_value": round(step_bytes / (e2e["pipelined_ms_per_step"] * 1e-3) / 1e9, 1),
                    "pipelined_ms_per_step": round(e2e["pipelined_ms_per_step"], 4), "pipe_chunks": e2e["pipe_chunks"], "pipe_streams": e2e["pipe_streams"],
                    "per_op_ms_per_step": round(e2e["per_op_ms_per_step"], 4),
                    "per_op_value": round(step_bytes / (e2e["per_op_ms_per_step"] * 1e-3) / 1e9, 1), "results_checked": e2e["checked"],
                    "note": "through the cuda_sm100 backend vtable (the calls behind scrapgpu_buffer_write / scrapgpu_plan_execute / scrapgpu_buffer_read / "
                            "scrapgpu_stream_sync), host time around steps that each end with stream_sync; weights resident (uploaded once with "
                            "tensor_upload, packed layout); every step moves its activations up from pinned host memory and its results down.  "
                            "one stream: ONE non-blocking buffer_write of the activation arena, one plan_execute of the 108 MUL_MAT nodes, ONE "
                            "non-blocking buffer_read of the results arena.  pipelined: the same step as %d plans of %d nodes over %d streams of the "
                            "device, each with its own buffer_write and buffer_read, so copies of one stream overlap kernels of the others and the "
                            "streams' launch chains overlap each other.  That schedule is only possible because the products of the sweep do not "
                            "depend on each other (a decode step's do), and its chunk and stream counts are the best of the combinations tried, so "
                            "it is reported beside the headline as pipelined_*: value is the ONE-STREAM form.  per_op_*: one buffer_write, one "
                            "op_execute and one buffer_read per matvec (324 vtable calls and 216 small copies per step)" % (e2e["pipe_chunks"], 108 // e2e["pipe_chunks"], e2e["pipe_streams"])},
            "roofline": {"bound": "hbm", "kernel": kernel_name, "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "peak_source": peak_src, "bytes_per_launch": round(per_launch_bytes, 1),
                         "us_per_launch": round(per_launch_us, 3),
                         # dram__bytes_read + write per launch, mean over the three shapes of one ncu capture of this kernel
                         "traffic": traffic, "traffic_source": traffic_src},
            "cpu_baseline": cpu,
            "clocks": clocks,
        }
    if dist is not None:
        dist.barrier()
    return out


def e2e_through_plugin(capi, stream, pool, order, dtype, device_index, rng, warmup, steps):
    """The sweep as a caller of the reference library drives it: device buffers, uploads, ops and read-backs all go
    through the backend vtable of the cuda_sm100 plugin (include/scrapgpu/backend.h:29-57 of the reference; the
    reference's core forwards scrapgpu_buffer_write / scrapgpu_plan_execute / ... to exactly these slots).  The
    plugin's weights are separate buffers of its own (tensor_upload with the packed-layout tag, the way
    examples/standalone_matmul.c:126-130 uploads)."""
    import ctypes as C
    from scrapgpulibrary_b200 import _build, abi
    if not os.path.exists(_build.PLUGIN_SO):
        raise FileNotFoundError(f"{_build.PLUGIN_SO} is missing: the end-to-end leg needs the backend plugin")
    P = C.CDLL(_build.PLUGIN_SO, mode=C.RTLD_GLOBAL)
    P.scrapgpu_cuda_sm100_vtable.restype = C.POINTER(abi.Vtable)
    vt = P.scrapgpu_cuda_sm100_vtable().contents
    L = capi.lib()

    def ok(st, what):
        if st != 0:
            raise RuntimeError(f"{what}: status {st}: {(L.sm100_last_error() or b'').decode()}")

    dev, st_ = C.c_void_p(), C.c_void_p()
    ok(vt.get_device(None, device_index, C.byref(dev)), "get_device")
    ok(vt.stream_create(dev, C.byref(st_)), "stream_create")

    def alloc(nbytes):
        b = C.c_void_p()
        ok(vt.buffer_alloc(dev, nbytes, C.byref(b)), "buffer_alloc")
        return b

    def pinned(nbytes):
        p = C.c_void_p()
        capi.check(L.sm100_host_alloc(nbytes, C.byref(p)), "host_alloc")
        return p

    # weights: natural bytes up, packed on the way (layout tag 1)
    wdesc = {}
    for s, (k, n) in enumerate(SHAPES):
        base = pool[s]["natural"]
        for layer in sorted({l for ss, l in order if ss == s}):
            buf = alloc(base.nbytes)
            d = abi.tensor_desc(dtype, [k, n], buffer=buf.value, layout=abi.LAYOUT_R32)
            rot = np.ascontiguousarray(np.roll(base, layer * 17, axis=0) if layer else base)
            ok(vt.tensor_upload(st_, C.byref(d), rot.ctypes.data_as(C.c_void_p), rot.nbytes), "tensor_upload")
            wdesc[(s, layer)] = d
    # one activation arena and one result arena on the device, mirrored by two pinned host arenas: a step's inputs
    # go up with ONE buffer_write and its results come back with ONE buffer_read (tensor i lives at its offset)
    xoff, yoff, xo, yo = [], [], 0, 0
    for s, _ in order:
        xoff.append(xo)
        yoff.append(yo)
        xo += 4 * SHAPES[s][0]
        yo += 4 * SHAPES[s][1]
    xarena, yarena = alloc(xo), alloc(yo)
    hx, hy = pinned(xo), pinned(yo)
    C.memmove(hx, rng.standard_normal(xo // 4).astype(np.float32).ctypes.data, xo)
    ops = []
    for i, (s, layer) in enumerate(order):
        k, n = SHAPES[s]
        ops.append(abi.Op(abi.OP_MUL_MAT, [wdesc[(s, layer)], abi.tensor_desc(abi.F32, [k], buffer=xarena.value, offset=xoff[i])],
                          [abi.tensor_desc(abi.F32, [n], buffer=yarena.value, offset=yoff[i])], abi.MulMatParams(0, 0)))
    nodes = (abi.PlanNode * len(ops))()
    for i, o in enumerate(ops):
        nodes[i].struct_size = C.sizeof(abi.PlanNode)
        nodes[i].op = o.desc
        nodes[i].output_use_count = 0
    pd = abi.PlanDesc(C.sizeof(abi.PlanDesc), nodes, len(ops))
    plan = C.c_void_p()
    ok(vt.plan_build(dev, C.byref(pd), C.byref(plan)), "plan_build")
    # the same step as PIPE_CHUNKS plans on PIPE_STREAMS streams of the device (the products are independent of each other):
    # while one stream's kernels run, another stream's activations go up and its results come down, and the launch chains
    # of the streams hide each other's hand-over phases (measured: 2 streams 3.54, 3: 4.0, 4: 4.16, 6: 4.30 TB/s)
    PIPE_CHUNKS = int(os.environ.get("BENCH_PIPE_CHUNKS", "6"))
    PIPE_STREAMS = int(os.environ.get("BENCH_PIPE_STREAMS", "6"))
    pipe_streams = [st_]
    for _ in range(PIPE_STREAMS - 1):
        sx = C.c_void_p()
        ok(vt.stream_create(dev, C.byref(sx)), "stream_create")
        pipe_streams.append(sx)
    bounds = [len(ops) * c // PIPE_CHUNKS for c in range(PIPE_CHUNKS + 1)]
    chunk_plans, keep = [], []
    for c in range(PIPE_CHUNKS):
        lo, hi = bounds[c], bounds[c + 1]
        cn = (abi.PlanNode * (hi - lo))()
        for j in range(lo, hi):
            cn[j - lo].struct_size = C.sizeof(abi.PlanNode)
            cn[j - lo].op = ops[j].desc
            cn[j - lo].output_use_count = 0
        cpd = abi.PlanDesc(C.sizeof(abi.PlanDesc), cn, hi - lo)
        cp = C.c_void_p()
        ok(vt.plan_build(dev, C.byref(cpd), C.byref(cp)), "plan_build")
        keep.append(cn)
        xlo, xhi = xoff[lo], (xoff[hi] if hi < len(ops) else xo)
        ylo, yhi = yoff[lo], (yoff[hi] if hi < len(ops) else yo)
        chunk_plans.append((cp, xlo, xhi - xlo, ylo, yhi - ylo))
    sizes = [(4 * SHAPES[s][0], 4 * SHAPES[s][1]) for s, _ in order]
    hxi = [C.c_void_p(hx.value + o) for o in xoff]
    hyi = [C.c_void_p(hy.value + o) for o in yoff]

    def step(per_op):
        if per_op == "pipelined":
            for c, (cp, xlo, xn, ylo, yn) in enumerate(chunk_plans):
                sc = pipe_streams[c % PIPE_STREAMS]
                ok(vt.buffer_write(sc, xarena, xlo, C.c_void_p(hx.value + xlo), xn, 0), "buffer_write")
                ok(vt.plan_execute(sc, cp), "plan_execute")
                ok(vt.buffer_read(sc, yarena, ylo, C.c_void_p(hy.value + ylo), yn, 0), "buffer_read")
            for sx in pipe_streams[1:]:
                ok(vt.stream_sync(sx), "stream_sync")
        elif per_op:     # one write, one op_execute and one read per matvec
            for i, o in enumerate(ops):
                ok(vt.buffer_write(st_, xarena, xoff[i], hxi[i], sizes[i][0], 0), "buffer_write")
                ok(vt.op_execute(st_, o.ptr()), "op_execute")
                ok(vt.buffer_read(st_, yarena, yoff[i], hyi[i], sizes[i][1], 0), "buffer_read")
        else:
            ok(vt.buffer_write(st_, xarena, 0, hx, xo, 0), "buffer_write")
            ok(vt.plan_execute(st_, plan), "plan_execute")
            ok(vt.buffer_read(st_, yarena, 0, hy, yo, 0), "buffer_read")
        ok(vt.stream_sync(st_), "stream_sync")

    def timed(per_op):
        for _ in range(warmup):
            step(per_op)
        t0 = time.perf_counter()      # every step ends with a stream_sync: host time brackets the device work
        for _ in range(steps):
            step(per_op)
        return (time.perf_counter() - t0) * 1e3 / steps

    plan_ms = timed(False)
    per_op_ms = timed(True)
    pipe_ms = timed("pipelined")
    C.memset(hy, 0xFF, yo)
    step("pipelined")     # the results checked below are those of the pipelined form
    # the results that arrived on the host are the device path's (same kernels): compare one product per shape
    checked = 0
    for s in range(len(SHAPES)):
        i = next(j for j, (ss, _) in enumerate(order) if ss == s)
        k, n = SHAPES[s]
        got = np.ctypeslib.as_array(C.cast(hyi[i], C.POINTER(C.c_float)), shape=(n,)).copy()
        xh = np.ctypeslib.as_array(C.cast(hxi[i], C.POINTER(C.c_float)), shape=(k,)).copy()
        xd, yd = capi.Buffer(4 * k), capi.Buffer(4 * n)
        xd.upload(stream, xh)
        capi.mul_mat(stream, dtype, 1, pool[s]["mats"][order[i][1]], k, n, xd, 1, yd)
        stream.sync()
        want = yd.download(stream, np.float32, n)
        # (the plan's products may be served by another kernel of the same integer arithmetic than a lone call: same block
        # sums, added in another order)
        err = float(np.sum((got.astype(np.float64) - want) ** 2) / max(np.sum(want.astype(np.float64) ** 2), 1e-30))
        if not np.isfinite(got).all() or err > 1e-10:
            raise RuntimeError(f"end-to-end result of shape {SHAPES[s]} differs from the device-resident call (NMSE {err:.3g})")
        checked += 1
        xd.free()
        yd.free()
    ok(vt.plan_free(plan), "plan_free")
    for cp, *_ in chunk_plans:
        ok(vt.plan_free(cp), "plan_free")
    for sx in pipe_streams[1:]:
        vt.stream_free(sx)
    for b in [xarena, yarena] + [C.c_void_p(d.buffer) for d in wdesc.values()]:
        vt.buffer_free(b)
    for p in (hx, hy):
        L.sm100_host_free(p)
    vt.stream_free(st_)
    return {"ms_per_step": plan_ms, "one_stream_ms_per_step": plan_ms, "pipelined_ms_per_step": pipe_ms, "per_op_ms_per_step": per_op_ms,
            "checked": checked, "form": "one stream", "pipe_chunks": PIPE_CHUNKS, "pipe_streams": PIPE_STREAMS}


def e2e_sharded(capi, stream, pool, order, enqueue_step, xs, ys, dist, warmup, steps):
    """N > 1: the sharded sweep with HOST activations and results through the C ABI of the compute library: per step one
    host->device copy of every activation buffer from pinned memory, the step's launches (matvecs and all-reduces, one
    graph), one device->host read of every result buffer, one sync.  Host clock, maximum over the ranks."""
    import ctypes as C
    import torch
    L = capi.lib()
    ks = sorted({pool[s]["k"] for s, _ in order})
    ns = sorted({pool[s]["n"] for s, _ in order})
    host = {}
    for key, size in [(("x", k), 4 * k) for k in ks] + [(("y", n), 4 * n) for n in ns]:
        p = C.c_void_p()
        capi.check(L.sm100_host_alloc(size, C.byref(p)), "host_alloc")
        C.memset(p, 0, size)
        host[key] = (p, size)
    with capi.Graph(stream) as g:
        enqueue_step(1, None)

    def step():
        for k in ks:
            p, size = host[("x", k)]
            capi.check(L.sm100_memcpy_h2d(stream.handle, C.c_void_p(xs[k].ptr), p, size, 0), "memcpy_h2d")
        g.launch()
        for n in ns:
            p, size = host[("y", n)]
            capi.check(L.sm100_memcpy_d2h(stream.handle, p, C.c_void_p(ys[n].ptr), size, 0), "memcpy_d2h")
        stream.sync()

    for _ in range(warmup):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    ms = (time.perf_counter() - t0) * 1e3 / steps
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    g.destroy()
    for p, _ in host.values():
        L.sm100_host_free(p)
    return {"ms_per_step": float(t.item()),
            "note": "the sharded sweep through the C ABI of the compute library with host buffers: per step the activation buffers go up from pinned host "
                    "memory (sm100_memcpy_h2d, non-blocking), one graph launch of the rank's matvecs and all-reduces, the result buffers come back "
                    "(sm100_memcpy_d2h, non-blocking), one sync; host clock, maximum over the ranks"}


def sharded_head(capi, rank: int, world: int, local_rank: int, dist, allreduce=None, reps: int = 50):
    """Q6_K output head, K = 4096, N = 151936 rows split evenly over the ranks (151936 / P is a multiple of the
    16-row tile for P = 2, 4, 8), each rank's slice of the logits all-gathered by NCCL.  One CUDA graph holds `reps`
    rounds of matvec + all-gather; the time is the maximum over the ranks.  A second graph times the greedy form: the
    matvec followed by the library's arg-max exchange (sm100_argmax_allreduce), which moves P candidates instead of the
    logits."""
    import torch
    from scrapgpulibrary_b200 import synth
    k, n = 4096, 151936
    n_local = n // world
    assert n_local * world == n and n_local % 16 == 0
    L = capi.lib()
    dev = torch.device("cuda", local_rank)
    ts = torch.cuda.Stream(device=dev)
    handle = C.c_void_p(ts.cuda_stream)
    base = synth.quantized_matrix(33, 99 + rank, 16384, k)
    nat = np.tile(base, (-(-n_local // base.shape[0]), 1))[:n_local]
    natural = torch.from_numpy(np.ascontiguousarray(nat)).to(dev)
    packed = torch.empty(natural.numel(), dtype=torch.uint8, device=dev)
    x = torch.randn(k, device=dev, dtype=torch.float32)
    y_local = torch.empty(n_local, device=dev, dtype=torch.float32)
    y_all = torch.empty(n, device=dev, dtype=torch.float32)
    with torch.cuda.stream(ts):
        capi.check(L.sm100_pack_device(handle, 33, k, n_local, C.c_void_p(natural.data_ptr()), C.c_void_p(packed.data_ptr())), "pack_device")

        def round_():
            capi.check(L.sm100_mul_mat(handle, 33, 1, C.c_void_p(packed.data_ptr()), 0, k, n_local, C.c_void_p(x.data_ptr()), k, 1,
                                       C.c_void_p(y_local.data_ptr()), n_local), "mul_mat")
            dist.all_gather_into_tensor(y_all, y_local)
        round_()
    torch.cuda.synchronize(dev)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=ts):
        for _ in range(reps):
            round_()
    torch.cuda.synchronize(dev)
    with torch.cuda.stream(ts):
        g.replay()
    torch.cuda.synchronize(dev)
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(ts):
        e0.record()
        g.replay()
        e1.record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    total = algorithmic_bytes(33, k, n)
    out = {"ranks": world, "rows_per_rank": n_local, "us_per_round": round(ms * 1e3, 1), "gbps_aggregate": round(total / (ms * 1e-3) / 1e9, 1),
           "collective": "NCCL all_gather_into_tensor of 151936 f32 logits"}
    if allreduce is not None:
        token = torch.zeros(1, device=dev, dtype=torch.int32)

        def greedy_round():
            capi.check(L.sm100_mul_mat(handle, 33, 1, C.c_void_p(packed.data_ptr()), 0, k, n_local, C.c_void_p(x.data_ptr()), k, 1,
                                       C.c_void_p(y_local.data_ptr()), n_local), "mul_mat")
            capi.check(L.sm100_argmax_allreduce(allreduce.ctx, handle, C.c_void_p(y_local.data_ptr()), n_local, rank * n_local,
                                                C.c_void_p(token.data_ptr())), "argmax_allreduce")
        with torch.cuda.stream(ts):
            greedy_round()
        torch.cuda.synchronize(dev)
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2, stream=ts):
            for _ in range(reps):
                greedy_round()
        torch.cuda.synchronize(dev)
        with torch.cuda.stream(ts):
            g2.replay()
        torch.cuda.synchronize(dev)
        dist.barrier()
        with torch.cuda.stream(ts):
            e0.record()
            g2.replay()
            e1.record()
        torch.cuda.synchronize(dev)
        t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out["us_per_round_greedy"] = round(float(t.item()) * 1e3, 1)
        out["greedy"] = "matvec + sm100_argmax_allreduce (local arg-max, P candidates exchanged by tagged peer stores): the token, not the logits"
    return out


def other_formats(capi, stream, reps: int = 20):
    """Algorithmic GB/s at M = 1 of the formats beside the headline: Q6_K on the three projection shapes, Q4_0
    4096 x 4096, and the Q6_K vocabulary head (4096 x 151936).  Weights rotate through enough distinct tensors to
    exceed L2 (the head is 510 MB on its own); graph replay of `reps` rounds."""
    from scrapgpulibrary_b200 import synth
    out = {}
    L = capi.lib()
    # (name, dtype, K, N, distinct tensors, batches)
    cases = [("q6_k", 33, 4096, 4096, 12, (1, 2, 4, 8)), ("q6_k", 33, 4096, 12288, 5, (1, 2, 4, 8)), ("q6_k", 33, 12288, 4096, 5, (1, 2, 4, 8)),
             ("q4_0", 16, 4096, 4096, 16, (1,)), ("q8_0", 17, 4096, 4096, 10, (1,)), ("q6_k_head", 33, 4096, 151936, 1, (1,))]
    for name, dtype, k, n, copies, batches in cases:
        base = synth.quantized_matrix(dtype, 40 + dtype + n % 97, min(n, 16384), k)
        if n > base.shape[0]:
            base = np.tile(base, (-(-n // base.shape[0]), 1))[:n]
        staging = capi.Buffer(base.nbytes)
        mats = []
        for c in range(copies):
            staging.upload(stream, np.roll(base, c * 17, axis=0) if c else base)
            dst = capi.Buffer(base.nbytes)
            capi.check(L.sm100_pack_device(stream.handle, dtype, k, n, staging.at(), dst.at()), "pack_device")
            stream.sync()
            mats.append(dst)
        staging.free()
        x = capi.Buffer(4 * k * 8)
        x.upload(stream, np.random.default_rng(k).standard_normal(k * 8).astype(np.float32))
        y = capi.Buffer(4 * n * 8)
        for m in batches:
            with capi.Graph(stream) as g:
                for w in mats:
                    capi.mul_mat(stream, dtype, 1, w, k, n, x, m, y)
            for _ in range(3):
                g.launch()
            e0, e1 = capi.Event(), capi.Event()
            e0.record(stream)
            for _ in range(reps):
                g.launch()
            e1.record(stream)
            e1.sync()
            ms = e0.elapsed_ms(e1) / (reps * copies)
            g.destroy()
            out[f"{name}_k{k}_n{n}_m{m}_gbps"] = round(algorithmic_bytes(dtype, k, n, m) / (ms * 1e-3) / 1e9, 1)
        for b in mats + [x, y]:
            b.free()
    return out


def prefill_gemm(capi, stream, reps: int = 20):
    """Q8_0 prefill MUL_MAT at M = 512: dense TFLOP/s (2 M K N / time) of the tensor-core path, weights rotating
    through at least 192 MB of tensors per shape so that successive launches do not find them in L2."""
    from scrapgpulibrary_b200 import synth
    out = {}
    m, k = 512, 4096
    x = capi.Buffer(4 * m * k)
    x.upload(stream, np.random.default_rng(5).standard_normal(m * k).astype(np.float32))
    for n in (4096, 12288):
        img = capi.pack(17, k, synth.quantized_matrix(17, 9, n, k))
        ws = []
        for _ in range(max(4, -(-(192 << 20) // img.nbytes))):   # rotate through more weight bytes than the 126 MB L2 holds
            b = capi.Buffer(img.nbytes)
            b.upload(stream, img)
            ws.append(b)
        y = capi.Buffer(4 * m * n)
        for i in range(3):
            capi.mul_mat(stream, 17, 1, ws[i], k, n, x, m, y)
        e0, e1 = capi.Event(), capi.Event()
        e0.record(stream)
        for i in range(reps):
            capi.mul_mat(stream, 17, 1, ws[i % len(ws)], k, n, x, m, y)
        e1.record(stream)
        e1.sync()
        ms = e0.elapsed_ms(e1) / reps
        out[f"q8_0_gemm_m{m}_k{k}_n{n}_tflops"] = round(2.0 * m * k * n / (ms * 1e-3) / 1e12, 1)
        out[f"q8_0_gemm_m{m}_k{k}_n{n}_us"] = round(ms * 1e3, 1)
        for b in ws + [y]:
            b.free()
    x.free()
    return out


def run_decode(args, rank: int, world: int, local_rank: int, dist, stream_sync):
    """Qwen3-8B-shaped layer-stack decode: 36 layers, hidden 4096, 32/8 heads of 128, FFN 12288,
    vocab 151936, random Q4_K_M-style weights, f32 KV cache pre-filled to position 1024, batch 1, greedy; one CUDA
    graph per token, tensor-parallel over `world` ranks with NCCL all-reduces.  Returns tok/s and the roofline view."""
    import torch
    from scrapgpulibrary_b200.decode import DecodeConfig, DecodeModel
    cfg = DecodeConfig()
    steps = args.decode_steps
    allreduce, exchange = None, "none"
    if world > 1:
        exchange = os.environ.get("SM100_TP_EXCHANGE", "peer")
        if exchange == "peer":   # the library's one-shot all-reduce over peer-mapped memory; "nccl" = torch.distributed
            from scrapgpulibrary_b200.collective import PeerAllReduce
            allreduce = PeerAllReduce(rank, world, local_rank, cfg.hidden, dist)
    model = DecodeModel(cfg, rank=rank, world=world, device_index=local_rank, seed=0x5CA9, allreduce=allreduce)
    model.reset(token=1234, prefill_seed=7)
    model.capture()
    model.reset(token=1234, prefill_seed=None)
    model.run(8)                                   # warm-up tokens
    torch.cuda.synchronize()
    model.reset(token=1234, prefill_seed=None)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(model.tstream):
        e0.record()
    model.run(steps)
    with torch.cuda.stream(model.tstream):
        e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    tokens = model.tokens(steps)
    # the CPU oracle's greedy tokens for this very model, first token and KV prefill (tests/golden/make_decode_golden.py)
    match = None
    try:
        gold = json.load(open(os.path.join(ROOT, "tests", "golden", "decode_qwen3_8b_shape.json")))
        if gold["seed"] == 0x5CA9 and gold["first_token"] == 1234 and gold["prefill_seed"] == 7 and steps >= len(gold["tokens"]):
            match = [int(x) for x in tokens[:len(gold["tokens"])]] == gold["tokens"]
    except Exception:
        match = None
    peak, _ = measured_peak_gbs()
    mid_pos = cfg.start_pos + steps // 2
    bytes_tok = model.bytes_per_token(mid_pos)      # this rank's share
    tok_s = steps / (ms * 1e-3)
    return {"tok_s": round(tok_s, 1), "ms_per_token": round(ms / steps, 4), "steps": steps, "tp": world, "all_reduce": exchange,
            "all_reduce_fault": allreduce.fault() if allreduce is not None else 0,
            "bytes_per_token_per_gpu": int(bytes_tok), "hbm_gbps_per_gpu": round(bytes_tok * tok_s / 1e9, 1),
            "hbm_frac_of_measured": round(bytes_tok * tok_s / 1e9 / peak, 4),
            "model": "Qwen3-8B shape, random Q4_K_M-style weights (Q6_K for attn_v / ffn_down in the more-bits layers and the head)",
            "first_tokens": [int(x) for x in tokens[:6]], "tokens_match_cpu_oracle": match}


def cpu_baseline(pool, threads: int, repeats: int):
    """The reference's CPU MUL_MAT on one layer's three matrices (natural blocks), GB/s of algorithmic bytes."""
    try:
        from oracle import refapi
        use_ref = refapi.available()
    except Exception:
        use_ref = False
    from oracle import sgref
    rng = np.random.default_rng(7)
    times = []
    total = sum(algorithmic_bytes(Q4_K, p["k"], p["n"]) for p in pool)
    xs = {p["k"]: rng.standard_normal((1, p["k"])).astype(np.float32) for p in pool}   # (N = 1: the pool holds whole matrices)
    for _ in range(repeats + 1):
        t0 = time.perf_counter()
        for p in pool:
            if use_ref:
                refapi.mul_mat(Q4_K, p["natural"], p["k"], xs[p["k"]], threads=threads)
            else:
                sgref.mul_mat(Q4_K, p["natural"], p["k"], xs[p["k"]], threads=threads)
        times.append(time.perf_counter() - t0)
    t = statistics.median(times[1:])
    return {"value": round(total / t / 1e9, 3), "unit": "GB/s", "cores": threads, "kind": "reference" if use_ref else "port",
            "sample": f"one layer (3 matrices, {total / 1e6:.1f} MB), M=1, median of {repeats} after 1 warm-up, {t * 1e3:.1f} ms per pass"}


def run_reference(args, rank: int, world: int):
    """The reference arm: the unmodified CPU implementation on the host cores, all threads."""
    if rank != 0:
        return None
    from scrapgpulibrary_b200 import synth
    threads = os.cpu_count() or 1
    pool = [{"k": k, "n": n, "natural": synth.quantized_matrix(Q4_K, 0x5CA9 + si, n, k)} for si, (k, n) in enumerate(SHAPES)]
    for _ in range(max(1, min(args.warmup, 3))):
        cpu_baseline(pool, threads, 1)
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    res = None
    for _ in range(steps):
        res = cpu_baseline(pool, threads, 1)
    elapsed = (time.perf_counter() - t0) / steps / 2.0  # each call runs 1 warm-up + 1 timed pass
    total = sum(algorithmic_bytes(Q4_K, p["k"], p["n"]) for p in pool)
    value = res["value"]
    return {"impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": args.warmup,
            "ms_per_step": round(total / (value * 1e9) * 1e3, 3), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32 (SSE2 scalar / panel code of the reference's CPU backend)", "data": "synthetic: seeded N(0, 0.02) weights in Q4_K blocks, N(0, 1) activations",
            "config": {"workload": f"Q4_K matvec sweep, M=1, Qwen3-8B projection shapes (K,N) in {SHAPES}; each step = one layer (bounded sample of the sweep)"},
            "cpu_baseline": {**res, "cores": threads}, "gpu_launches": 0,
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "wall_s_per_step": round(elapsed, 3)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--decode-steps", type=int, default=128)
    ap.add_argument("--no-decode", action="store_true", help="skip the layer-stack decode measurement")
    ap.add_argument("--no-pdl", action="store_true", help="launch without programmatic dependent launch (profiler runs)")
    ap.add_argument("--gemm-only", action="store_true", help="Q8_0 prefill GEMM shapes only, single GPU: for profiler runs")
    ap.add_argument("--decode-only", action="store_true", help="layer-stack decode only, single GPU: for profiler runs")
    ap.add_argument("--quick", action="store_true", help="headline sweep only (no per-shape detail, e2e, CPU baseline, decode): for profiler runs")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        out = run_reference(args, rank, world)
    else:
        out = run_ours(args, rank, world, local_rank)
    if rank == 0 and out is not None:
        print(json.dumps(out), flush=True)
    if world > 1:
        # Leave without tearing the NCCL communicator down: destroy_process_group() was seen to block for minutes
        # while captured CUDA graphs still reference the communicator.  All ranks have passed the final barrier,
        # nothing is in flight.
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
