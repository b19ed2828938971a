"""Benchmark of the compressed-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (single GPU): every projection of a Mistral-7B decoder block (q 4096x4096, k/v
1024x4096, o 4096x4096, gate/up 14336x4096, down 4096x14336), weights N(0, 0.02) compressed
to 4-bit codes at 50 % sparsity with 128-wide groups, one decode token (M = 1).  A "step" is
one pass of the decode GEMV over the seven matrices.  Several copies of the block are
rotated so that every step streams its weights from HBM (the working set is several times
the 126 MB L2).

  value      GB/s of algorithmic compressed bytes (bitmask + codes + fp16 scale/zero +
             activations in/out) with all inputs resident in HBM, timed with CUDA events
             around K steps replayed from a CUDA graph.  q|k|v and gate|up read the same
             activations and go out as one fused launch each (4 launches per step).
  e2e        the same metric through the library's host-buffer entry points: pinned host
             activations copied in and the results copied back by every call
             (cobalt_gemv_fused_host_async for q|k|v and gate|up, cobalt_linear_host_async for o and
             down); the four calls of a step alternate between two streams and the caller waits
             for both once per step.
  roofline   the GEMV kernel against the measured HBM copy bandwidth.
  cpu_baseline  the reference path (dense bf16 weight, torch.matmul) on the host cores.

With --gpus N > 1 (launched by torch.distributed.run) the run is tensor-parallel with the work
per GPU held fixed (weak scaling): every rank streams one shard with the 7B block's shapes of
a block N times as wide - q/k/v/gate/up split by output rows (no exchange), o/down split by
input columns, their fp32 partial sums all-reduced once per layer (the library's peer-memory kernel; NCCL with
--nccl-allreduce or when the symmetric buffer cannot be set up) and rounded once.  The end-to-end leg of a
multi-GPU run goes through the same tensor-parallel step, host copies included.

The line also carries two short extra legs (single GPU, skipped with --no-extra): `prefill` - the tcgen05 GEMM on
two 7B shapes at M = 128 and 2048 against the measured bf16 peak - and `model` - a reduced-depth (4-layer)
Mistral-7B-shaped greedy decode with ms per layer and the 32-layer tokens/s extrapolated from it (labelled).

Other workloads: `--workload prefill` (tcgen05 GEMM sweep over the 7B shapes, M in --prefill-m, 3-bit/70 % and
2-bit/50 %) and `--workload model` (full greedy decode of a random-init model: `--model mistral7b|gemma27b`,
`--context`, `--new-tokens`, `--batch` sequences decoded together, `--head-bits` for a compressed and, with several
GPUs, vocabulary-split head, `--prefill-tokens` for the timed prompt; tensor-parallel under torch.distributed.run).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES_7B = [("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096),
             ("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336)]
ROW_PARALLEL = ("o", "down")
BITS, SPARSITY, BETA = 4, 0.5, 0.5
L2_BYTES = 126 * 1024 * 1024


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                mhz.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


# ----------------------------------------------------------------------------- workload construction
def build_block(device, rank=0, seed0=1000):
    """Compress and pack the seven projections of one block (rank `rank`'s shard of the wide block) on `device`."""
    from cobalt_b200 import CobaltSparseLinear, SparseQuantConfig, compress_weight
    from cobalt_b200.format import pack_tiles
    mods, info = {}, {}
    seed0 += 100 * rank
    cfg = SparseQuantConfig(BITS, SPARSITY, BETA)
    for idx, (name, K, N) in enumerate(SHAPES_7B):
        g = torch.Generator(device="cpu").manual_seed(seed0 + idx)
        W = (torch.randn(K, N, generator=g) * 0.02).half().float().to(device)
        norm = (torch.randn(N, generator=g).abs() + 0.1).to(device)
        keep, q, sc, zr = compress_weight(W, norm, cfg)
        del W
        mod = CobaltSparseLinear.__new__(CobaltSparseLinear)
        torch.nn.Module.__init__(mod)
        mod._install(pack_tiles(keep.contiguous(), q.contiguous(), sc.contiguous(), zr.contiguous(), BITS), None, None,
                     {"nbits": BITS})
        mods[name] = mod
        info[name] = dict(K=mod.out_features, N=mod.in_features, bytes=mod.compressed_bytes())
        del keep, q, sc, zr
    torch.cuda.empty_cache()
    return mods, info


def clone_block(mods):
    from cobalt_b200 import CobaltSparseLinear
    from cobalt_b200.format import TileImage
    out = {}
    for name, m in mods.items():
        c = CobaltSparseLinear.__new__(CobaltSparseLinear)
        torch.nn.Module.__init__(c)
        c._install(TileImage.from_meta(m.packed.clone(), m._img_meta), None, None, {"nbits": m.bits})
        out[name] = c
    return out


def step_bytes(info, M):
    w = sum(v["bytes"] for v in info.values())
    act = sum(M * v["N"] * 2 + M * v["K"] * 2 for v in info.values())
    return w, act


def _finish(dist):
    """Leave a multi-rank run without tearing NCCL down: the process group may hold communicators that a
    captured CUDA graph still references, and its destructor has been seen to wait forever.  All ranks meet at a
    barrier (so nobody is killed mid-collective), flush their output and exit the process directly."""
    if dist is None:
        return
    try:
        dist.barrier()
        torch.cuda.synchronize()
    finally:
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


# ----------------------------------------------------------------------------- our arm
def run_ours(args):
    from cobalt_b200 import _lib
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))
    lib = _lib.load()
    M = args.tokens

    global SHAPES_7B
    if args.shapes:
        want = args.shapes.split(",")
        SHAPES_7B = [t for t in SHAPES_7B if t[0] in want]
    mods0, info = build_block(dev, rank)
    wbytes, abytes = step_bytes(info, M)
    copies = max(2, -(-4 * L2_BYTES // max(wbytes, 1)))          # working set >= 4 x L2
    copies = min(copies, 64)
    if args.copies > 0:
        copies = args.copies
    blocks = [mods0] + [clone_block(mods0) for _ in range(copies - 1)]
    stream = torch.cuda.Stream(dev)
    xs = {name: (torch.randn(M, v["N"], device=dev) ).to(torch.bfloat16) for name, v in info.items()}
    ys = {name: torch.empty(M, v["K"], dtype=torch.bfloat16, device=dev) for name, v in info.items()}

    from cobalt_b200 import FusedProjections
    reducer = None
    if world > 1 and not args.nccl_allreduce:
        try:                                                 # all-reduce over peer memory; NCCL if it cannot be set up
            from cobalt_b200.tp import PeerReducer
            reducer = PeerReducer(M * max(v["K"] for n, v in info.items() if n in ROW_PARALLEL), dev)
        except Exception as e:                               # noqa: BLE001 - any failure means "use NCCL"
            if rank == 0:
                print(f"peer all-reduce unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)
            reducer = None
    names = [t[0] for t in SHAPES_7B]
    fuse_groups = [] if args.no_fuse else [g for g in (("q", "k", "v"), ("gate", "up")) if all(n in names for n in g)]
    fused_of = {n: g for g in fuse_groups for n in g}
    launches_per_step = len(names) - sum(len(g) - 1 for g in fuse_groups)

    def make_fused(blk):
        return {g: FusedProjections([blk[n] for n in g]) for g in fuse_groups}

    def one_step(blk, fused):
        done = set()
        for name in names:
            if name in done:
                continue
            if name in fused_of:                            # q|k|v and gate|up share their activations: one launch
                fused[fused_of[name]](xs[name])
                done.update(fused_of[name])
            elif world > 1 and name in ROW_PARALLEL:        # fp32 partial sums, one all-reduce, one rounding
                if reducer is not None:
                    n = M * info[name]["K"]
                    blk[name](xs[name], out_fp32=True, out=reducer.slot_view(n))
                    reducer.reduce(n, ys[name].view(-1))
                else:
                    part = blk[name](xs[name], out_fp32=True)
                    dist.all_reduce(part)
                    ys[name].copy_(part)
            else:
                blk[name](xs[name])

    fuseds = [make_fused(b) for b in blocks]
    with torch.cuda.stream(stream):
        for b, f in zip(blocks, fuseds):                     # allocate scratch, configure kernels
            one_step(b, f)
        stream.synchronize()
        graph, step_graphs = None, []
        if not args.profile and not args.no_graph:
            # the all-reduces of the tensor-parallel run are captured with the kernels (NCCL supports capture).
            # One graph holds a step on every block copy; one more graph per copy serves step counts that are not a
            # multiple of the number of copies, so that every timed (and warm-up) step is a replay.
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for b, f in zip(blocks, fuseds):
                    one_step(b, f)
            for b, f in zip(blocks, fuseds):
                gs = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gs, stream=stream):
                    one_step(b, f)
                step_graphs.append(gs)

        def run_steps(n):
            done = 0
            while done < n:
                if graph is not None and n - done >= len(blocks):
                    graph.replay()
                    done += len(blocks)
                elif step_graphs:
                    step_graphs[done % len(blocks)].replay()
                    done += 1
                else:
                    one_step(blocks[done % len(blocks)], fuseds[done % len(blocks)])
                    done += 1

        # the timed region is ONE graph of exactly `steps` steps (copies rotated), so that no launch gap between graphs
        # falls inside it; very long runs fall back to replaying the per-copy graphs
        timed_graph = None
        if graph is not None and args.steps <= 1000:
            timed_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(timed_graph, stream=stream):
                for i in range(args.steps):
                    one_step(blocks[i % len(blocks)], fuseds[i % len(blocks)])
        run_steps(max(args.warmup, 3))
        if timed_graph is not None:
            timed_graph.replay()                             # first replay uploads the graph; it is warm-up too
        stream.synchronize()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()                                  # before the barrier: starting the sampler takes rank 0 about a
        if dist is not None:                                 # millisecond, which the other ranks would spend waiting in their
            dist.barrier()                                   # first all-reduce inside the timed region
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.nvtx.range_push("cobalt_timed")          # lets a profiler restrict itself to the timed region
        e0.record(stream)
        if timed_graph is not None:
            timed_graph.replay()
        else:
            run_steps(args.steps)
        e1.record(stream)
        stream.synchronize()
        torch.cuda.nvtx.range_pop()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        # per-shape launch time (graph of one launch per copy, replayed)
        per_shape = {}
        if world == 1 and not args.profile:
            for name, _, _ in SHAPES_7B:
                gsh = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gsh, stream=stream):
                    for b in blocks:
                        b[name](xs[name])
                for _ in range(3):
                    gsh.replay()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = 20
                a0.record(stream)
                for _ in range(reps):
                    gsh.replay()
                a1.record(stream)
                stream.synchronize()
                us = a0.elapsed_time(a1) * 1e3 / (reps * len(blocks))
                nbytes = info[name]["bytes"] + M * (info[name]["N"] + info[name]["K"]) * 2
                per_shape[name] = {"us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1)}
        # the same step on a single block copy: its 88.6 MB stay in the 126 MB L2 (labelled, not the headline)
        l2_resident = None
        if world == 1 and not args.profile and graph is not None:
            g1 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g1, stream=stream):
                for _ in range(len(blocks)):
                    one_step(blocks[0], fuseds[0])
            for _ in range(3):
                g1.replay()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(stream)
            for _ in range(10):
                g1.replay()
            a1.record(stream)
            stream.synchronize()
            l2_ms = a0.elapsed_time(a1) / (10 * len(blocks))
            l2_resident = {"value": round((wbytes + abytes) / (l2_ms * 1e-3) / 1e9, 2), "unit": "GB/s", "ms_per_step": round(l2_ms, 5),
                           "note": "one block copy replayed: weights stay in L2"}
        # hold the load a little longer so that the clock sampler sees it
        if not args.profile:
            if world == 1:
                t_end = time.time() + 1.0
                while time.time() < t_end:
                    run_steps(len(blocks))
                    stream.synchronize()
            else:                                           # same fixed count on every rank: the steps contain collectives
                run_steps(max(2000, 10 * args.steps))
                stream.synchronize()
        clocks = sampler.stop() if rank == 0 else None
        status = max(m.device_status() for b in blocks for m in b.values())

    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps
    total_bytes = (wbytes + abytes) * world                  # every rank streams its shard
    value = total_bytes / (ms_step * 1e-3) / 1e9

    if args.profile:
        if rank == 0:
            print(json.dumps({"profile_run": True, "value": round(value, 2), "unit": "GB/s", "ms_per_step": round(ms_step, 5),
                              "shapes": [t[0] for t in SHAPES_7B], "copies": copies}), flush=True)
        _finish(dist)
        return
    # ---- end to end through the host-buffer entry point (rank-local; aggregated like `value`)
    e2e_steps = max(3, min(args.steps, 20))
    hx = {n: xs[n].cpu().pin_memory() for n in xs}
    hy = {n: torch.empty(M, info[n]["K"], dtype=torch.bfloat16).pin_memory() for n in xs}
    scr = {}
    for name, m in mods0.items():
        need = lib.cobalt_gemv_scratch_bytes(ctypes.byref(m._descriptor()), M)
        scr[name] = torch.zeros(need + 256, dtype=torch.uint8, device=dev)

    side = torch.cuda.Stream(dev)                            # the seven calls are independent: two streams let one
    e2e_streams = (stream, side)                             # call's copy-out overlap the next call's copy-in and kernel

    dx = {n: torch.empty_like(xs[n]) for n in xs}             # device staging of the tensor-parallel end-to-end step

    # single GPU: the calls of the device-timed step (q|k|v and gate|up as one fused call each, o, down), each fed from
    # pinned host activations and read back to pinned host outputs by the library's host entry points
    fused_scr, fused_args = {}, {}
    for g in fuse_groups:
        descs = (ctypes.POINTER(_lib.CobaltMat) * len(g))(*[ctypes.pointer(mods0[n]._descriptor()) for n in g])
        need = lib.cobalt_gemv_fused_scratch_bytes(len(g), descs, M)
        fused_scr[g] = torch.zeros(need + 256, dtype=torch.uint8, device=dev)

    def e2e_step(blk, fused):
        if world == 1:
            done, k = set(), 0
            for name in names:
                if name in done:
                    continue
                st = e2e_streams[k & 1].cuda_stream
                k += 1
                if name in fused_of:
                    g = fused_of[name]
                    key = (id(blk), g)
                    if key not in fused_args:                # descriptor and pointer arrays of a call, built once per block copy
                        fused_args[key] = ((ctypes.POINTER(_lib.CobaltMat) * len(g))(*[ctypes.pointer(blk[n]._descriptor()) for n in g]),
                                           (ctypes.c_void_p * len(g))(*[hy[n].data_ptr() for n in g]),
                                           (ctypes.c_void_p * len(g))(*[ys[n].data_ptr() for n in g]))
                    descs, yh, yd = fused_args[key]
                    sp = (fused_scr[g].data_ptr() + 255) // 256 * 256
                    rc = lib.cobalt_gemv_fused_host_async(len(g), descs, hx[name].data_ptr(), yh, M, xs[name].data_ptr(), yd, sp,
                                                          fused_scr[g].numel() - 256, st)
                    _lib.check("cobalt_gemv_fused_host_async", rc)
                    done.update(g)
                else:
                    m = blk[name]
                    sp = (scr[name].data_ptr() + 255) // 256 * 256
                    rc = lib.cobalt_linear_host_async(ctypes.byref(m._descriptor()), hx[name].data_ptr(), hy[name].data_ptr(), None, M,
                                                      xs[name].data_ptr(), ys[name].data_ptr(), sp, scr[name].numel() - 256, st)
                    _lib.check("cobalt_linear_host_async", rc)
            stream.synchronize()                              # the caller reads the results: one wait per block
            side.synchronize()
            return
        # tensor parallel: the same step as the device-timed one (fused launches, fp32 partial sums of o and down
        # all-reduced over the ranks), fed from pinned host activations and read back to pinned host outputs
        with torch.cuda.stream(stream):
            done = set()
            for name in names:
                if name in done:
                    continue
                dx[name].copy_(hx[name], non_blocking=True)
                if name in fused_of:
                    outs = fused[fused_of[name]](dx[name])
                    for n2, o in zip(fused_of[name], outs):
                        hy[n2].copy_(o, non_blocking=True)
                    done.update(fused_of[name])
                elif name in ROW_PARALLEL:
                    if reducer is not None:
                        n = M * info[name]["K"]
                        blk[name](dx[name], out_fp32=True, out=reducer.slot_view(n))
                        reducer.reduce(n, ys[name].view(-1))
                    else:
                        part = blk[name](dx[name], out_fp32=True)
                        dist.all_reduce(part)
                        ys[name].copy_(part)
                    hy[name].copy_(ys[name], non_blocking=True)
                else:
                    hy[name].copy_(blk[name](dx[name]), non_blocking=True)
        stream.synchronize()

    for i in range(3):
        e2e_step(blocks[i % len(blocks)], fuseds[i % len(blocks)])
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(blocks[i % len(blocks)], fuseds[i % len(blocks)])
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    if dist is not None:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_val = total_bytes / (e2e_ms * 1e-3) / 1e9

    if rank != 0:
        _finish(dist)
        return
    peak, peak_kind = measured_peaks()
    out = {
        "metric": "compressed-linear achieved GB/s (7B block decode, compressed bytes)",
        "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_step, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"Mistral-7B block projections q/k/v/o/gate/up/down, {BITS}-bit, {int(SPARSITY*100)}% sparse, "
                               f"g=128, M={M} decode GEMV" + (f"; tensor-parallel x{world}, one such shard per GPU, fp32 all-reduce "
                                                               f"after o and down ({'peer-memory kernel' if reducer is not None else 'NCCL'})" if world > 1 else ""),
                   "l2": f"{copies} block copies rotated ({copies * wbytes / 1e6:.0f} MB working set > L2)",
                   "bytes_per_step": int(wbytes + abytes), "peak": peak_kind},
        "clocks": clocks,
        "e2e": {"value": round(e2e_val, 2), "unit": "GB/s", "ms_per_step": round(e2e_ms, 4),
                "path": "cobalt_gemv_fused_host_async (q|k|v, gate|up) and cobalt_linear_host_async (o, down), two streams, one wait per step" if world == 1 else
                        "tensor-parallel step through the module API: pinned host x in, fused launches, all-reduce of o and down, pinned host y out",
                "h2d_bytes_per_step": int(sum(M * info[n]["N"] * 2 for n in names if n not in fused_of or fused_of[n][0] == n)),
                "d2h_bytes_per_step": int(sum(M * v["K"] * 2 for v in info.values()))},
        # this library's kernels inside the timed region: the GEMVs, a fragment-ordering copy in front of each GEMV that
        # cannot stage its activations (more than 8 tokens), and the peer all-reduce kernels of a tensor-parallel step
        "gpu_launches": int(args.steps * (launches_per_step * (2 if M > 8 else 1) +
                                          (len([n for n in names if n in ROW_PARALLEL]) if (world > 1 and reducer is not None) else 0))),
        "roofline": {"bound": "hbm", "achieved": round(value / world, 2), "peak": peak, "unit": "GB/s",
                     "frac": round(value / world / peak, 4),
                     # DRAM bytes per launch: 1.005 x algorithmic, from an ncu capture of the gate projection
                     # (24.03 MB read for 23.9 MB); traffic grows in proportion to the tiles streamed
                     "traffic": int(1.005 * (wbytes + abytes) / launches_per_step),
                     "kernel": f"gemv_mma_kernel<{BITS},{2 if M > 8 else 1},{'true' if M <= 8 else 'false'}>", "launches_per_step": launches_per_step,
                     "bytes_per_launch": int((wbytes + abytes) / launches_per_step)},
        "device_status": status,
        "per_shape": per_shape,
        "l2_resident": l2_resident,
    }
    if world == 1:
        out["cpu_baseline"] = cpu_baseline(info, M, limit_s=15.0)
        if not args.no_extra:
            del blocks, fuseds, mods0
            torch.cuda.empty_cache()
            try:
                out.update(extra_legs(dev))
            except Exception as e:                            # noqa: BLE001 - the extra legs never take the headline line down
                out["extra_legs_error"] = f"{type(e).__name__}: {e}"
    print(json.dumps(out), flush=True)
    _finish(dist)


# ----------------------------------------------------------------------------- short extra legs of the default line
def extra_legs(dev, steps=5):
    """Two short single-GPU legs appended to the decode line: the tensor-bound prefill GEMM on two 7B shapes and a
    reduced-depth model decode.  Both use seeded synthetic weights; every timed prefill launch follows an L2 flush."""
    from cobalt_b200 import CobaltSparseLinear, SparseQuantConfig, compress_weight
    from cobalt_b200.decoder import build_random_decoder
    out = {}
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = json.load(open(p))["bf16_tflops"] if os.path.exists(p) else 1590.0
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    cases = []
    for name, K, N in (("down", 4096, 14336), ("q", 4096, 4096)):
        g = torch.Generator().manual_seed(4003)
        W = (torch.randn(K, N, generator=g) * 0.02).half().float().to(dev)
        norm = (torch.randn(N, generator=g).abs() + 0.1).to(dev)
        keep, q, sc, zr = compress_weight(W, norm, SparseQuantConfig(3, 0.7, 0.5))
        mod = CobaltSparseLinear(q, sc, zr, keep, None, None, {"nbits": 3})
        del W, keep, q, sc, zr
        for M in (2048, 128):
            x = torch.randn(M, N, device=dev).to(torch.bfloat16)
            for _ in range(3):
                mod(x)
            times = []
            for _ in range(steps):
                flush.fill_(1)
                torch.cuda._sleep(400_000)                     # device-side spacer: the host enqueues the launch meanwhile
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                mod(x)
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
            ms = sorted(times)[len(times) // 2]
            tf = 2.0 * M * K * N / (ms * 1e-3) / 1e12
            cases.append({"shape": name, "M": M, "bits": 3, "sparsity": 0.7, "ms": round(ms, 4), "tflops": round(tf, 1),
                          "tensor_frac": round(tf / peak, 4), "status": mod.device_status()})
        del mod
    del flush
    torch.cuda.empty_cache()
    out["prefill"] = {"metric": "prefill GEMM TFLOP/s (dense-equivalent 2*M*K*N), 3-bit 70 % sparse", "peak_tflops": peak,
                      "kernel": "gemm_tcgen05_kernel<3>", "l2": "256 MB flush before every timed launch", "cases": cases}
    # reduced-depth model decode: 4 layers of the 7B shape (every layer its own copy of one set of seeded matrices)
    layers, ctx, n_new = 4, 2048, 64
    cfg = dict(model_type="mistral", hidden_size=4096, num_hidden_layers=layers, num_attention_heads=32, num_key_value_heads=8,
               head_dim=128, intermediate_size=14336, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=1e6, sliding_window=None)
    dec = build_random_decoder(cfg, SparseQuantConfig(BITS, SPARSITY, BETA), ctx + n_new + 8, dev, clone_first_layer=True)
    g = torch.Generator().manual_seed(2048)
    prompt = torch.randint(0, cfg["vocab_size"], (ctx,), generator=g)
    dec.generate(prompt, 4, use_graph=True)
    torch.cuda.synchronize()
    dec.pos.fill_(ctx)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_new):
        dec._graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms4 = e0.elapsed_time(e1) / n_new
    ms_head = dec.time_head_ms()
    ms_layer = max(ms4 - ms_head, 0.0) / layers
    out["model"] = {"metric": "Mistral-7B-shape greedy decode, batch 1, context 2048", "layers_run": layers,
                    "ms_per_token_4_layers": round(ms4, 4), "ms_head_and_embedding": round(ms_head, 4), "ms_per_layer": round(ms_layer, 4),
                    "tokens_per_s_32_layers_extrapolated": round(1e3 / (32 * ms_layer + ms_head), 1),
                    "note": "extrapolated from 4 layers: 32 * ms_per_layer + head; the full-depth run is `--workload model`",
                    "status": max(m.device_status() for m in dec.lin.values())}
    del dec
    torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------- CPU arm (reference path)
def cpu_baseline(info, M, limit_s=15.0, steps=None, warmup=1):
    """The reference path on the host cores: SparseQuantLinear keeps a dense bf16 copy of the
    dequantised weight after its first call and multiplies with torch.matmul
    (benchmarks/benchmark_suite.py:1200-1217).  The weight values do not influence the time, so a
    seeded dense bf16 matrix of the right shape stands in for the dequantised one."""
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(1)
    Ws = {n: (torch.randn(v["K"], v["N"], generator=g) * 0.02).to(torch.bfloat16) for n, v in info.items()}
    xs = {n: torch.randn(M, v["N"], generator=g).to(torch.bfloat16) for n, v in info.items()}

    def step():
        for n in Ws:
            torch.matmul(xs[n], Ws[n].t())

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    n = 0
    while True:
        step()
        n += 1
        el = time.perf_counter() - t0
        if (steps is not None and n >= steps) or (steps is None and (el > limit_s or n >= 50)):
            break
    ms = el * 1e3 / n
    wbytes, abytes = step_bytes(info, M)
    out = {"value": round((wbytes + abytes) / (ms * 1e-3) / 1e9, 3), "unit": "GB/s", "cores": threads, "kind": "port",
           "ms_per_step": round(ms, 3),
           "sample": f"{n} passes over one block (7 dense bf16 matmuls, cached-weight mode of the reference module), M={M}"}
    # the reference's low-memory mode dequantises on every call (benchmarks/benchmark_suite.py:1203-1209): one matrix, few calls
    name = "q" if "q" in info else next(iter(info))
    K, N = info[name]["K"], info[name]["N"]
    from oracle import cobalt_oracle as O
    raw = O.synth_raw(K, N, SPARSITY, BITS, seed=3)
    keep, q, sc, zr = raw["keep"], raw["q"], raw["scale"], raw["zero"]
    x = xs[name]
    O.linear_forward(x, q, sc, zr, keep)
    t0 = time.perf_counter()
    reps = 2
    for _ in range(reps):
        O.linear_forward(x, q, sc, zr, keep)
    lm = (time.perf_counter() - t0) * 1e3 / reps
    out["lowmem"] = {"value": round((info[name]["bytes"] + M * (K + N) * 2) / (lm * 1e-3) / 1e9, 3), "unit": "GB/s", "ms": round(lm, 2),
                     "sample": f"dequantise + matmul of {name} ({K}x{N}) on every call, {reps} calls"}
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    info = {}
    for name, K, N in SHAPES_7B:
        nnz = int(K * N * (1 - SPARSITY))
        info[name] = dict(K=K, N=N, bytes=K * N // 8 + (BITS * nnz + 7) // 8 + K * (N // 128) * 4)
    M = args.tokens
    cb = cpu_baseline(info, M, steps=max(1, args.steps), warmup=max(1, min(args.warmup, 3)))
    wbytes, abytes = step_bytes(info, M)
    out = {"impl": "reference", "metric": "compressed-linear achieved GB/s (7B block decode, compressed bytes)",
           "value": cb["value"], "unit": "GB/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": cb["ms_per_step"], "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
           "config": {"workload": f"Mistral-7B block projections q/k/v/o/gate/up/down, {BITS}-bit, {int(SPARSITY*100)}% sparse, "
                                  f"g=128, M={M}: reference CPU path (dense bf16 weight + torch.matmul)",
                      "bytes_per_step": int(wbytes + abytes)},
           "cpu_baseline": cb,
           "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out), flush=True)


# ----------------------------------------------------------------------------- prefill sweep (tensor-bound leg)
def run_prefill(args):
    """Prefill GEMM sweep on the 7B projection shapes: M in {128, 512, 2048}, 3-bit/70 % and 2-bit/50 %.
    Prints one JSON line with TFLOP/s (2*M*K*N per launch) per case against the measured bf16 peak.
    Every timed launch is preceded by an L2 flush (256 MB written) and timed with its own event pair."""
    from cobalt_b200 import CobaltSparseLinear, SparseQuantConfig, compress_weight
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = json.load(open(p))["bf16_tflops"] if os.path.exists(p) else 1590.0
    shapes = [("q", 4096, 4096), ("kv", 1024, 4096), ("gate_up", 14336, 4096), ("down", 4096, 14336)]
    if args.shapes:
        shapes = [t for t in shapes if t[0] in args.shapes.split(",")]
    if args.probe_shape:                                     # one custom matrix, e.g. 128,512 = a single CTA with 8 stages
        K, N = (int(v) for v in args.probe_shape.split(","))
        shapes = [("probe", K, N)]
    Ms = [int(m) for m in args.prefill_m.split(",")]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    cases = []
    for bits, sp in ((3, 0.7), (2, 0.5)):
        for name, K, N in shapes:
            g = torch.Generator().manual_seed(4000 + bits)
            W = (torch.randn(K, N, generator=g) * 0.02).half().float().to(dev)
            norm = (torch.randn(N, generator=g).abs() + 0.1).to(dev)
            keep, q, sc, zr = compress_weight(W, norm, SparseQuantConfig(bits, sp, 0.5))
            mod = CobaltSparseLinear(q, sc, zr, keep, None, None, {"nbits": bits})
            del W, keep, q, sc, zr
            for M in Ms:
                x = torch.randn(M, N, device=dev).to(torch.bfloat16)
                for _ in range(3):
                    mod(x)
                times = []
                for _ in range(args.steps if args.steps < 50 else 10):
                    flush.fill_(1)
                    torch.cuda._sleep(400_000)                 # ~0.2 ms of device time: the host enqueues the launch meanwhile,
                    torch.cuda.nvtx.range_push("cobalt_timed")  # so the events bracket the kernel, not the host's launch path
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    mod(x)
                    e1.record()
                    torch.cuda.synchronize()
                    torch.cuda.nvtx.range_pop()
                    times.append(e0.elapsed_time(e1))
                times.sort()
                ms = times[len(times) // 2]
                tf = 2.0 * M * K * N / (ms * 1e-3) / 1e12
                cases.append({"shape": name, "K": K, "N": N, "M": M, "bits": bits, "sparsity": sp, "ms": round(ms, 4),
                              "tflops": round(tf, 1), "frac": round(tf / peak, 4), "status": mod.device_status()})
            del mod
            torch.cuda.empty_cache()
    best = max(cases, key=lambda c: c["tflops"])
    print(json.dumps({"metric": "prefill GEMM TFLOP/s (dense-equivalent 2*M*K*N)", "unit": "TFLOP/s", "value": best["tflops"],
                      "roofline": {"bound": "tensor", "achieved": best["tflops"], "peak": peak, "unit": "TFLOP/s",
                                   "frac": best["frac"], "kernel": "gemm_tcgen05_kernel"},
                      "config": {"workload": "prefill sweep on Mistral-7B projection shapes", "l2": "256 MB flush before every timed launch"},
                      "cases": cases}), flush=True)


# ----------------------------------------------------------------------------- full decode (7B shape)
def run_model(args):
    """Random-init Mistral-7B-shaped decoder, every projection 4-bit / 50 % sparse: the KV cache is pre-filled
    with 2048 seeded random tokens (one prefill through the tcgen05 GEMM), then 256 greedy tokens are decoded
    from a CUDA graph.  Prints tokens/s over the replayed decode steps (the prefill is not timed)."""
    from cobalt_b200 import SparseQuantConfig
    from cobalt_b200.decoder import build_random_decoder
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist, reducer = None, None
    cfg = dict(model_type="mistral", hidden_size=4096, num_hidden_layers=args.layers, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=32000, rms_norm_eps=1e-5,
               rope_theta=1e6, sliding_window=None)
    bits, sparsity, label = BITS, SPARSITY, "Mistral-7B"
    if args.model == "gemma27b":                             # Gemma-3-27B text shape, 3-bit / 60 % sparse
        cfg = dict(model_type="gemma3_text", hidden_size=5376, num_hidden_layers=62 if args.layers == 32 else args.layers,
                   num_attention_heads=32, num_key_value_heads=16, head_dim=128, intermediate_size=21504, vocab_size=262144,
                   rms_norm_eps=1e-6, sliding_window=1024, sliding_window_pattern=6, query_pre_attn_scalar=168,
                   rope_theta=1e6, rope_local_base_freq=1e4, rope_scaling={"rope_type": "linear", "factor": 8.0})
        bits, sparsity, label = 3, 0.6, "Gemma-3-27B"
    if world > 1:                                            # tensor parallel: heads and MLP columns split over the ranks
        import datetime
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
        if not args.nccl_allreduce:
            try:
                from cobalt_b200.tp import PeerReducer
                reducer = PeerReducer(16 * cfg["hidden_size"], dev)
            except Exception as e:                           # noqa: BLE001 - any failure means "use NCCL"
                if rank == 0:
                    print(f"peer all-reduce unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)
    ctx, n_new, B = args.context, args.new_tokens, args.batch
    dec = build_random_decoder(cfg, SparseQuantConfig(bits, sparsity, BETA), ctx + n_new, dev, tp_rank=rank, tp_world=world,
                               reducer=reducer, clone_first_layer=args.model == "gemma27b", batch=B, head_bits=args.head_bits)
    dec.fused_prompt_attention = bool(args.fused_prompt_attention)
    dec.push_partials = bool(args.push)
    g = torch.Generator().manual_seed(2048)
    prompt = torch.randint(0, cfg["vocab_size"], (ctx,) if B == 1 else (B, ctx), generator=g)
    n_pre = min(args.prefill_tokens or ctx, ctx)
    t0 = time.perf_counter()
    dec.generate(prompt, 4, use_graph=True)                     # prefill + graph capture + a few steps (warm-up)
    torch.cuda.synchronize()
    warm_s = time.perf_counter() - t0
    # time to first token: one more prefill of the same prompt through the tcgen05 GEMM (kernels are configured now)
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    p0.record()
    dec.prefill(prompt[..., :n_pre] if B == 1 else prompt[:1, :n_pre])   # one sequence; a prefix rewrites the same cache slots
    p1.record()
    torch.cuda.synchronize()
    prefill_ms = p0.elapsed_time(p1)
    if dist is not None:
        t = torch.tensor([prefill_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        prefill_ms = float(t.item())
    # timed: replay the captured step n_new times (token and position advance on the device)
    dec.pos.fill_(ctx)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(n_new):
        dec._graph.replay()
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = e0.elapsed_time(e1) / n_new
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    wbytes = sum(m.compressed_bytes() for m in dec.lin.values()) * world
    status = max(m.device_status() for m in dec.lin.values())
    if rank != 0:
        _finish(dist)
        return
    head_bytes = dec.head.compressed_bytes() * world if dec.head is not None else cfg["vocab_size"] * cfg["hidden_size"] * 2
    head_txt = f"{args.head_bits}-bit group-128 RTN head" + (" split over the vocabulary" if world > 1 else "") \
        if dec.head is not None else "dense bf16 lm_head"
    print(json.dumps({"metric": f"{label}-shape decode tokens/s (batch {B})", "value": round(B * 1e3 / ms, 2), "unit": "tokens/s",
                      "ms_per_step": round(ms, 4), "batch": B, "n_gpus": world, "dtype": "bf16", "data": "synthetic",
                      "scaling": "strong",
                      "config": {"workload": f"{label} shape, {cfg['num_hidden_layers']} layers, {bits}-bit {int(sparsity*100)}% sparse, "
                                             f"batch {B}, context {ctx}, {n_new} greedy tokens, CUDA graph; {head_txt}"
                                             + ("; every layer holds its own copy of the first layer's seeded matrices" if args.model == "gemma27b" else "")
                                             + (f"; tensor-parallel x{world} ({'peer-memory' if reducer is not None else 'NCCL'} all-reduce)" if world > 1 else ""),
                                 "compressed_bytes_per_token": int(wbytes), "lm_head_bytes": head_bytes},
                      "linear_GBps": round(wbytes / (ms * 1e-3) / 1e9, 1), "clocks": clocks, "device_status": status,
                      "prefill_attention": "fused library kernel (not the spec's rounding points)" if args.fused_prompt_attention else "spec arithmetic",
                      "prefill_tokens": n_pre, "prefill_ms": round(prefill_ms, 2),
                      "prefill_tokens_per_s": round(n_pre / (prefill_ms * 1e-3), 1),
                      "warmup_s": round(warm_s, 1)}), flush=True)
    _finish(dist)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=1, help="decode batch M (1..16)")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "model"],
                    help="decode = headline 7B block GEMV bench; prefill = tcgen05 GEMM sweep; model = full 7B-shape "
                         "greedy decode tokens/s (both single GPU)")
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--batch", type=int, default=1, help="--workload model: sequences decoded together (1..16)")
    ap.add_argument("--head-bits", type=int, default=0, help="--workload model: compress the head with group-128 RTN at this width (0 = dense bf16)")
    ap.add_argument("--prefill-tokens", type=int, default=0, help="--workload model: tokens of the timed prefill (0 = the whole context)")
    ap.add_argument("--prefill-m", default="128,512,2048")
    ap.add_argument("--probe-shape", default="", help="--workload prefill: K,N of one custom matrix instead of the 7B shapes")
    ap.add_argument("--shapes", default="", help="comma-separated subset of q,k,v,o,gate,up,down (profiling aid)")
    ap.add_argument("--copies", type=int, default=0, help="block copies to rotate (0 = enough for 4 x L2)")
    ap.add_argument("--no-graph", action="store_true", help="launch every step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--bits", type=int, default=0, help="decode workload: code width (default 4, the headline configuration)")
    ap.add_argument("--sparsity", type=float, default=-1.0, help="decode workload: pruned fraction (default 0.5)")
    ap.add_argument("--fused-prompt-attention", action="store_true", help="--workload model: fused library attention for the prompt")
    ap.add_argument("--model", default="mistral7b", choices=["mistral7b", "gemma27b"], help="shape of --workload model")
    ap.add_argument("--nccl-allreduce", action="store_true", help="multi-GPU: use NCCL instead of the peer-memory all-reduce kernel")
    ap.add_argument("--no-fuse", action="store_true", help="one launch per projection instead of fused q|k|v and gate|up")
    ap.add_argument("--push", action="store_true",
                    help="--workload model, multi-GPU: partial sums pushed by the GEMV and added by the next projection's staging "
                         "instead of the copy-based peer all-reduce kernel")
    ap.add_argument("--no-extra", action="store_true", help="skip the short prefill and reduced-depth model legs of the default line")
    ap.add_argument("--profile", action="store_true",
                    help="plain launches only: no CUDA graph, no end-to-end leg, no CPU baseline (for ncu captures)")
    args = ap.parse_args()
    global BITS, SPARSITY
    if args.bits:
        BITS = args.bits
    if args.sparsity >= 0:
        SPARSITY = args.sparsity
    if args.workload == "prefill":
        run_prefill(args)
    elif args.workload == "model":
        run_model(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
