#!/usr/bin/env python
"""Benchmark of the Q4_K x Q8 hot path.

Workload at every N (the row-sharded whole-model weight stream of the benchmark configurations, config[4]):
64 synthetic layers of the decode projection set (QKV 7168x5120, O 5120x5120, gate+up 34816x5120,
down 5120x17408; Q4_K weights, 11.9 GB), walked once with M = 1 token and once with M = 64 tokens per step;
bf16 N(0,1) activations are quantised on the device in front of every layer.  With N > 1 GPUs every matrix is
split by output rows over the ranks (strong scaling) and every projection stores its rows into every rank's
copy of the gathered output over NVLink, inside the projection kernel.  64 distinct layers are far larger
than L2, so HBM serves the weights.  One step is captured once as a CUDA graph and replayed.

Prints ONE JSON line (rank 0).  Extra keys at N = 1: the single-layer decode set by token count (config[1]),
prefill shapes (config[2]) with their own roofline object against the int8 tensor peak measured in the same
run, the ragged batch (config[3]), the fitter.  `--impl reference` times the CPU restatement of the reference
equation on the host cores instead (rank 0 only).  `--only project|fit|deq` runs one small case a few times
for a profiler and prints nothing of the above."""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPES = [("qkv", 7168, 5120), ("o", 5120, 5120), ("gate_up", 34816, 5120), ("down", 5120, 17408)]
STREAM_TOKENS = [1, 64]          # config[4]
STREAM_LAYERS = 64
SET_TOKENS = [1, 2, 4, 8, 16]    # config[1]
SET_LAYERS = 8
METRIC = "q4k_q8_decode_weight_stream_GBps"
WORKLOAD = ("config[4]: 64 synthetic layers of the decode projection set (QKV 7168x5120, O 5120x5120, gate+up 34816x5120, "
            "down 5120x17408; Q4_K, 11.9 GB), each matrix split by output rows over the GPUs, one pass at M=1 and one at M=64 "
            "per step, bf16 activations quantised on device")


def weight_bytes(n, k):
    return n * (k // 256) * 144


def algorithmic_bytes(m, n, k):
    """Q4_K weights read once + Q8 activations (codes, fp32 scale, int32 sum) + fp32 output."""
    return weight_bytes(n, k) + m * (k + (k // 32) * 8) + m * n * 4


def set_bytes(m, quantise=True):
    """One projection set at m tokens (+ the two bf16 inputs when the quantiser runs in the timed region)."""
    return sum(algorithmic_bytes(m, n, k) for _, n, k in SHAPES) + (m * (5120 + 17408) * 2 if quantise else 0)


def stream_step_bytes():
    return sum(STREAM_LAYERS * set_bytes(m) for m in STREAM_TOKENS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [l for (t, l) in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l for (_, l) in self.lines]
        sm, smax, reasons = [], [], set()
        for l in rows:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference equation on the host cores
# ----------------------------------------------------------------------------------------------
def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        return os.cpu_count() or 1


def cpu_sample(repeats: int, rows_per_matrix: int = 256):
    """Times the CPU restatement on a bounded sample of the workload: `rows_per_matrix` output rows of every
    matrix of the set at M = 1 and M = 64, on all host cores (the thread count is set explicitly: a launcher may
    have exported OMP_NUM_THREADS=1).  Returns (GB/s, cores, text)."""
    from oracle import oracle as orc
    from qw38_b200 import synth
    handle = orc.lib(native=True)
    cores = orc.set_threads(host_cores(), handle)
    mats = []
    for i, (_, n, k) in enumerate(SHAPES):
        codes, meta = synth.logical_q4k(rows_per_matrix, k, seed=100 + i)
        mats.append((k,) + synth.split_tiles(codes, meta))
    acts = {}
    for m in STREAM_TOKENS:
        for k in (5120, 17408):
            xb = synth.f32_to_bf16_bits(synth.activations(m, k, seed=m))
            acts[(m, k)] = orc.q8_quantize(xb, bf16_bits=True)[:3]
    nbytes = sum(algorithmic_bytes(m, rows_per_matrix, k) for m in STREAM_TOKENS for _, _, k in SHAPES)
    best = float("inf")
    for _ in range(max(1, repeats)):
        t0 = time.perf_counter()
        for m in STREAM_TOKENS:
            for (k, hc, hs) in mats:
                z, a, s = acts[(m, k)]
                orc.project_rows(hc, hs, rows_per_matrix, k, z, a, s, 0, rows_per_matrix, handle=handle)
        best = min(best, time.perf_counter() - t0)
    return (nbytes / best / 1e9, cores,
            f"{rows_per_matrix} rows of each of the 4 matrices, M in {STREAM_TOKENS}, best of {max(1, repeats)}")


def cpu_reference_gemv_sample(rows: int = 512):
    """The reference's own host GEMV for this weight format (compiler::reference_gemv_packed: dequantise to bf16,
    fp32 FMA with the bf16 activations; single thread), compiled from the reference's sources: one token,
    `rows` rows of the gate matrix.  None when that library is not present."""
    from oracle import oracle as orc
    from qw38_b200 import synth
    if orc.ref() is None:
        return None
    k = 5120
    codes, meta = synth.logical_q4k(rows, k, seed=7)
    hc, hs = synth.split_tiles(codes, meta)
    xb = synth.f32_to_bf16_bits(synth.activations(1, k, seed=3))[0]
    orc.ref_gemv_packed(hc, hs, rows, k, xb)
    best = float("inf")
    for _ in range(3):
        t0 = time.perf_counter()
        orc.ref_gemv_packed(hc, hs, rows, k, xb)
        best = min(best, time.perf_counter() - t0)
    nbytes = weight_bytes(rows, k) + k * 2 + rows * 4
    return {"value": nbytes / best / 1e9, "unit": "GB/s", "cores": 1, "kind": "_ref",
            "sample": f"reference_gemv_packed (bf16-operand policy), {rows} rows x {k}, one token, best of 3"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warm = max(1, args.steps), max(0, args.warmup)
    cpu_sample(1)  # build + warm caches
    for _ in range(warm):
        cpu_sample(1)
    t0 = time.perf_counter()
    vals = [cpu_sample(1) for _ in range(steps)]
    elapsed = time.perf_counter() - t0
    gbps = statistics.median(v[0] for v in vals)
    cores, sample = vals[0][1], vals[0][2]
    line = {"impl": "reference", "metric": METRIC, "value": gbps, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": warm, "ms_per_step": elapsed / steps * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8 dot / fp32 affine", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sample": sample},
            "cpu_baseline": {"value": gbps, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": gbps, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------
# Profiler cases: one small operation a few times, nothing else
# ----------------------------------------------------------------------------------------------
def run_only(args):
    import torch
    from qw38_b200 import synth
    from qw38_b200.q4k_q8 import dequantize_bf16, pack_q8, q4k_q8_project, quantize_q4k_weight
    dims = [int(v) for v in args.shape.split(",")]
    if args.only == "deq":
        wd = synth.device_weight(dims[0], dims[1], seed=0)
        for _ in range(3):
            o = dequantize_bf16(wd)
        torch.cuda.synchronize()
        print("ok", float(o.float().abs().mean()))
    elif args.only == "fit":
        wf = torch.randn((dims[0], dims[1]), device="cuda") * 0.02
        for _ in range(3):
            pw = quantize_q4k_weight(wf, check=False)
        torch.cuda.synchronize()
        print("ok", int(pw.codes.sum()))
    elif args.only == "project":
        n, k, m = dims
        w = synth.device_weight(n, k, seed=0)
        f = torch.zeros(1, dtype=torch.int32, device="cuda")
        q = pack_q8(torch.randn((m, k), device="cuda").to(torch.bfloat16), f)
        out = torch.empty((m, n), dtype=torch.float32, device="cuda")
        for _ in range(3):
            q4k_q8_project(w, q, out=out, kernel=args.kernel, split_k=args.split_k, row_groups=args.row_groups, trusted=True)
        torch.cuda.synchronize()
        print("ok", float(out.abs().mean()))
    else:
        raise SystemExit(f"unknown --only {args.only}")


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the N = 1 extra keys (config[1], prefill, ragged, fitter)")
    ap.add_argument("--layers", type=int, default=STREAM_LAYERS, help="debug: fewer layers than the workload's 64")
    ap.add_argument("--no-graph", action="store_true", help="debug / profiling: eager launches instead of CUDA graph replay")
    ap.add_argument("--no-overlap", action="store_true",
                    help="launch every kernel fully serialised (no programmatic dependent launch)")
    ap.add_argument("--only", default="", help="profiler case: project (--shape n,k,m --kernel id), fit or deq (--shape n,k)")
    ap.add_argument("--shape", default="34816,5120,8")
    ap.add_argument("--kernel", type=int, default=0)
    ap.add_argument("--split-k", type=int, default=0)
    ap.add_argument("--row-groups", type=int, default=0)
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.only:
        return run_only(args)

    import torch
    import torch.distributed as dist
    from qw38_b200 import _lib as L
    from qw38_b200 import synth
    from qw38_b200.q4k_q8 import (new_q8_input, pack_q8, peer_wait, q4k_q8_project, q4k_q8_project_gather,
                                  reserve_scratch, set_launch_overlap)
    from qw38_b200.sharding import row_shard, symmetric_pool

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = L.load()
    steps, warm = max(1, args.steps), max(3, args.warmup)
    n_layers = max(1, args.layers)
    workload = WORKLOAD if n_layers == STREAM_LAYERS else WORKLOAD.replace("64 synthetic layers", f"{n_layers} synthetic layers (debug)")

    def shard(n):
        row0, rows, per = row_shard(n, world, rank)
        if rows != per:
            raise SystemExit(f"{n} rows do not split evenly over {world} ranks in row groups of 8")
        return row0, rows

    # ---- weights: this rank's row shard of every matrix of every layer
    layers = [[synth.device_weight(shard(n)[1], k, seed=1000 * l + 10 * i + rank, device=dev) for i, (_, n, k) in enumerate(SHAPES)]
              for l in range(n_layers)]
    g = torch.Generator(device=dev)
    g.manual_seed(1234)
    failure = torch.zeros(1, dtype=torch.int32, device=dev)

    # ---- activations: one bf16 buffer per parity (so that the end-to-end leg can refill one while the other is read)
    tokens = STREAM_TOKENS
    x_words = sum(m * (5120 + 17408) for m in tokens)
    x_host = torch.randn(x_words, generator=torch.Generator().manual_seed(99)).to(torch.bfloat16).pin_memory()
    x_pool = [x_host.to(dev), x_host.to(dev)]

    def x_views(pool):
        views, off = {}, 0
        for m in tokens:
            for k in (5120, 17408):
                views[(m, k)] = pool[off:off + m * k].view(m, k)
                off += m * k
        return views
    x_in = [x_views(x_pool[0]), x_views(x_pool[1])]
    q8 = {(m, k): new_q8_input(m, k, dev) for m in tokens for k in (5120, 17408)}

    # ---- outputs: the full [m, n] result of every (token count, matrix), two copies (step parity).  With several GPUs
    # they live in one symmetric allocation so that each projection kernel can store its rows into every peer.
    out_words = sum(m * n for m in tokens for _, n, _ in SHAPES)
    fused = world > 1
    if fused:
        pool, bases, pool_handle = symmetric_pool(2 * out_words + 16, dev)
        flag_ptrs = [b + 4 * 2 * out_words for b in bases]
    else:
        pool, bases = torch.empty(2 * out_words, dtype=torch.float32, device=dev), None
    outs, out_ptrs, out_group = {}, {}, {}
    off = 0
    for parity in (0, 1):
        start = off
        for m in tokens:
            for i, (_, n, _) in enumerate(SHAPES):
                outs[(parity, m, i)] = pool[off:off + m * n].view(m, n)
                if fused:
                    out_ptrs[(parity, m, i)] = [b + 4 * off for b in bases]
                off += m * n
        out_group[parity] = pool[start:off]

    def projection(m, i, layer, parity):
        # Both activation packs of a layer are enqueued before its four projections, so no projection's input is
        # written by the launch directly before it: the projections may run into each other (input_settled).
        _, n, k = SHAPES[i]
        settled = not args.no_overlap
        if fused:
            q4k_q8_project_gather(layers[layer][i], q8[(m, k)], out_ptrs[(parity, m, i)], flag_ptrs, rank, shard(n)[0], n,
                                  input_settled=settled)
        else:
            q4k_q8_project(layers[layer][i], q8[(m, k)], out=outs[(parity, m, i)], trusted=True, input_settled=settled)

    def stream_step(parity, quantise=True, only_m=None, wait=True):
        for m in tokens:
            if only_m is not None and m != only_m:
                continue
            for layer in range(n_layers):
                if quantise:
                    for k in (5120, 17408):
                        pack_q8(x_in[parity][(m, k)], failure, out=q8[(m, k)])
                for i in range(len(SHAPES)):
                    projection(m, i, layer, parity)
        if fused and wait:
            peer_wait(flag_ptrs, rank)  # this step's rows of every peer have landed

    stream = torch.cuda.Stream(device=dev)
    copy_stream = torch.cuda.Stream(device=dev)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    # ---- one eager step, then the gathered outputs against the CPU statement of the equation (every rank checks every
    # rank's rows in its OWN copy: a row that did not arrive over NVLink fails here)
    for m in tokens:  # split-K scratch at its final size before anything is captured
        for _, n, _ in SHAPES:
            reserve_scratch(16 * m * shard(n)[1] * 4)
    with torch.cuda.stream(stream):
        stream_step(0)
    barrier()
    if failure.item() != 0:
        raise SystemExit("non-finite activation flagged")
    checked = verify_against_oracle(torch, dist, world, rank, layers[n_layers - 1], q8, outs, shard, tokens)
    barrier()

    # The weights are final from here on, which is what the overlapped launches require.
    set_launch_overlap(not args.no_overlap)

    class Eager:
        def __init__(self, fn):
            self.fn = fn

        def replay(self):
            self.fn()

    def capture(fn):
        if args.no_graph:
            return Eager(fn)
        with torch.cuda.stream(stream):
            fn()
            torch.cuda.synchronize(dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                fn()
        return graph

    def timed(graphs, n):
        """n replays, graphs[s % len] for step s; device time by CUDA events, max over ranks."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for s in range(n):
                graphs[s % len(graphs)].replay()
            e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    step_graphs = [capture(lambda p=p: stream_step(p)) for p in (0, 1)]
    timed(step_graphs, warm)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    t0 = time.time()
    ms = timed(step_graphs, steps)
    t1 = time.time()
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    if failure.item() != 0:
        raise SystemExit("non-finite activation flagged during the benchmark")
    scale = n_layers / STREAM_LAYERS
    total_bytes = stream_step_bytes() * scale
    value = total_bytes * steps / (ms * 1e-3) / 1e9
    launches_per_step = len(tokens) * n_layers * (2 + len(SHAPES)) + (1 if fused else 0)

    # ---- the projection kernels alone, per token count (no quantiser, no cross-GPU wait inside the graph)
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    hbm_peak, peak_src = (peaks["hbm_gbs"], "measured") if "hbm_gbs" in peaks else (6650.0, "fallback")
    kernel_of = {1: "gemv_tma_kernel" if not args.no_overlap else "gemv_dp4a_kernel", 64: "mmq_tcgen05_kernel<64,64>"}
    by_tokens = {}
    for m in tokens:
        gk = [capture(lambda p=p, mm=m: stream_step(p, quantise=False, only_m=mm)) for p in (0, 1)]
        timed(gk, 2)
        reps = max(2, min(steps, 6))
        msk = timed(gk, reps)
        launches = n_layers * len(SHAPES)
        rank_bytes = n_layers * sum(weight_bytes(shard(n)[1], k) + m * (k + k // 32 * 8) + m * shard(n)[1] * 4 for _, n, k in SHAPES)
        by_tokens[m] = {"kernel": kernel_of[m], "avg_us": msk * 1e3 / (reps * launches), "ms_per_pass": msk / reps,
                        "GBps_per_gpu": rank_bytes * reps / (msk * 1e-3) / 1e9, "bytes_per_launch": rank_bytes / launches,
                        "launches_per_step": launches}
        del gk

    # ---- end to end: the step's activations arrive from pinned host memory (the copy for step s+1 is issued while
    # step s computes, into the other buffer), the step's result -- the gathered outputs as they stand after the
    # last layer -- goes back to pinned host memory and the step ends when that copy has landed.  Outputs alternate
    # between two buffers by step parity: a peer may already be storing step s+1 while this rank still copies step s.
    h_out = [torch.empty(out_group[0].shape, dtype=torch.float32).pin_memory() for _ in (0, 1)]

    def e2e_step(parity):
        main_stream = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(main_stream)
        copy_stream.wait_event(start)
        with torch.cuda.stream(copy_stream):
            x_pool[1 - parity].copy_(x_host, non_blocking=True)  # the next step's inputs
        stream_step(parity)
        ev = torch.cuda.Event()
        ev.record(main_stream)
        copy_stream.wait_event(ev)
        with torch.cuda.stream(copy_stream):
            if rank == 0:
                h_out[parity].copy_(out_group[parity], non_blocking=True)
        done = torch.cuda.Event()
        done.record(copy_stream)
        main_stream.wait_event(done)

    e2e_graphs = [capture(lambda p=p: e2e_step(p)) for p in (0, 1)]
    timed(e2e_graphs, warm)
    ms_e2e = timed(e2e_graphs, steps)
    e2e_value = total_bytes * steps / (ms_e2e * 1e-3) / 1e9
    e2e_checked = bool(torch.equal(h_out[(steps - 1) % 2], out_group[(steps - 1) % 2].cpu())) if rank == 0 else None
    del e2e_graphs

    extras = {}
    if rank == 0 and world == 1 and not args.no_extras:
        del step_graphs
        extras = single_gpu_extras(torch, lib, L, synth, dev, stream, g, failure, peaks, hbm_peak, capture, timed, args)

    if rank == 0:
        dom = max(by_tokens, key=lambda m: by_tokens[m]["ms_per_pass"])
        d = by_tokens[dom]
        traffic = None
        tpath = ROOT / "qw38_b200" / "measured_traffic.json"
        if tpath.exists():  # DRAM read+write of one captured launch over its algorithmic bytes, per kernel
            ratio = json.loads(tpath.read_text()).get(d["kernel"].split("<")[0], {}).get("dram_over_algorithmic")
            traffic = None if ratio is None else d["bytes_per_launch"] * ratio
        line = {"metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warm,
                "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "int8 dot / fp32 affine", "data": "synthetic",
                "config": {"workload": workload, "layers": n_layers, "tokens": tokens,
                           "l2": f"{n_layers} distinct layers ({total_bytes / 2e9:.1f} GB of weights) >> 126 MB L2",
                           "parallelism": f"rows/{world}" + (" + peer stores fused into the projection kernels, one bounded "
                                                                     "cross-GPU wait per step" if fused else ""),
                           "launch": ("eager" if args.no_graph else "CUDA graph replay, one graph per step") +
                                     ("" if args.no_overlap else ", programmatic dependent launch (every kernel of the step; projections flagged input_settled)"),
                           "bytes_per_step": total_bytes, "parity_check": checked},
                "clocks": clocks, "gpu_launches": launches_per_step * steps,
                "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": x_words * 2,
                        "d2h_bytes_per_step": out_words * 4, "ms_per_step": ms_e2e / steps, "result_matches_device": e2e_checked},
                "roofline": {"bound": "hbm", "kernel": d["kernel"], "tokens": dom, "achieved": d["GBps_per_gpu"], "peak": hbm_peak,
                             "unit": "GB/s", "frac": d["GBps_per_gpu"] / hbm_peak, "peak_source": peak_src, "per": "GPU",
                             "traffic": traffic, "avg_launch_us": d["avg_us"], "bytes_per_launch": d["bytes_per_launch"],
                             "by_tokens": {str(m): {"kernel": v["kernel"], "GBps_per_gpu": round(v["GBps_per_gpu"], 1),
                                                    "frac": round(v["GBps_per_gpu"] / hbm_peak, 4), "avg_us": round(v["avg_us"], 3),
                                                    "ms_per_pass": round(v["ms_per_pass"], 4), "launches_per_step": v["launches_per_step"]}
                                           for m, v in by_tokens.items()}}}
        line.update(extras)
        if not args.no_cpu and world == 1:
            gbps, cores, sample = cpu_sample(3)
            line["cpu_baseline"] = {"value": gbps, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample}
            line["cpu_baseline_reference_gemv"] = cpu_reference_gemv_sample()
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line))
    if world > 1:
        # Every collective of this process has completed (the timed regions end with a device synchronise).  Tearing
        # NCCL down with captured graphs still alive can block, so leave without it.
        torch.cuda.synchronize(dev)
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def verify_against_oracle(torch, dist, world, rank, last_layer, q8, outs, shard, tokens):
    """Sampled rows of the gathered outputs of the last layer against the CPU restatement (the checker, not the thing
    measured): each rank computes the reference for two 8-row groups of its own shard of every matrix, the references
    are exchanged, and every rank compares ALL of them with its own copy of the gathered output."""
    from oracle import oracle as orc
    mine = []
    for m in tokens:
        for i, (_, n, k) in enumerate(SHAPES):
            w = last_layer[i]
            row0, rows = shard(n)
            x = q8[(m, k)]
            z, a, s = x.codes.cpu().numpy(), x.scales.cpu().numpy(), x.sums.cpu().numpy()
            for r in sorted({0, (rows // 8 - 1) * 8}):
                ws = w.row_slice(r, 8)
                ref = orc.project_rows(ws.codes.cpu().numpy(), ws.scales.cpu().numpy(), 8, k, z, a, s, 0, 8)
                mine.append((m, i, row0 + r, ref))
    everyone = [mine]
    if world > 1:
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)
    worst, count = 0.0, 0
    for items in everyone:
        for (m, i, r, ref) in items:
            got = outs[(0, m, i)][:, r:r + 8].cpu().numpy()
            err = np.abs(got - ref)
            if not (err <= 0.02 + 0.002 * np.abs(ref)).all():
                raise SystemExit(f"rank {rank}: gathered output differs from the oracle at m={m}, matrix {i}, rows {r}..{r + 8}")
            worst = max(worst, float((err / np.maximum(np.abs(ref), 1e-3)).max()))
            count += ref.size
    return {"values": count, "ranks_checked": len(everyone), "tolerance": "0.02 + 0.002|ref|", "worst_rel": worst}


def single_gpu_extras(torch, lib, L, synth, dev, stream, g, failure, peaks, hbm_peak, capture, timed, args):
    from qw38_b200.q4k_q8 import (dequantize_bf16, new_q8_input, pack_q8, q4k_q8_project, q4k_q8_project_ragged,
                                  quantize_q4k_weight)
    out = {}
    # ---- config[1]: one projection set, M in {1,2,4,8,16}, 8 rotating layer copies (1.49 GB >> L2)
    layers = [[synth.device_weight(n, k, seed=5000 + 10 * l + i, device=dev) for i, (_, n, k) in enumerate(SHAPES)]
              for l in range(SET_LAYERS)]
    per_m = {}
    for m in SET_TOKENS:
        qs = {k: pack_q8(torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16), failure) for k in (5120, 17408)}
        os_ = [torch.empty((m, n), dtype=torch.float32, device=dev) for _, n, _ in SHAPES]

        def fn(mm=m, qs=qs, os_=os_):
            for layer in range(SET_LAYERS):
                for i, (_, n, k) in enumerate(SHAPES):
                    # the activations were packed before the graph: never the work of the launch before
                    q4k_q8_project(layers[layer][i], qs[k], out=os_[i], trusted=True, input_settled=not args.no_overlap)
        gm = [capture(fn)]
        timed(gm, 3)
        t = timed(gm, 10)
        per_m[str(m)] = round(set_bytes(m, quantise=False) * SET_LAYERS * 10 / (t * 1e-3) / 1e9, 1)
        del gm
    out["decode_GBps_by_tokens"] = per_m
    out["decode_set_frac_of_hbm_peak"] = {k: round(v / hbm_peak, 4) for k, v in per_m.items()}
    del layers

    # ---- int8 tensor peak of this device, measured with the prefill kernel's own MMA instruction
    tops, ms_ = ctypes.c_double(0), ctypes.c_double(0)
    burst = sustained = None
    if lib.q4k_measure_int8_peak(100_000, ctypes.byref(tops), ctypes.byref(ms_), ctypes.c_void_p(stream.cuda_stream)) == 0:
        burst = {"TOPS": tops.value, "ms": ms_.value}
    if lib.q4k_measure_int8_peak(6_000_000, ctypes.byref(tops), ctypes.byref(ms_), ctypes.c_void_p(stream.cuda_stream)) == 0:
        sustained = {"TOPS": tops.value, "ms": ms_.value}
    out["int8_peak"] = {"instruction": "tcgen05.mma kind::i8 M128 N256 K32, operands in shared memory", "burst": burst,
                        "sustained": sustained}
    int8_peak = burst["TOPS"] if burst else None

    # ---- config[2]: prefill shapes
    prefill = {}
    for (m, n, k) in [(512, 17408, 5120), (512, 5120, 17408), (2048, 17408, 5120), (2048, 5120, 17408), (8192, 17408, 5120)]:
        w = synth.device_weight(n, k, seed=99, device=dev)
        xq = pack_q8(torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16) * 0.5, failure)
        o = torch.empty((m, n), dtype=torch.float32, device=dev)
        with torch.cuda.stream(stream):
            for _ in range(3):
                q4k_q8_project(w, xq, out=o, trusted=True)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 10
            e0.record(stream)
            for _ in range(reps):
                q4k_q8_project(w, xq, out=o, trusted=True)
            e1.record(stream)
        stream.synchronize()
        t = e0.elapsed_time(e1) / reps
        tops_ = 2.0 * m * n * k / (t * 1e-3) / 1e12
        prefill[f"M{m}_N{n}_K{k}"] = {"ms": round(t, 4), "int8_TOPS": round(tops_, 1), "kernel": "mmq_tcgen05_kernel<128,128>",
                                      "frac_of_measured_int8_peak": None if not int8_peak else round(tops_ / int8_peak, 4),
                                      "frac_of_nominal_4500": round(tops_ / 4500.0, 4)}
        # comparator: the reference's other prefill route on this GPU, unpack to bf16 + library GEMM (a library path,
        # timed for context only)
        wb = dequantize_bf16(w)
        xb = (torch.randn((m, k), device=dev, generator=g) * 0.5).to(torch.bfloat16)
        with torch.cuda.stream(stream):
            for _ in range(3):
                torch.matmul(xb, wb.t())
            e0.record(stream)
            for _ in range(reps):
                torch.matmul(xb, wb.t())
            e1.record(stream)
        stream.synchronize()
        prefill[f"M{m}_N{n}_K{k}"]["bf16_library_gemm_ms"] = round(e0.elapsed_time(e1) / reps, 4)
        del wb, xb, w, o, xq
    # config[3]: packed ragged batch, 48 single-row requests + 512 + 237 + 1024 rows = 1821 rows
    offs = list(range(49)) + [560, 797, 1821]
    m, n, k = 1821, 34816, 5120
    w = synth.device_weight(n, k, seed=98, device=dev)
    xq = pack_q8(torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16) * 0.5, failure)
    o = torch.empty((m, n), dtype=torch.float32, device=dev)
    with torch.cuda.stream(stream):
        for _ in range(3):
            q4k_q8_project_ragged(w, xq, offs, out=o)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(10):
            q4k_q8_project_ragged(w, xq, offs, out=o)
        e1.record(stream)
    stream.synchronize()
    t = e0.elapsed_time(e1) / 10
    prefill["ragged_M1821_N34816_K5120"] = {"ms": round(t, 4), "int8_TOPS": round(2.0 * m * n * k / (t * 1e-3) / 1e12, 1),
                                            "kernel": "mmq_tcgen05_kernel<128,128>", "requests": len(offs) - 1}
    del w, o, xq
    out["prefill"] = prefill
    head = prefill["M2048_N17408_K5120"]
    out["prefill_roofline"] = {"bound": "tensor", "kernel": "mmq_tcgen05_kernel<128,128>", "workload": "config[2]: M=2048, N=17408, K=5120",
                               "achieved": head["int8_TOPS"], "peak": int8_peak, "unit": "TOP/s",
                               "frac": None if not int8_peak else head["int8_TOPS"] / int8_peak,
                               "peak_source": "measured" if int8_peak else "unavailable",
                               "ops": "2*M*N*K per launch; time by CUDA events over 10 launches"}

    # ---- offline step of the same path: bf16 weights -> split-tile Q4_K on the device, and back to bf16
    n, k = 5120, 17408
    wf = (torch.randn((n, k), device=dev, generator=g) * 0.02).to(torch.bfloat16)
    with torch.cuda.stream(stream):
        for _ in range(2):
            quantize_q4k_weight(wf, check=False)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(5):
            quantize_q4k_weight(wf, check=False)
        e1.record(stream)
    stream.synchronize()
    t = e0.elapsed_time(e1) / 5
    fitter = {"workload": f"fit bf16 {n}x{k} -> split-tile Q4_K", "ms": round(t, 3), "kernel": "fit_q4k_kernel",
              "Mblocks_per_s": round(n * k / 256 / (t * 1e-3) / 1e6, 1)}
    pw = quantize_q4k_weight(wf, check=False)
    del wf
    deq = torch.empty((n, k), dtype=torch.bfloat16, device=dev)
    ws = pw.c_struct()
    with torch.cuda.stream(stream):
        for _ in range(3):
            lib.q4k_dequantize_bf16(ctypes.byref(ws), ctypes.c_void_p(deq.data_ptr()), deq.numel(), ctypes.c_void_p(stream.cuda_stream))
        e0.record(stream)
        for _ in range(20):
            lib.q4k_dequantize_bf16(ctypes.byref(ws), ctypes.c_void_p(deq.data_ptr()), deq.numel(), ctypes.c_void_p(stream.cuda_stream))
        e1.record(stream)
    stream.synchronize()
    t = e0.elapsed_time(e1) / 20
    nbytes = pw.nbytes() + deq.numel() * 2
    fitter["dequantize_bf16"] = {"ms": round(t, 4), "kernel": "dequantize_bf16_kernel", "GBps": round(nbytes / (t * 1e-3) / 1e9, 1),
                                 "frac_of_hbm_peak": round(nbytes / (t * 1e-3) / 1e9 / hbm_peak, 4), "bytes": nbytes}
    out["fitter"] = fitter
    return out


if __name__ == "__main__":
    main()
