#!/usr/bin/env python
"""Benchmark of the Q4_K x Q8 decode hot path (and, as extra keys, of the prefill path).

Workload at every N: one hybrid-layer decode projection set (QKV 7168x5120, O 5120x5120,
gate+up 34816x5120, down 5120x17408, Q4_K weights, bf16 N(0,1) activations quantised on the
device) at M in {1,2,4,8,16}.  One step = the five token counts over one layer copy each;
weights rotate over LAYERS distinct copies (>126 MB L2) so HBM serves them.  With N>1 GPUs
every matrix is split by output rows over the ranks and the output slices are all-gathered.

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the reference
equation on the host cores instead (rank 0 only)."""
from __future__ import annotations

import argparse
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
TOKENS = [1, 2, 4, 8, 16]
LAYERS = 8
METRIC = "q4k_q8_decode_projection_set_GBps"


def weight_bytes(n, k):
    return n * (k // 256) * 144


def algorithmic_bytes(m, n, k, with_quantise=True):
    """Q4_K weights read once + Q8 activations (codes, fp32 scale, int32 sum) + fp32 output
    (+ the bf16 rows when the quantiser runs inside the timed region)."""
    b = weight_bytes(n, k) + m * (k + (k // 32) * 8) + m * n * 4
    return b + (m * k * 2 if with_quantise else 0)


def step_bytes():
    total = 0
    for m in TOKENS:
        for _, n, k in SHAPES:
            total += algorithmic_bytes(m, n, k, with_quantise=False)
        total += m * 5120 * 2 + m * 17408 * 2  # two bf16 inputs quantised per token count
    return total


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
WORKLOAD = ("config[1]: decode projection set QKV 7168x5120, O 5120x5120, gate+up 34816x5120, down 5120x17408, "
            "Q4_K weights, M in {1,2,4,8,16}, bf16 activations quantised on device")


def cpu_sample(repeats: int, rows_per_matrix: int = 256):
    """Times the CPU restatement on a bounded sample: `rows_per_matrix` output rows of every
    matrix of the set, all five token counts, all host cores.  Returns (GB/s, cores, text)."""
    from oracle import oracle as orc
    from qw38_b200 import synth
    handle = orc.lib(native=True)
    cores = handle.orc_num_threads()
    mats = []
    for i, (_, n, k) in enumerate(SHAPES):
        codes, meta = synth.logical_q4k(rows_per_matrix, k, seed=100 + i)
        mats.append((k,) + synth.split_tiles(codes, meta))
    acts = {}
    for m in TOKENS:
        for k in (5120, 17408):
            xb = synth.f32_to_bf16_bits(synth.activations(m, k, seed=m))
            acts[(m, k)] = orc.q8_quantize(xb, bf16_bits=True)[:3]
    nbytes = sum(algorithmic_bytes(m, rows_per_matrix, k, with_quantise=False) for m in TOKENS for _, _, k in SHAPES)
    best = float("inf")
    for _ in range(max(1, repeats)):
        t0 = time.perf_counter()
        for m in TOKENS:
            for (k, hc, hs) in mats:
                z, a, s = acts[(m, k)]
                orc.project_rows(hc, hs, rows_per_matrix, k, z, a, s, 0, rows_per_matrix, handle=handle)
        best = min(best, time.perf_counter() - t0)
    return nbytes / best / 1e9, cores, f"{rows_per_matrix} rows of each of the 4 matrices, M in {TOKENS}, best of {max(1, repeats)}"


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
# GPU arm
# ----------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill extra keys")
    ap.add_argument("--only", default="", help="debug / profiling: \"decode\" runs the device-resident timing only "
                                                "(no per-token-count pass, no end-to-end leg, no prefill extras)")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N > 1: projection kernels store into every rank's output over NVLink (fused), or "
                         "NCCL all-gather after each projection")
    ap.add_argument("--no-graph", action="store_true", help="debug / profiling: eager launches instead of CUDA graph replay")
    ap.add_argument("--no-overlap", action="store_true",
                    help="launch every kernel fully serialised (no programmatic dependent launch)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import torch.distributed as dist
    from qw38_b200 import _lib as L
    from qw38_b200 import synth
    from qw38_b200.q4k_q8 import (new_q8_input, pack_q8, peer_wait, q4k_q8_project, q4k_q8_project_gather,
                                  set_launch_overlap)
    from qw38_b200.sharding import symmetric_pool

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
    L.load()
    steps, warm = max(1, args.steps), max(3, args.warmup)

    # Row shard of every matrix: multiples of 8 rows (one row group is the unit of the layout).
    def shard(n):
        per = (n // 8 + world - 1) // world * 8
        r0 = min(n, rank * per)
        return r0, min(n, r0 + per) - r0, per

    layers = []
    for l in range(LAYERS):
        mats = []
        for i, (_, n, k) in enumerate(SHAPES):
            _, rows, _ = shard(n)
            mats.append(synth.device_weight(rows, k, seed=1000 * l + 10 * i + rank, device=dev))
        layers.append(mats)

    g = torch.Generator(device=dev)
    g.manual_seed(1234)
    x_in = {m: {k: torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16) for k in (5120, 17408)} for m in TOKENS}
    q8 = {m: {k: new_q8_input(m, k, dev) for k in (5120, 17408)} for m in TOKENS}
    failure = torch.zeros(1, dtype=torch.int32, device=dev)
    # Inputs and outputs are slices of one buffer each, ordered by token count, so that the end-to-end leg
    # moves a step's activations in one host->device copy and each token count's results in one device->host copy.
    x_pool = torch.empty(sum(m * (5120 + 17408) for m in TOKENS), dtype=torch.bfloat16, device=dev)
    off = 0
    for m in TOKENS:
        for k in (5120, 17408):
            view = x_pool[off:off + m * k].view(m, k)
            view.copy_(x_in[m][k])
            x_in[m][k] = view
            off += m * k
    outs, gathered, out_group = {}, {}, {}
    out_pool = torch.empty(sum(m * shard(n)[1] for m in TOKENS for _, n, _ in SHAPES), dtype=torch.float32, device=dev)
    off = 0
    for m in TOKENS:
        start = off
        for i, (_, n, k) in enumerate(SHAPES):
            _, rows, per = shard(n)
            if rows != per:
                raise SystemExit(f"{n} rows do not split evenly over {world} ranks in row groups of 8")
            outs[(m, i)] = out_pool[off:off + m * rows].view(m, rows)
            off += m * rows
            if world > 1:  # rank g's slice lands in gathered[g]; out[t, g*per + j] = gathered[g, t, j]
                gathered[(m, i)] = torch.empty((world * m, per), dtype=torch.float32, device=dev)
        out_group[m] = out_pool[start:off]

    # Fused gather: every rank's full [m, n] outputs and one arrival-counter array live in one symmetric
    # allocation, so each projection kernel can store its rows straight into every peer.
    fused = world > 1 and args.gather == "fused"
    full, full_ptrs, flag_ptrs, full_group = {}, {}, [], {}
    if fused:
        try:
            words = sum(m * n for m in TOKENS for _, n, _ in SHAPES) + 16
            pool, bases, pool_handle = symmetric_pool(words, dev)
            off = 0
            for m in TOKENS:
                start = off
                for i, (_, n, _) in enumerate(SHAPES):
                    full[(m, i)] = pool[off:off + m * n].view(m, n)
                    full_ptrs[(m, i)] = [b + 4 * off for b in bases]
                    off += m * n
                full_group[m] = pool[start:off]
            flag_ptrs = [b + 4 * off for b in bases]
        except Exception as exc:  # symmetric memory can be unavailable; the NCCL path still measures the shards
            fused = False
            print(f"[bench] symmetric memory unavailable ({type(exc).__name__}: {exc}); using NCCL all-gather", file=sys.stderr)
        ok = torch.tensor([1 if fused else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        fused = bool(ok.item())

    launches = {"n": 0}

    def projection(m, i, layer, count=True, force_nccl=False):
        _, n, k = SHAPES[i]
        if count:
            launches["n"] += 1
        if fused and not force_nccl:
            row0, _, _ = shard(n)
            q4k_q8_project_gather(layers[layer][i], q8[m][k], full_ptrs[(m, i)], flag_ptrs, rank, row0, n)
            return
        # the check of the fused path pins the kernel: automatic choice for one token depends on the overlap switch
        q4k_q8_project(layers[layer][i], q8[m][k], out=outs[(m, i)], trusted=True,
                       kernel=L.KERNEL_GEMV_TMA if force_nccl else L.KERNEL_AUTO)
        if world > 1:
            dist.all_gather_into_tensor(gathered[(m, i)], outs[(m, i)])

    def which_kernel(m, rows):
        """The library's own dispatch rule for m <= 16 and 16-byte aligned weights (csrc/abi.cu):
        the TMA-streamed kernel for two to sixteen tokens, and for one token too when launches overlap;
        dp4a for one token otherwise."""
        return "dp4a" if (m == 1 and args.no_overlap) else "tma"

    def one_step(step, count=True, quantise=True, only_kernel=None, after_group=None, largest_first=False, xin=None):
        # largest_first: the end-to-end leg runs the big token counts first, so that their device->host
        # copies overlap the remaining projections and only the smallest copy is left exposed at the end
        order = list(enumerate(TOKENS))
        for mi, m in (reversed(order) if largest_first else order):
            layer = (step * len(TOKENS) + mi) % LAYERS
            if quantise:
                for k in (5120, 17408):
                    pack_q8((xin or x_in)[m][k], failure, out=q8[m][k])
                    if count:
                        launches["n"] += 1
            for i in range(len(SHAPES)):
                if only_kernel and which_kernel(m, layers[layer][i].n) != only_kernel:
                    continue
                projection(m, i, layer, count)
            if after_group is not None:
                if fused:  # this token count's gathered rows are complete once every peer has delivered them
                    peer_wait(flag_ptrs, rank)
                after_group(m)
        if fused and after_group is None:
            # the step's outputs are complete on this rank once every peer has delivered as many projections
            peer_wait(flag_ptrs, rank)
            if count:
                launches["n"] += 1

    stream = torch.cuda.Stream(device=dev)
    copy_stream = torch.cuda.Stream(device=dev)

    def capture(fn, n_steps):
        """Capture n_steps consecutive steps (distinct layer rotation) into one graph."""
        with torch.cuda.stream(stream):
            for s in range(2):
                fn(s)
            torch.cuda.synchronize(dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for s in range(n_steps):
                    fn(s)
        return graph

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    def timed(graph, n_replays):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(n_replays):
                graph.replay()
            e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    if fused:
        # One untimed step both ways: the fused stores must reproduce the NCCL all-gather bit for bit.
        for m in TOKENS:
            for k in (5120, 17408):
                pack_q8(x_in[m][k], failure, out=q8[m][k])
            for i in range(len(SHAPES)):
                projection(m, i, 0, count=False)
        peer_wait(flag_ptrs, rank)
        torch.cuda.synchronize(dev)
        dist.barrier()
        for m in TOKENS:
            for i, (_, n, _) in enumerate(SHAPES):
                projection(m, i, 0, count=False, force_nccl=True)
                _, _, per = shard(n)
                want = gathered[(m, i)].view(world, m, per).permute(1, 0, 2).reshape(m, world * per)[:, :n]
                if not torch.equal(full[(m, i)], want):
                    raise SystemExit(f"fused gather differs from NCCL all-gather at m={m}, matrix {i}")
        torch.cuda.synchronize(dev)
        dist.barrier()

    # The weights are final from here on, which is what the overlapped launches require.
    torch.cuda.synchronize()
    set_launch_overlap(not args.no_overlap)

    # A graph holds UNROLL steps so that the LAYERS weight copies are all visited.
    UNROLL = LAYERS
    use_graph = not args.no_graph
    try:
        graph = capture(lambda s: one_step(s, count=False), UNROLL) if use_graph else None
    except Exception as exc:  # NCCL capture can be refused; fall back to eager launches
        if world == 1:
            raise
        use_graph = False
        print(f"[bench] graph capture unavailable ({type(exc).__name__}); timing eager launches", file=sys.stderr)

    class Eager:
        def __init__(self, fn, n):
            self.fn, self.n = fn, n

        def replay(self):
            for s in range(self.n):
                self.fn(s)

    if not use_graph:
        graph = Eager(lambda s: one_step(s, count=False), UNROLL)

    replays = max(1, (steps + UNROLL - 1) // UNROLL)
    steps = replays * UNROLL  # exactly this many steps are timed
    warm_replays = max(1, (warm + UNROLL - 1) // UNROLL)
    timed(graph, warm_replays)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    t0 = time.time()
    ms = timed(graph, replays)
    t1 = time.time()
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    launches_per_step = len(TOKENS) * (2 + len(SHAPES)) + (1 if fused else 0)
    total_bytes = step_bytes()
    value = total_bytes * steps / (ms * 1e-3) / 1e9
    if failure.item() != 0:
        raise SystemExit("non-finite activation flagged during the benchmark")

    extra = {}
    if rank == 0:
        peaks = {}
        pk_path = ROOT / "MEASURED_PEAKS.json"
        if pk_path.exists():
            peaks = json.loads(pk_path.read_text())
        hbm_peak, peak_src = (peaks["hbm_gbs"], "measured") if "hbm_gbs" in peaks else (6650.0, "fallback")
    # Per-kernel passes (all ranks take part so collectives match).
    per_kernel = {}
    for kern in ("dp4a", "tma"):
        pairs = [(m, i) for m in TOKENS for i in range(len(SHAPES)) if which_kernel(m, layers[0][i].n) == kern]
        if not pairs:
            continue
        fn = (lambda s, kk=kern: one_step(s, count=False, quantise=False, only_kernel=kk))
        gk = capture(fn, UNROLL) if use_graph else Eager(fn, UNROLL)
        timed(gk, warm_replays)
        msk = timed(gk, replays)
        n_launch = len(pairs) * steps
        bytes_k = sum(algorithmic_bytes(m, SHAPES[i][1], SHAPES[i][2], with_quantise=False) for m, i in pairs) * steps
        per_kernel[kern] = {"launches": n_launch, "avg_us": msk * 1e3 / n_launch, "GBps": bytes_k / (msk * 1e-3) / 1e9,
                            "ms": msk, "bytes_per_launch": bytes_k / n_launch}
    per_m = {}
    if world == 1 and not args.only:
        for m in TOKENS:
            def fn(s, mm=m):
                layer = s % LAYERS
                for i in range(len(SHAPES)):
                    projection(mm, i, layer, count=False)
            gm = capture(fn, UNROLL)
            timed(gm, 2)
            mm_ms = timed(gm, max(2, replays // 2))
            b = sum(algorithmic_bytes(m, n, k, with_quantise=False) for _, n, k in SHAPES) * UNROLL * max(2, replays // 2)
            per_m[str(m)] = round(b / (mm_ms * 1e-3) / 1e9, 1)

    # End to end: every step's activations arrive from pinned host memory in one copy, issued on a second
    # stream while the step before it computes (two device buffers alternate); each token count's results
    # leave in one copy on that stream as soon as they are complete, overlapping the next projections; a step
    # ends when its last result copy has landed.  With several GPUs every rank receives its inputs, each token
    # count gets its own cross-GPU wait so that its gathered rows can leave at once, and rank 0 alone reads
    # the (identical) result back.  (NCCL variant: one copy per gathered tensor, one stream.)
    pooled = fused or world == 1
    groups = full_group if fused else out_group
    h_x = x_pool.cpu().pin_memory()
    h_group = {m: torch.empty(t.shape, dtype=t.dtype).pin_memory() for m, t in groups.items()} if pooled else {}
    h_out = {} if pooled else {key: torch.empty(t.shape, dtype=t.dtype).pin_memory() for key, t in gathered.items()}
    x_pool_b = x_pool.clone()
    x_in_b, off = {}, 0
    for m in TOKENS:
        x_in_b[m] = {}
        for k in (5120, 17408):
            x_in_b[m][k] = x_pool_b[off:off + m * k].view(m, k)
            off += m * k
    x_sets = [(x_pool, x_in), (x_pool_b, x_in_b)]

    def e2e_step(s):
        main = torch.cuda.current_stream()
        if not pooled:
            x_pool.copy_(h_x, non_blocking=True)
            one_step(s, count=False)
            for key, t in gathered.items():
                h_out[key].copy_(t, non_blocking=True)
            return
        # the next step's inputs: into the buffer whose last readers (the step before this one) are done
        start = torch.cuda.Event()
        start.record(main)
        copy_stream.wait_event(start)
        with torch.cuda.stream(copy_stream):
            x_sets[(s + 1) % 2][0].copy_(h_x, non_blocking=True)

        def drain(m):  # the gathered result is read back once, by rank 0
            if rank != 0:
                return
            ev = torch.cuda.Event()
            ev.record(main)
            copy_stream.wait_event(ev)
            with torch.cuda.stream(copy_stream):
                h_group[m].copy_(groups[m], non_blocking=True)

        one_step(s, count=False, after_group=drain, largest_first=True, xin=x_sets[s % 2][1])
        done = torch.cuda.Event()
        done.record(copy_stream)
        main.wait_event(done)

    if args.only:  # debug / profiler runs of the device-resident part alone: no end-to-end number
        ms_e2e = float("nan")
    else:
        ge = capture(e2e_step, UNROLL) if use_graph else Eager(e2e_step, UNROLL)
        timed(ge, warm_replays)
        ms_e2e = timed(ge, replays)
    h2d = sum(m * (5120 + 17408) * 2 for m in TOKENS)
    d2h = sum(t.numel() * 4 for t in (h_group if pooled else h_out).values())
    e2e_value = total_bytes * steps / (ms_e2e * 1e-3) / 1e9

    prefill = None
    peaks_all = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    if world == 1 and not args.no_prefill and not args.only:
        prefill = {}
        for (m, n, k) in [(512, 17408, 5120), (512, 5120, 17408), (2048, 17408, 5120), (8192, 17408, 5120)]:
            w = synth.device_weight(n, k, seed=99, device=dev)
            xq = pack_q8(torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16) * 0.5, failure)
            out = torch.empty((m, n), dtype=torch.float32, device=dev)
            with torch.cuda.stream(stream):
                for _ in range(3):
                    q4k_q8_project(w, xq, out=out, trusted=True)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = 10
                e0.record(stream)
                for _ in range(reps):
                    q4k_q8_project(w, xq, out=out, trusted=True)
                e1.record(stream)
            stream.synchronize()
            t = e0.elapsed_time(e1) / reps
            tops = 2.0 * m * n * k / (t * 1e-3) / 1e12
            int8_peak = 2.0 * peaks_all.get("bf16_tflops", 1590.0)  # int8 dense nominal = 2x bf16; bf16 burst is measured
            prefill[f"M{m}_N{n}_K{k}"] = {"ms": round(t, 4), "int8_TOPS": round(tops, 1), "kernel": "mmq_tcgen05_kernel",
                                          "frac_of_2x_measured_bf16": round(tops / int8_peak, 4),
                                          "frac_of_nominal_4500": round(tops / 4500.0, 4)}
            # comparator: the reference's other prefill route on this GPU, unpack to bf16 (timed under "fitter") + library GEMM
            from qw38_b200.q4k_q8 import dequantize_bf16
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
            del wb, xb
            del w, out, xq
        # config[3]: packed ragged batch, 48 single-row requests + 512 + 237 + 1024 rows = 1821 rows
        from qw38_b200.q4k_q8 import q4k_q8_project_ragged
        offs = list(range(49)) + [560, 797, 1821]
        m, n, k = 1821, 34816, 5120
        w = synth.device_weight(n, k, seed=98, device=dev)
        xq = pack_q8(torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16) * 0.5, failure)
        out = torch.empty((m, n), dtype=torch.float32, device=dev)
        with torch.cuda.stream(stream):
            for _ in range(3):
                q4k_q8_project_ragged(w, xq, offs, out=out)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(10):
                q4k_q8_project_ragged(w, xq, offs, out=out)
            e1.record(stream)
        stream.synchronize()
        t = e0.elapsed_time(e1) / 10
        prefill["ragged_M1821_N34816_K5120"] = {"ms": round(t, 4), "int8_TOPS": round(2.0 * m * n * k / (t * 1e-3) / 1e12, 1),
                                                "kernel": "mmq_tcgen05_kernel", "requests": len(offs) - 1}
        del w, out, xq

    fitter = None
    if world == 1 and not args.no_prefill and not args.only:
        # Offline step of the same path: bf16 weights -> split-tile Q4_K on the device (the reference fits on the host).
        from qw38_b200.q4k_q8 import quantize_q4k_weight
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
        # and back: resident split tiles -> bf16 [n, k] (the operand of the reference's unpack -> cuBLAS prefill path)
        import ctypes
        from qw38_b200 import _lib as L
        pw = quantize_q4k_weight(wf, check=False)
        del wf
        deq = torch.empty((n, k), dtype=torch.bfloat16, device=dev)
        ws = pw.c_struct()
        lib = L.load()
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
        del pw, deq

    if rank == 0:
        dom = max(per_kernel, key=lambda kk: per_kernel[kk]["ms"])
        pkk = per_kernel[dom]
        achieved = pkk["GBps"]
        kernel_name = {"dp4a": "gemv_dp4a_kernel", "tma": "gemv_tma_kernel"}[dom]
        line = {"metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warm_replays * UNROLL,
                "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "int8 dot / fp32 affine", "data": "synthetic",
                "config": {"workload": WORKLOAD,
                           "layers_rotated": LAYERS, "l2": f"weights rotate over {LAYERS} layer copies (1.49 GB) > 126 MB L2",
                           "parallelism": f"rows/{world}" + ((" + peer stores fused into the projection kernel, one bounded "
                                                                     "cross-GPU wait per step") if fused else
                                                                    (" + NCCL all-gather" if world > 1 else "")),
                           "launch": ("CUDA graph replay" if use_graph else "eager") +
                                     ("" if args.no_overlap else ", programmatic dependent launch"),
                           "bytes_per_step": total_bytes},
                "clocks": clocks, "gpu_launches": launches_per_step * steps,
                "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": ms_e2e / steps},
                "roofline": {"bound": "hbm", "kernel": kernel_name, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                             "frac": achieved / hbm_peak, "peak_source": peak_src,
                             # DRAM read+write of one launch = algorithmic bytes x the ratio measured by ncu on the
                             # 34816x5120 captures under profiles/ (1.06 TMA kernel at M=8, 1.03 dp4a at M=1)
                             "traffic": pkk["bytes_per_launch"] * (1.06 if dom == "tma" else 1.03),
                             "avg_launch_us": pkk["avg_us"], "bytes_per_launch": pkk["bytes_per_launch"],
                             "by_kernel": {kk: {"GBps": round(v["GBps"], 1), "frac": round(v["GBps"] / hbm_peak, 4),
                                                "avg_us": round(v["avg_us"], 3), "launches": v["launches"]}
                                           for kk, v in per_kernel.items()}},
                "decode_GBps_by_tokens": per_m, "prefill": prefill, "fitter": fitter}
        if not args.no_cpu and world == 1:
            gbps, cores, sample = cpu_sample(3)
            line["cpu_baseline"] = {"value": gbps, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line))
    if world > 1:
        # Every collective of this process has completed (the timed regions end with a device
        # synchronise).  Tearing NCCL down with captured graphs still alive can block, so leave
        # without it.
        torch.cuda.synchronize(dev)
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
