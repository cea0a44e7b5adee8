#!/usr/bin/env python
"""Benchmark of the sampling hot path: sampled edges/s, device-timed.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2] [--mode tp_lb]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A "step" is one sample() pass over the whole batch of samples.  Default workload (one GPU):
node2vec p=2 q=0.5, length 100, one walk per vertex, on a synthetic R-MAT graph with 2^20
vertices and 16M undirected edges (seed 0, generated on the device), transit-parallel mode with
load balancing.  With N ranks every rank holds a replica of the graph and samples its own range
of seeds (weak scaling: rank r owns the samples [r*S, (r+1)*S)); no collective is on the data
path, the final all-gather is timed separately.

Prints ONE JSON line (rank 0).  --impl reference times the reference's own next() bodies on the
host cores (oracle/_ref, else the oracle port) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WALK, KHOP, COLL = "walk", "khop", "collective"
WORKLOADS = {
    "c1": dict(kind=WALK, app=0, V=56944, M=400_000, steps=100, desc="uniform walk, length 100, one walk per vertex, 56,944 vertices, ~800K CSR entries"),
    "c2": dict(kind=WALK, app=3, V=1 << 20, M=1 << 24, steps=100, desc="node2vec p=2 q=0.5, length 100, one walk per vertex, 2^20 vertices, 16M undirected edges"),
    "c2u": dict(kind=WALK, app=0, V=1 << 20, M=1 << 24, steps=100, desc="uniform walk on the c2 graph"),
    "c2d": dict(kind=WALK, app=1, V=1 << 20, M=1 << 24, steps=100, desc="DeepWalk (weighted rejection) on the c2 graph"),
    "c3": dict(kind=KHOP, app=5, V=1 << 21, M=1 << 25, fanout=[25, 10], S=256 * 1024,
               desc="GraphSAGE 2-hop, fan-out 25 then 10 without replacement + distinct, 256 batches of 1024 uniform seeds, 2^21 vertices, 32M undirected edges"),
    "c3r": dict(kind=KHOP, app=4, V=1 << 21, M=1 << 25, fanout=[25, 10], S=256 * 1024,
                desc="k-hop with replacement (the reference's KHopApp) on the c3 graph and seeds"),
    "c3rv": dict(kind=KHOP, app=4, V=1 << 21, M=1 << 25, fanout=[25, 10], S=1 << 21,
                 desc="k-hop with replacement, one sample per vertex (the shape of the reference's KHopApp::numSamples) on the c3 graph"),
    "c4f": dict(kind=COLL, app=8, V=1 << 20, M=1 << 24, steps=2, L=64, B=64, S=1024,
                desc="FastGCN importance sampling (degree^2), 2 layers x 64, 1024 batches of 64 uniform seeds, 2^20 vertices, 16M undirected edges"),
    "c4l": dict(kind=COLL, app=9, V=1 << 20, M=1 << 24, steps=2, L=64, B=64, S=1024,
                desc="LADIES importance sampling (squared row-normalised weights), 2 layers x 64, 1024 batches of 64 uniform seeds, c4 graph"),
    "c5": dict(kind=WALK, app=2, V=1 << 24, M=1 << 28, steps=100, stop_prob=0.15, desc="weighted PPR, stop probability 0.15, max length 100, one walk per vertex, 2^24 vertices, 256M undirected edges"),
    "c5s": dict(kind=WALK, app=2, V=1 << 22, M=1 << 26, steps=100, stop_prob=0.15, desc="weighted PPR stop 0.15 on 2^22 vertices, 64M undirected edges"),
}
APP_NAMES = {0: "uniform_walk", 1: "deepwalk", 2: "ppr", 3: "node2vec", 4: "khop", 5: "khop_distinct", 8: "fastgcn_is", 9: "ladies_is"}
MODES = {"tp": 0, "tp_lb": 1, "sp": 2}
E2E_CHUNKS = 1   # the per-step kernels are latency-bound at these sizes: cutting a job costs more than it gains;
E2E_DEPTH = 2    # instead two sampler sets alternate, so a job's result copy runs under the next job's sampling


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """nvidia-smi clocks and throttle reasons during the timed region."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.rows, self.stop_flag = index, [], False

    def run(self):
        while not self.stop_flag:
            try:
                r = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits"],
                                   capture_output=True, text=True, timeout=5)
                if r.returncode == 0 and r.stdout.strip():
                    self.rows.append([x.strip() for x in r.stdout.strip().split(",")])
            except Exception:
                pass
            time.sleep(0.1)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        sm = sorted(int(float(r[0])) for r in self.rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": int(float(self.rows[0][1])), "reasons": reasons,
                "samples": len(self.rows)}


def params_for(mod, wl, seed):
    """AppParams (product) or oracle Params for a workload; `mod` is nextdoor_b200.api or oracle.ndo."""
    make = mod.app_params if hasattr(mod, "app_params") else mod.make_params
    if wl["kind"] == WALK:
        return make(wl["app"], steps=wl["steps"], seed=seed, stop_prob=wl.get("stop_prob", 0.01))
    if wl["kind"] == KHOP:
        return make(wl["app"], fanout=wl["fanout"], seed=seed)
    return make(wl["app"], steps=wl["steps"], fanout=wl["L"], batch=wl["B"], seed=seed)


def seeds_for(wl, first, S):
    """Initial transits of samples [first, first+S): walks start sample i at vertex i % V; k-hop and
    collective batches draw their seeds uniformly (numpy Philox stream keyed by the sample range)."""
    V = wl["V"]
    if wl["kind"] == WALK:
        return (np.arange(first, first + S, dtype=np.int64) % V).astype(np.int32)
    per = 1 if wl["kind"] == KHOP else wl["B"]
    rng = np.random.Generator(np.random.Philox(key=first + 1))
    return rng.integers(0, V, S * per, dtype=np.int64).astype(np.int32)


def next_bytes(wl, st, mode):
    """Algorithmic bytes of the next() launches of one sample(), from the device's event counters.
    Walks: per live pair 8 B map-in + 8 B row offsets, per sampled edge 4 B neighbour + 4 B output,
    8 B map-out per pair of every step but the last (no maps in sample-parallel mode); weighted
    apps + 4 B max weight per next() and 4 B per weight read; node2vec + previous vertex (4+4 B,
    kept in a register in sample-parallel mode), 8 B for its row, and per try 4 B candidate + 4 B per
    word read by the membership test (one 8-id bucket of the previous vertex's neighbour set = 32 B;
    tests the draw decides without are not made and not counted).  k-hop: per pair 8 B map-in + 8 B row offsets, per neighbour 4 B + 4 B,
    8 B map-out per neighbour of every hop but the last.  Collective: 4 B per gathered neighbour id
    (+4 B weight for LADIES), 8 B per unique candidate, 8 B per sampled vertex."""
    pairs, edges = st["live_pairs"], st["sampled_edges"]
    app = wl["app"]
    if wl["kind"] == WALK:
        steps = wl["steps"]
        b = 8 * pairs + 8 * edges
        if mode != 2:
            b += 8 * pairs + 8 * pairs * (steps - 1) / steps
        if app in (1, 2):
            b += 4 * pairs + 4 * st["weight_tries"]
        if app == 3:
            b += (16 if mode != 2 else 8) * pairs + 4 * st["n2v_tries"] + 4 * st["n2v_probes"]
        return b
    if wl["kind"] == KHOP:
        f = wl["fanout"]
        last_share = 1.0  # neighbours of the last hop carry no map-out
        n, tot = 1, 0
        for k in f:
            n *= k
            tot += n
        last_share = n / tot
        return (16 if mode != 2 else 8) * pairs + 8 * edges + (8 * edges * (1 - last_share) if mode != 2 else 0)
    return (8 if app == 9 else 4) * st["union_ids"] + 8 * st["union_unique"] + 8 * edges


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the next() kernel, from the ncu captures
# summarised under profiles/ (bytes; same workload and mode, warm caches)
NCU_TRAFFIC = {("c2", "tp_lb"): 167.4e6}


def gather_ceiling(wl, st, g, next_ms, next_launches, device):
    """The second ceiling of the walk kernels, measured live: next() is a few independent random
    4-byte gathers into the graph arrays per pair, and a GPU serves those at a rate set by the
    arrays' footprint against the L2 (nd_probe_random_gather), far below the copy bandwidth that
    `peak` is.  graph_gathers = the gathers into graph-sized arrays one pass needs (uniform walk:
    one neighbour id per edge; weighted: one (id, weight) record per try; node2vec: one candidate
    per try + one set bucket per membership test), floor = graph_gathers / rate."""
    import ctypes as C
    from nextdoor_b200._lib import lib, check
    app = wl["app"]
    if app == 0:
        gathers, footprint = st["sampled_edges"], 4 * g.E
    elif app in (1, 2):
        gathers, footprint = st["weight_tries"], 8 * g.E
    else:
        gathers, footprint = st["n2v_tries"] + st["n2v_probes"] // 8, 12 * g.E
    per_launch = max(int(gathers / max(next_launches, 1)), 1)
    rate = C.c_double(0.0)
    check(lib.nd_probe_random_gather(device, int(footprint), 1 << 24, 3, C.byref(rate)))
    small = C.c_double(0.0)   # the same at the size of one launch: fixed launch and ramp costs included
    check(lib.nd_probe_random_gather(device, int(footprint), per_launch, 20, C.byref(small)))
    floor_ms = gathers / rate.value * 1e3
    return {"footprint_bytes": int(footprint), "rate_gathers_per_s": rate.value,
            "rate_at_launch_size": small.value, "graph_gathers_per_pass": int(gathers),
            "floor_ms_per_pass": floor_ms, "frac": floor_ms / next_ms if next_ms > 0 else None,
            "note": "frac = time the pass's graph gathers take at the measured random-gather rate / next() time"}


def cpu_baseline(hg, wl, seed, budget_s=12.0):
    """The reference's own next() bodies (oracle/_ref) where they exist for the workload, else the
    oracle port, on all host threads, on a bounded prefix of the workload's samples."""
    from oracle import ndo
    app = wl["app"]
    use_ref = ndo.ref_available() and wl["kind"] == WALK and not (app == 2 and abs(wl.get("stop_prob", 0.01) - 0.01) > 1e-9)
    use_ref = use_ref or (ndo.ref_available() and app == 4 and wl["fanout"] == [25, 10])
    pr = params_for(ndo, wl, seed)
    # all host cores this process may run on, set explicitly: launchers such as torchrun export
    # OMP_NUM_THREADS=1 to their ranks, which would silently make this a one-thread baseline
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    S_all = wl.get("S", wl["V"])

    def run(n):
        init = seeds_for(wl, 0, n)
        t0 = time.perf_counter()
        if use_ref:
            e = ndo.ref_sample(hg, app, pr.steps, n, seed=seed, initial=init, threads=threads)["sampled_edges"]
        else:
            e = ndo.sample(hg, pr, n, initial=init, want_adj=False, threads=threads)["counters"]["sampled_edges"]
        return e, time.perf_counter() - t0

    n = max(1, min(S_all, 20000 if wl["kind"] == WALK else (2000 if wl["kind"] == KHOP else 8)))
    e, t = run(n)
    n2 = int(min(S_all, max(n, n * budget_s / max(t, 1e-3))))
    if n2 > 2 * n:
        n = n2
        e, t = run(n)
    return {"value": e / t, "unit": "sampled edges/s", "cores": int(threads), "kind": "reference" if use_ref else "port",
            "sample": f"first {n} of {S_all} samples, {t:.2f} s", "seconds": t}


def partitioned_bench(a, wl, nd, torch, rank, world, local, seed):
    """Strong-scaling figure of the partitioned path: the workload's walks over a graph whose rows
    are split across the ranks (each GPU holds 1/N of the CSR entries), walkers routed by
    all-to-all every step.  Device-timed, max over ranks."""
    import torch.distributed as dist
    from nextdoor_b200 import partitioned as ndp
    V, S = wl["V"], wl.get("S", wl["V"])
    g = nd.Graph.rmat(V, wl["M"], seed, device=local)
    row_ptr, col, w, _ = g.to_host()
    E = int(g.E)
    del g
    bounds = ndp.split_bounds(row_ptr, world)
    rp, lc, lw = ndp.local_rows(row_ptr, col, w, int(bounds[rank]), int(bounds[rank + 1]))
    pr = params_for(nd, wl, seed)
    walker = ndp.PartitionedWalker(rp, lc, lw, bounds, pr, device=f"cuda:{local}")
    for _ in range(max(a.warmup, 2)):
        out, _ = walker.run(S)
        edges = int((out != V).sum())
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    walker.bytes_sent = 0
    e0.record()
    for _ in range(a.steps):
        out, _ = walker.run(S)
    e1.record()
    torch.cuda.synchronize()
    edges = int((out != V).sum())
    t = torch.tensor([e0.elapsed_time(e1), float(edges), float(walker.bytes_sent)], dtype=torch.float64, device="cuda")
    if world > 1:
        tm = t.clone()
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        t[0] = tm[0]
    if rank == 0:
        ms = float(t[0]) / a.steps
        print(json.dumps({"metric": "sampled edges/sec", "path": "partitioned graph", "value": float(t[1]) / (ms * 1e-3),
                          "unit": "sampled edges/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms,
                          "scaling": "strong", "config": {"workload": f"{a.workload}: {wl['desc']}",
                                                          "csr_entries_per_gpu": [int(row_ptr[bounds[r + 1]] - row_ptr[bounds[r]]) for r in range(world)],
                                                          "csr_entries": E},
                          "all_to_all_bytes_per_step": float(t[2]) / a.steps}))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default="c2", choices=list(WORKLOADS))
    ap.add_argument("--mode", default="tp_lb", choices=list(MODES))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--partitioned", action="store_true",
                    help="walk over the graph PARTITIONED across the ranks (nextdoor_b200.partitioned) instead of replicated; "
                         "walk workloads without node2vec; prints its own JSON line")
    ap.add_argument("--profile-only", action="store_true",
                    help="build the graph, run warmup+steps passes of sample() and exit (short launch list for ncu)")
    a = ap.parse_args()
    wl = WORKLOADS[a.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    seed = 0
    hbm_peak, peak_kind = peaks()
    V, M, app = wl["V"], wl["M"], wl["app"]
    S = wl.get("S", V)

    if a.impl == "reference":
        if rank != 0:
            return
        from oracle import ndo
        t0 = time.perf_counter()
        hg = ndo.rmat_graph(V, M, seed)      # same generator definition as the device one
        t_graph = time.perf_counter() - t0
        vals = []
        for i in range(a.warmup + a.steps):
            cb = cpu_baseline(hg, wl, seed, budget_s=6.0)
            if i >= a.warmup:
                vals.append(cb)
        v = float(np.mean([c["value"] for c in vals]))
        cb = dict(vals[-1], value=v)
        print(json.dumps({
            "impl": "reference", "metric": "sampled edges/sec", "value": v, "unit": "sampled edges/s", "n_gpus": a.gpus,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": 1e3 * float(np.mean([c["seconds"] for c in vals])),
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int32", "data": "synthetic",
            "config": {"workload": f"{a.workload}: {wl['desc']}", "host_graph_build_s": round(t_graph, 2)},
            "cpu_baseline": cb, "e2e": {"value": v, "unit": "sampled edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    import torch
    from nextdoor_b200 import api as nd
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if a.partitioned:
        return partitioned_bench(a, wl, nd, torch, rank, world, local, seed)
    mode = MODES[a.mode]
    g = nd.Graph.rmat(V, M, seed, device=local)
    pr = params_for(nd, wl, seed)
    first = rank * S
    init_np = seeds_for(wl, first, S)
    smp = nd.Sampler(g, pr, num_samples=S, first_sample=first, initial=init_np)
    fs = smp.fs
    stream = torch.cuda.Stream()          # a non-default stream, so the library can replay its CUDA graph
    torch.cuda.set_stream(stream)
    smp.set_stream(stream.cuda_stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if a.profile_only:
        for _ in range(a.warmup + a.steps):
            smp.sample(mode, sync=False)
        barrier()
        print(json.dumps({"profile_only": True, "workload": a.workload, "mode": a.mode, "stats": smp.stats()}))
        return

    # ---- device-timed throughput (inputs resident)
    for _ in range(a.warmup):
        smp.sample(mode, sync=False)
    barrier()
    clocks = ClockSampler(local)
    clocks.start()
    l0 = nd.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(a.steps):
        smp.sample(mode, sync=False)
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    launches = nd.launch_count() - l0
    edges_step = smp.stats()["sampled_edges"]

    # ---- the same job in the reference's other kernel type (-k SampleParallel), for comparison
    ms_sp = None
    if mode != 2:
        for _ in range(2):
            smp.sample(2, sync=False)
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record(stream)
        for _ in range(a.steps):
            smp.sample(2, sync=False)
        s1.record(stream)
        barrier()
        ms_sp = s0.elapsed_time(s1)

    # ---- end to end through the public API with host buffers: seeds H2D from pinned memory,
    # sample, result D2H into pinned memory, through nextdoor_b200.api.PipelinedSampler: the result of a
    # step is copied on a second stream while the next step is sampled (two sampler sets alternate).
    init_host = torch.from_numpy(init_np).pin_memory()
    out_host = torch.empty(S * fs, dtype=torch.int32).pin_memory()
    out_host2 = torch.empty(S * fs, dtype=torch.int32).pin_memory()   # consecutive steps land in alternating buffers
    init_pin, out_pin, out_pin2 = init_host.numpy(), out_host.numpy(), out_host2.numpy()
    copy_stream = torch.cuda.Stream()
    pipe = nd.PipelinedSampler(g, pr, S, first_sample=first, initial=init_np, chunks=E2E_CHUNKS, depth=E2E_DEPTH,
                               stream=stream.cuda_stream, copy_stream=copy_stream.cuda_stream)
    # walks: in the sample-parallel mode, the one the reference's Python sample() runs (src/nextDoorPythonModule.cu:54-58)
    e2e_mode = 2 if wl["kind"] == WALK else mode
    for _ in range(2):
        pipe.run(init_pin, out_pin, e2e_mode)
    barrier()
    x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    x0.record(stream)
    for i in range(a.steps):                  # step i+1 starts sampling while the tail of step i is being copied
        pipe.run_async(init_pin, out_pin if i % 2 == 0 else out_pin2, e2e_mode)
    pipe.wait()                               # every step's result has landed on the host
    x1.record(stream)
    barrier()
    if a.steps % 2 == 0:
        out_pin = out_pin2                    # the buffer the last step wrote
    clocks.stop_flag = True
    ms_e2e = x0.elapsed_time(x1)
    e2e_check = int((out_pin != V).sum()) if wl["kind"] != COLL else None
    pipe.free()

    # ---- the final sample gather (the only step that crosses NVLink): sample() + NCCL all-gather
    ms_gather = None
    if world > 1:
        # two samplers alternate: the all-gather of a step's samples runs on NCCL's stream while the
        # next step is sampled; a sampler's next run waits for the gather that still reads its buffer
        from nextdoor_b200 import dist as nd_dist
        smp2 = nd.Sampler(g, pr, num_samples=S, first_sample=first, initial=init_np)
        smp2.set_stream(stream.cuda_stream)
        pair = [(smp, nd_dist.device_samples(smp)), (smp2, nd_dist.device_samples(smp2))]
        # (two gathered arrays; when they would not fit comfortably -- the 2^24-vertex workload on 8 GPUs
        # gathers 54 GB -- one array is used and a gather waits for the previous one: less overlap)
        n_full = 2 if 2 * world * S * fs * 4 < (48 << 30) else 1
        fulls = [torch.empty((world * S, fs), dtype=torch.int32, device="cuda") for _ in range(n_full)]
        side = torch.cuda.Stream()
        pending = [None, None]

        def gather_step(i):
            k = i % 2
            s_k, shard_k = pair[k]
            if pending[k] is not None:
                pending[k].wait()
            s_k.sample(mode, sync=False)
            ev = torch.cuda.Event()
            ev.record(stream)
            if n_full == 1 and pending[k ^ 1] is not None:
                pending[k ^ 1].wait()          # the single gathered array is still being written
            with torch.cuda.stream(side):
                side.wait_event(ev)
                pending[k] = dist.all_gather_into_tensor(fulls[k % n_full], shard_k, async_op=True)

        def gather_drain():
            for k in range(2):
                if pending[k] is not None:
                    pending[k].wait()
                    pending[k] = None

        for i in range(2):
            gather_step(i)
        gather_drain()
        barrier()
        y0, y1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        y0.record(stream)
        for i in range(a.steps):
            gather_step(i)
        gather_drain()
        y1.record(stream)
        barrier()
        ms_gather = y0.elapsed_time(y1)
        gather_ok = bool((fulls[((a.steps - 1) % 2) % n_full][rank * S:(rank + 1) * S] == pair[(a.steps - 1) % 2][1]).all())
        assert gather_ok, "the gathered array does not hold this rank's shard"
        del fulls
        smp2.free()

    # ---- per-phase device time of one instrumented pass (roofline of the next() kernels)
    smp.set_profiling(True)
    smp.sample(mode)
    ph = smp.phase_ms()
    smp.set_profiling(False)
    st = smp.stats()

    tms = torch.tensor([ms, ms_e2e, ms_gather or 0.0, ms_sp or 0.0], dtype=torch.float64, device="cuda")
    tot = torch.tensor([float(edges_step)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    ms, ms_e2e, ms_gather, ms_sp = float(tms[0]), float(tms[1]), float(tms[2]), float(tms[3])
    total_edges = float(tot[0])

    if rank == 0:
        nb = next_bytes(wl, st, mode)
        next_ms, next_launches = ph["next"] if wl["kind"] != COLL else (ph["next"][0] + ph["collect"][0], ph["next"][1] + ph["collect"][1])
        achieved = nb / (next_ms * 1e-3) / 1e9 if next_ms > 0 else 0.0
        kernel = {WALK: {0: "walk_next_tp_kernel", 1: "walk_next_count_kernel", 2: "walk_sp_kernel"}[mode],
                  KHOP: "khop_pairs_kernel + khop_staged_kernel" if mode == 1 else "khop_pairs_kernel",
                  COLL: "coll_gather/sort/weigh/sample kernels"}[wl["kind"]]
        kernel = kernel if wl["kind"] != COLL else "coll_bitmap_kernel"
        gather = gather_ceiling(wl, st, g, next_ms, next_launches, torch.cuda.current_device()) if wl["kind"] == WALK else None
        cb = None
        if world == 1 and not a.no_cpu_baseline:
            from oracle import ndo
            row_ptr, col, w, mw = g.to_host()
            cb = cpu_baseline(ndo.HostGraph(row_ptr, col, w, mw), wl, seed)
        line = {
            "metric": "sampled edges/sec", "value": total_edges * a.steps / (ms * 1e-3), "unit": "sampled edges/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int32", "data": "synthetic",
            "config": {"workload": f"{a.workload}: {wl['desc']}", "app": APP_NAMES[app], "mode": a.mode,
                       "samples_per_gpu": S, "final_sample_size": fs,
                       "graph": f"R-MAT a=.57 b=.19 c=.19 d=.05 seed 0, V={V}, CSR entries={g.E}, max degree={g.max_degree}",
                       "l2": "working set (graph + sample buffers) larger than L2; no flush between steps",
                       "sampled_edges_per_step_per_gpu": edges_step},
            "e2e": {"value": total_edges * a.steps / (ms_e2e * 1e-3), "unit": "sampled edges/s",
                    "h2d_bytes_per_step": int(init_np.nbytes), "d2h_bytes_per_step": int(S * fs * 4),
                    "chunks": E2E_CHUNKS, "depth": E2E_DEPTH, "mode": {0: "tp", 1: "tp_lb", 2: "sp"}[e2e_mode], "valid_vertices_in_host_result": e2e_check},
            "gpu_launches": int(launches),
            "sample_parallel": None if mode == 2 else {"value": total_edges * a.steps / (ms_sp * 1e-3), "unit": "sampled edges/s",
                                                       "note": "same sampler, same samples, nd_mode SampleParallel"},
            "with_gather": None if world == 1 else {
                "value": total_edges * a.steps / (ms_gather * 1e-3), "unit": "sampled edges/s",
                "collective": "ncclAllGather of the final samples, overlapped with the next step's sampling (two samplers alternate)", "bytes_per_rank_per_step": int(S * fs * 4)},
            "roofline": {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "peak_kind": f"of {peak_kind}",
                         "traffic": NCU_TRAFFIC.get((a.workload, a.mode)),
                         "launches": next_launches, "avg_launch_us": 1e3 * next_ms / max(next_launches, 1),
                         "algorithmic_bytes_per_pass": nb, "random_gather": gather},
            "phases_ms": {k: round(v[0], 4) for k, v in ph.items()},
            "counters": st,
            "cpu_baseline": cb,
            "clocks": clocks.summary(),
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
