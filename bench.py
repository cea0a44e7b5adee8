#!/usr/bin/env python
"""Benchmark of the sampling hot path: sampled edges/s, device-timed.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c5] [--mode tp_lb]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A "step" is one sample() pass over the whole job.  Default workload: weighted PPR, stop
probability 0.15, maximum length 100, one walk per vertex, on a synthetic R-MAT graph with 2^24
vertices and 256M undirected edges (seed 0, generated on the device), transit-parallel mode with
load balancing.  With N ranks every rank holds a replica of the graph and ONE job is cut into
contiguous seed ranges by the reference's rule (PartStartPointer / PartDivisionSize,
src/utils.hpp:26-27; used at src/nextdoor.cu:2024-2025, 3221-3222): strong scaling, the draws are
keyed by the global sample index, so the concatenated shards equal the 1-GPU output.  No collective
is on the sampling path; the gather of the final samples to rank 0 is timed separately
(`with_gather`).  Next to the main workload a short node2vec pass on the 2^20-vertex graph (workload
c2) gives the roofline of the transit-parallel next() kernel the target is stated on
(`c2_next_roofline`), and on one GPU the reference's own GPU build is timed on the same c2 graph
(`reference_gpu`) when its binaries are present.

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
    """Initial transits of samples [first, first+S) of the job: walks start sample i at vertex i % V;
    k-hop and collective batches draw their seeds uniformly (one numpy Philox stream for the whole
    job, so a shard's seeds do not depend on how the job is cut)."""
    V = wl["V"]
    if wl["kind"] == WALK:
        return (np.arange(first, first + S, dtype=np.int64) % V).astype(np.int32)
    per = 1 if wl["kind"] == KHOP else wl["B"]
    rng = np.random.Generator(np.random.Philox(key=1))
    total = wl.get("S", V)
    return rng.integers(0, V, total * per, dtype=np.int64).astype(np.int32)[first * per:(first + S) * per]


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
        pairs -= st.get("pairs_not_entered", 0)   # PPR, load-balanced mode: pairs that were never written to or read from a map
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


def ncu_traffic(workload, mode, pairs_per_launch):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of the next() kernel, from the ncu
    captures recorded in profiles/ncu_traffic.json (each entry names its capture command).  An entry
    captured on a smaller case of the same kernel carries the pairs one captured launch processed
    and is scaled to this run's launches by the pairs per launch."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            tab = json.load(f)
    except Exception:
        return None, None
    e = tab.get(f"{workload}:{mode}")
    if not e:
        return None, None
    b = float(e["dram_bytes_per_launch"])
    if e.get("scale_by_pairs") and e.get("pairs_per_launch") and pairs_per_launch:
        b *= pairs_per_launch / float(e["pairs_per_launch"])
    return b, e.get("source")


def build_probe():
    """libnd_bench_probe.so beside this file (bench_probe.cu), compiled on first use if absent."""
    so, src = os.path.join(ROOT, "libnd_bench_probe.so"), os.path.join(ROOT, "bench_probe.cu")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run([os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc"), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
                        "-O3", "-shared", "-Xcompiler", "-fPIC", src, "-o", so], check=True, capture_output=True)
    return so


def gather_ceiling(wl, st, g, next_ms, next_launches, device):
    """The second ceiling of the walk kernels, measured live: next() is a few independent random
    4-byte gathers into the graph arrays per pair, and a GPU serves those at a rate set by the
    arrays' footprint against the L2 (bench_probe.cu), far below the copy bandwidth that
    `peak` is.  graph_gathers = the gathers into graph-sized arrays one pass needs (uniform walk:
    one neighbour id per edge; weighted: one (id, weight) record per try; node2vec: one candidate
    per try + one set bucket per membership test), floor = graph_gathers / rate."""
    import ctypes as C
    probe = C.CDLL(build_probe())
    probe.nd_bench_random_gather.argtypes = [C.c_int, C.c_int64, C.c_int64, C.c_int, C.POINTER(C.c_double)]
    app = wl["app"]
    if app == 0:
        gathers, footprint = st["sampled_edges"], 4 * g.E
    elif app in (1, 2):
        gathers, footprint = st["weight_tries"], 8 * g.E
    else:
        gathers, footprint = st["n2v_tries"] + st["n2v_probes"] // 8, 12 * g.E
    per_launch = max(int(gathers / max(next_launches, 1)), 1)
    rate = C.c_double(0.0)
    small = C.c_double(0.0)   # the same at the size of one launch: fixed launch and ramp costs included
    if probe.nd_bench_random_gather(device, int(footprint), 1 << 24, 3, C.byref(rate)) != 0 or \
            probe.nd_bench_random_gather(device, int(footprint), per_launch, 20, C.byref(small)) != 0:
        return None
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


def idle_kw(a):
    return {} if a.idle_weight is None else {"idle": a.idle_weight}


def emulated_shards(a, wl, nd, torch, local, seed):
    """--emulate-shards N on ONE GPU: the job is cut into the N seed ranges `--gpus N` would give
    the ranks, and every range is timed by itself, one after the other, on this GPU.  The slowest
    range is what the N-GPU job's device time (max over ranks) comes to, short of the barrier: at
    N = 2 and 4 the figure is within 3 % of the real runs.  Prints its own JSON line."""
    from nextdoor_b200 import dist as nd_dist
    V, S_total, N = wl["V"], wl.get("S", wl["V"]), a.emulate_shards
    mode = MODES[a.mode]
    g = nd.Graph.rmat(V, wl["M"], seed, device=local)
    pr = params_for(nd, wl, seed)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    bounds = None
    if wl["kind"] == WALK and a.shard_cut == "balanced":
        all_init = torch.from_numpy(seeds_for(wl, 0, S_total)).cuda()
        bounds = nd_dist.balanced_bounds(nd_dist.walk_start_weights(g, all_init, **idle_kw(a)), N)
        del all_init
    rows, edges = [], 0
    for r in range(N):
        first, S = nd_dist.shard(S_total, r, N, bounds)
        smp = nd.Sampler(g, pr, num_samples=S, first_sample=first, initial=seeds_for(wl, first, S))
        smp.set_stream(stream.cuda_stream)
        ms = timed_passes(torch, stream, torch.cuda.synchronize, lambda: smp.sample(mode, sync=False), a.steps, a.warmup) / a.steps
        e = smp.stats()["sampled_edges"]
        edges += e
        rows.append({"rank": r, "first_sample": first, "samples": S, "ms_per_step": round(ms, 4), "sampled_edges": e})
        smp.free()
    worst = max(x["ms_per_step"] for x in rows)
    print(json.dumps({"emulated_shards": N, "workload": f"{a.workload}: {wl['desc']}", "mode": a.mode, "shard_cut": a.shard_cut if bounds else "equal",
                      "steps": a.steps, "warmup": a.warmup, "slowest_shard_ms": worst, "value_at_slowest_shard": edges / (worst * 1e-3),
                      "unit": "sampled edges/s", "note": "every shard timed alone on one GPU; not a multi-GPU measurement", "shards": rows}))


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


def reference_arm(a, wl, seed):
    """--impl reference: the reference's next() bodies (oracle/_ref) or the oracle port on all host
    threads, each step a bounded prefix of the workload's samples."""
    from oracle import ndo
    V, M = wl["V"], wl["M"]
    t0 = time.perf_counter()
    hg = host_graph_cached(ndo, V, M, seed)   # same generator definition as the device one
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
        "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int32", "data": "synthetic",
        "config": {"workload": f"{a.workload}: {wl['desc']}", "host_graph_build_s": round(t_graph, 2)},
        "cpu_baseline": cb, "e2e": {"value": v, "unit": "sampled edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def host_graph_cached(ndo, V, M, seed):
    """The oracle's R-MAT graph on the host.  Building the 2^24-vertex graph takes minutes on the
    host cores and the driver runs this arm once per GPU count, so the arrays are kept in the
    system's temporary directory between runs of one box."""
    import tempfile
    if M < (1 << 26):
        return ndo.rmat_graph(V, M, seed)
    d = os.path.join(tempfile.gettempdir(), f"nd_b200_rmat_{V}_{M}_{seed}")
    names = ("row_ptr", "col", "w", "max_w")
    try:
        if os.path.exists(os.path.join(d, "done")):
            arrs = [np.load(os.path.join(d, n + ".npy")) for n in names]
            if arrs[0].shape[0] == V + 1 and arrs[1].shape[0] == int(arrs[0][-1]):
                return ndo.HostGraph(*arrs)
    except Exception:
        pass
    hg = ndo.rmat_graph(V, M, seed)
    try:
        os.makedirs(d, exist_ok=True)
        for n in names:
            np.save(os.path.join(d, n + ".npy"), getattr(hg, n))
        open(os.path.join(d, "done"), "w").close()
    except Exception:
        pass
    return hg


def next_kernel_name(nd, smp, mode):
    """The next() kernel the library launches for this sampler and mode (asked from the library)."""
    import ctypes as C
    buf = C.create_string_buffer(128)
    nd.check(nd.lib.nd_sampler_next_kernel(smp._h, mode, buf, 128))
    return buf.value.decode()


def timed_passes(torch, stream, barrier, fn, steps, warmup):
    """`warmup` untimed and `steps` timed calls of fn() between barriers; device time in ms."""
    for _ in range(warmup):
        fn()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    barrier()
    return e0.elapsed_time(e1)


def roofline_of(nd, smp, wl, workload, mode_name, mode, ms_per_step, hbm_peak, peak_kind, device, with_gather_probe=True):
    """One instrumented pass (an event pair around every launch; no graph replay) -> the roofline
    object of the next() launches."""
    smp.set_profiling(True)
    smp.sample(mode)
    ph = smp.phase_ms()
    smp.set_profiling(False)
    st = smp.stats()
    nb = next_bytes(wl, st, mode)
    tail_ms = ph.get("tail", (0.0, 0))[0]
    if wl["kind"] != COLL:
        next_ms, next_launches = ph["next"]          # the per-step next() launches ...
        next_ms += tail_ms                            # ... and the tail launch: its pairs are in the byte count too
    else:
        next_ms, next_launches = ph["next"][0] + ph["collect"][0], ph["next"][1] + ph["collect"][1]
    achieved = nb / (next_ms * 1e-3) / 1e9 if next_ms > 0 else 0.0
    phase_sum = sum(v[0] for v in ph.values())
    # in the replayed step the tail launch runs on a second stream beside the result update (the
    # instrumented pass runs them one after the other): the shorter of the two is hidden
    if tail_ms and "finalize" in ph and os.environ.get("ND_WALK_TAIL_INLINE", "0") in ("", "0"):
        phase_sum -= min(tail_ms, ph["finalize"][0])
    # the timed steps replay a CUDA graph, the instrumented pass does not: the same launches, scaled
    # by their share of the instrumented pass, inside the replayed step
    replay_ms = ms_per_step * (next_ms - tail_ms) / phase_sum if phase_sum > 0 and ms_per_step else None
    pairs_per_launch = None
    if wl["kind"] == WALK:      # pairs in the maps the step launches read (the tail launch and its pairs are not among them)
        pairs_per_launch = (float(smp.live_pairs()[:next_launches].sum()) if mode != 2 else float(st["live_pairs"])) / max(next_launches, 1)
    traffic, traffic_src = ncu_traffic(workload, mode_name, pairs_per_launch)
    gather = None
    if wl["kind"] == WALK and with_gather_probe:
        gather = gather_ceiling(wl, st, smp.graph, next_ms, next_launches, device)
    r = {"bound": "hbm", "kernel": next_kernel_name(nd, smp, mode), "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
         "frac": achieved / hbm_peak, "peak_kind": f"of {peak_kind}", "traffic": traffic, "traffic_source": traffic_src,
         "launches": next_launches, "avg_launch_us": 1e3 * (next_ms - tail_ms) / max(next_launches, 1),
         "tail_launch_us": 1e3 * tail_ms if tail_ms else None,
         "avg_launch_us_in_replayed_step": 1e3 * replay_ms / max(next_launches, 1) if replay_ms else None,
         "algorithmic_bytes_per_pass": nb, "random_gather": gather}
    return r, ph, st


def side_pass_c2(nd, torch, stream, barrier, local, seed, hbm_peak, peak_kind, steps):
    """A short node2vec pass on the 2^20-vertex graph in the transit-parallel + load-balanced mode:
    the kernel and workload the roofline target is stated on.  Every rank runs it (a replica each,
    one walk per vertex); rank 0 reports."""
    wl = WORKLOADS["c2"]
    g = nd.Graph.rmat(wl["V"], wl["M"], seed, device=local)
    pr = params_for(nd, wl, seed)
    smp = nd.Sampler(g, pr, num_samples=wl["V"], first_sample=0, initial=seeds_for(wl, 0, wl["V"]))
    smp.set_stream(stream.cuda_stream)
    ms = timed_passes(torch, stream, barrier, lambda: smp.sample(1, sync=False), steps, 3) / steps
    edges = smp.stats()["sampled_edges"]
    r, ph, st = roofline_of(nd, smp, wl, "c2", "tp_lb", 1, ms, hbm_peak, peak_kind, local)
    r.update({"workload": f"c2: {wl['desc']}", "mode": "tp_lb", "ms_per_step": ms, "value": edges / (ms * 1e-3),
              "unit_of_value": "sampled edges/s (one GPU)", "phases_ms": {k: round(v[0], 4) for k, v in ph.items()}})
    smp.free()
    return r, g


def reference_gpu_leg(g, wl, timeout=120):
    """The reference's own GPU build (oracle/_ref/ref_gpu_*, compiled from the reference tree for
    sm_100 where that tree is present) on the graph `g`, in its three modes; the figure is its own
    "End to end time" print (src/nextdoor.cu:2965, :3194).  A baseline leg like cpu_baseline."""
    import re
    import tempfile
    names = {0: "ref_gpu_uniform", 1: "ref_gpu_deepwalk", 2: "ref_gpu_ppr", 3: "ref_gpu_node2vec", 4: "ref_gpu_khop"}
    exe = os.path.join(ROOT, "oracle", "_ref", names.get(wl["app"], "none"))
    if not os.path.exists(exe):
        return {"unavailable": "the reference's GPU build is not present (oracle/_ref/ref_gpu_*: built only where the reference tree is)"}
    out = {"graph": "the c2 graph written as the reference's 12-byte binary edge list", "unit": "sampled edges/s"}
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "graph.bin")
        row_ptr, col, w, _ = g.to_host()
        rec = np.empty(col.shape[0], dtype=[("s", "<i4"), ("d", "<i4"), ("w", "<f4")])
        rec["s"] = np.repeat(np.arange(g.V, dtype=np.int32), np.diff(row_ptr))
        rec["d"], rec["w"] = col, w
        rec.tofile(path)
        del rec, row_ptr, col, w
        for key, kernel, lb in (("tp", "TransitParallel", 0), ("tp_lb", "TransitParallel", 1), ("sp", "SampleParallel", 0)):
            try:
                r = subprocess.run([exe, path, kernel, str(lb), "1"], capture_output=True, text=True, timeout=timeout)
            except subprocess.TimeoutExpired:
                out[key] = None
                out["error"] = f"{kernel} lb={lb}: no result within {timeout} s"
                break      # no further run after one that did not end
            t = re.search(r"End to end time ([0-9.eE+-]+) secs", r.stdout)
            n = re.search(r"totalSampledVertices (\d+)", r.stdout)
            if r.returncode != 0 or not t or not n or float(t.group(1)) <= 0:
                out[key] = None
                out["error"] = f"{kernel} lb={lb}: rc {r.returncode}: {(r.stderr or r.stdout)[-200:]}"
                break
            out[key] = int(n.group(1)) / float(t.group(1))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default="c5", choices=list(WORKLOADS))
    ap.add_argument("--mode", default="tp_lb", choices=list(MODES))
    ap.add_argument("--shard-cut", default="balanced", choices=["balanced", "equal"],
                    help="N > 1, walk workloads: cut the job's seed range where the ranks' expected work is equal "
                         "(nextdoor_b200.dist.balanced_bounds) or into the reference's equal counts (src/utils.hpp:26-27)")
    ap.add_argument("--idle-weight", type=float, default=None,
                    help="balanced cut: weight of a walk that cannot start (default: nextdoor_b200.dist.IDLE_WALK_WEIGHT)")
    ap.add_argument("--emulate-shards", type=int, default=0,
                    help="one GPU: time each of the N seed ranges an N-GPU run would use, one after the other; prints the slowest")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-side", action="store_true", help="skip the c2 roofline pass and the reference-GPU leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end and gather legs (kernel A/B runs)")
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
    S_total = wl.get("S", V)

    if a.impl == "reference":
        if rank == 0:
            reference_arm(a, wl, seed)
        return

    import torch
    from nextdoor_b200 import api as nd
    torch.cuda.set_device(local)
    if world > 1 and "ND_HOST_THREADS" not in os.environ:   # the ranks of one box share its host cores
        os.environ["ND_HOST_THREADS"] = str(max(4, min(32, len(os.sched_getaffinity(0)) // world)))
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if a.partitioned:
        return partitioned_bench(a, wl, nd, torch, rank, world, local, seed)
    if a.emulate_shards:
        assert world == 1, "--emulate-shards runs on one GPU"
        return emulated_shards(a, wl, nd, torch, local, seed)
    mode = MODES[a.mode]
    g = nd.Graph.rmat(V, M, seed, device=local)
    pr = params_for(nd, wl, seed)
    # one job, cut N ways into contiguous seed ranges: the reference's equal counts, or -- walks start
    # sample i at vertex i and the generator leaves most high vertex ids without neighbours -- ranges
    # of equal expected work (the samples are the same either way: the draws are keyed by sample index)
    bounds = None
    if world > 1 and wl["kind"] == WALK and a.shard_cut == "balanced":
        from nextdoor_b200 import dist as nd_dist
        all_init = torch.from_numpy(seeds_for(wl, 0, S_total)).cuda()
        bounds = nd_dist.balanced_bounds(nd_dist.walk_start_weights(g, all_init, **idle_kw(a)), world)
        del all_init
        first, S = nd_dist.shard(S_total, rank, world, bounds)
    else:
        first, S = nd.shard_range(S_total, rank, world)
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
        live = smp.live_pairs()[:30].tolist() if wl["kind"] == WALK and mode != 2 else None
        print(json.dumps({"profile_only": True, "workload": a.workload, "mode": a.mode, "stats": smp.stats(),
                          "live_pairs_of_the_first_steps": live}))
        return

    # ---- device-timed throughput (inputs resident)
    for _ in range(a.warmup):
        smp.sample(mode, sync=False)
    barrier()
    clocks = ClockSampler(local)
    clocks.start()
    l0 = nd.launch_count()
    ms = timed_passes(torch, stream, barrier, lambda: smp.sample(mode, sync=False), a.steps, 0)
    launches = nd.launch_count() - l0
    edges_step = smp.stats()["sampled_edges"]

    # ---- the same job in the reference's other kernel type (-k SampleParallel), for comparison
    ms_sp = None
    if mode != 2:
        ms_sp = timed_passes(torch, stream, barrier, lambda: smp.sample(2, sync=False), a.steps, 2)

    # ---- end to end through the public API with host buffers, in the SAME mode as `value`: seeds
    # H2D from pinned memory, sample, result D2H into pinned memory, through
    # nextdoor_b200.api.PipelinedSampler: the result of a step is copied on a second stream while
    # the next step is sampled (two sampler sets alternate).
    ms_e2e = e2e_check = d2h = ms_e2e_dense = None
    e2e_sparse, e2e_values = False, 0
    if not a.no_e2e:
        # this leg is bound by the result rows each rank copies to the host, empty or not: equal counts
        first_e, S_e = (first, S) if bounds is None else nd.shard_range(S_total, rank, world)
        init_e = init_np if bounds is None else seeds_for(wl, first_e, S_e)
        init_host = torch.from_numpy(init_e).pin_memory()
        out_host = torch.empty(S_e * fs, dtype=torch.int32).pin_memory()
        out_host2 = torch.empty(S_e * fs, dtype=torch.int32).pin_memory()   # consecutive steps land in alternating buffers
        init_pin, out_pin, out_pin2 = init_host.numpy(), out_host.numpy(), out_host2.numpy()
        copy_stream = torch.cuda.Stream()
        pipe = nd.PipelinedSampler(g, pr, S_e, first_sample=first_e, initial=init_e, chunks=E2E_CHUNKS, depth=E2E_DEPTH,
                                   stream=stream.cuda_stream, copy_stream=copy_stream.cuda_stream, sparse_rows=True)
        def e2e_passes(p):
            p.run(init_pin, out_pin, mode)            # untimed: both host arrays have been filled once
            p.run(init_pin, out_pin2, mode)
            barrier()
            x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            x0.record(stream)
            for i in range(a.steps):                  # step i+1 is sampled while the result of step i is on its way
                p.run_async(init_pin, out_pin if i % 2 == 0 else out_pin2, mode)
            p.wait()                                  # every step's result has landed in the host array
            x1.record(stream)
            barrier()
            return x0.elapsed_time(x1)

        ms_e2e = e2e_passes(pipe)
        last_pin = out_pin if a.steps % 2 == 1 else out_pin2    # the buffer the last step wrote
        e2e_check = int((last_pin != V).sum()) if wl["kind"] != COLL else None
        e2e_sparse, e2e_values = pipe.sparse_rows, pipe.values_copied
        pipe.free()
        ms_e2e_dense = None
        if e2e_sparse:      # the same leg with the dense array copied every step, for comparison
            pipe = nd.PipelinedSampler(g, pr, S_e, first_sample=first_e, initial=init_e, chunks=E2E_CHUNKS, depth=E2E_DEPTH,
                                       stream=stream.cuda_stream, copy_stream=copy_stream.cuda_stream, sparse_rows=False)
            ms_e2e_dense = e2e_passes(pipe)
            pipe.free()
        # the ceiling of that leg: the same result copy alone (every rank at once, nothing sampled)
        src = torch.empty(S_e * fs, dtype=torch.int32, device="cuda")
        for _ in range(1):
            out_host.copy_(src, non_blocking=True)
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record(stream)
        for _ in range(2):
            out_host.copy_(src, non_blocking=True)
        c1.record(stream)
        barrier()
        d2h = c0.elapsed_time(c1) / 2
        del src, out_host, out_host2, init_host
    clocks.stop_flag = True

    # ---- the final sample gather (the only step that crosses NVLink): every rank sends its shard to
    # rank 0, which holds the whole job's [S_total, finalSampleSize] array (getFinalSamples,
    # src/nextdoor.cu:3211-3237).  Two samplers alternate: the transfer of a step's samples runs on
    # NCCL's stream while the next step is sampled; a sampler's next run waits for the transfer
    # that still reads its buffer.
    ms_gather = ms_gather_dense = None
    gather_values = 0
    if world > 1 and not a.no_e2e:
        from nextdoor_b200 import dist as nd_dist
        smp2 = nd.Sampler(g, pr, num_samples=S, first_sample=first, initial=init_np)
        smp2.set_stream(stream.cuda_stream)
        pair = [(smp, nd_dist.device_samples(smp)), (smp2, nd_dist.device_samples(smp2))]
        n_full = 2 if 2 * S_total * fs * 4 < (48 << 30) else 1
        fulls = [torch.empty((S_total, fs), dtype=torch.int32, device="cuda") for _ in range(n_full)] if rank == 0 else []
        side = torch.cuda.Stream()
        pending = [None, None]

        def wait_all(k):
            if pending[k] is not None:
                for wk in pending[k]:
                    wk.wait()
                pending[k] = None

        def gather_step(i):
            k = i % 2
            s_k, shard_k = pair[k]
            wait_all(k)
            s_k.sample(mode, sync=False)
            ev = torch.cuda.Event()
            ev.record(stream)
            if n_full == 1:
                wait_all(k ^ 1)                # the single gathered array is still being written
            with torch.cuda.stream(side):
                side.wait_event(ev)
                pending[k] = nd_dist.gather_samples_start(shard_k, S_total, fulls[k % n_full] if rank == 0 else None, bounds=bounds) or None

        def gather_drain():
            for k in range(2):
                wait_all(k)
            side.synchronize()

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
        if rank == 0:      # the gathered array holds the job: its valid vertices are the job's sampled edges (checked below)
            gathered_edges = int((fulls[((a.steps - 1) % 2) % n_full] != V).sum()) if wl["kind"] != COLL else None
        del fulls
        # ---- walks: the same gather by row prefixes (every rank packs, rank 0 unpacks into the dense
        # array it keeps from step to step); the transfer and unpacking of a step run on the side stream
        # under the next step's sampling
        if wl["kind"] == WALK:
            ms_gather_dense = ms_gather
            pg = nd_dist.PackedRowsGather(S_total, fs, V, dst=0, bounds=bounds)
            waiting = [None]

            def packed_step(i):
                s_k = pair[i % 2][0]
                s_k.sample(mode, sync=False)
                h = pg.start(s_k)
                if waiting[0] is not None:
                    with torch.cuda.stream(side):
                        pg.finish(waiting[0])
                waiting[0] = h

            def packed_drain():
                if waiting[0] is not None:
                    with torch.cuda.stream(side):
                        pg.finish(waiting[0])
                    waiting[0] = None

            for i in range(2):
                packed_step(i)
            packed_drain()
            barrier()
            y0, y1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            y0.record(stream)
            for i in range(a.steps):
                packed_step(i)
            packed_drain()
            y1.record(stream)
            barrier()
            ms_gather = y0.elapsed_time(y1)
            gather_values = pg.values_moved
            if rank == 0:
                assert int((pg.full != V).sum()) == gathered_edges, "the array gathered by row prefixes differs from the dense gather"
            del pg
        smp2.free()

    # ---- per-phase device time of one instrumented pass (roofline of the next() kernels)
    roof, ph, st = roofline_of(nd, smp, wl, a.workload, a.mode, mode, ms / a.steps, hbm_peak, peak_kind, local,
                               with_gather_probe=(rank == 0))

    tms = torch.tensor([ms, ms_e2e or 0.0, ms_gather or 0.0, ms_sp or 0.0, d2h or 0.0, ms_e2e_dense or 0.0, ms_gather_dense or 0.0],
                       dtype=torch.float64, device="cuda")
    tot = torch.tensor([float(edges_step), float(e2e_check or 0), float(e2e_values)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    ms, ms_e2e, ms_gather, ms_sp, d2h, ms_e2e_dense, ms_gather_dense = (float(x) for x in tms)
    total_edges, e2e_total, e2e_values = float(tot[0]), float(tot[1]), float(tot[2])
    if ms_e2e and wl["kind"] == WALK:
        assert int(e2e_total) == int(total_edges), "the host arrays of the end-to-end leg do not hold the job's sampled vertices"
    if world > 1 and ms_gather and rank == 0 and gathered_edges is not None:
        assert gathered_edges == int(total_edges), "the array gathered on rank 0 does not hold the whole job"

    # ---- cpu baseline (one GPU only), then the main sampler's buffers are released for the side passes
    cb = None
    if rank == 0 and world == 1 and not a.no_cpu_baseline:
        from oracle import ndo
        row_ptr, col, w, mw = g.to_host()
        cb = cpu_baseline(ndo.HostGraph(row_ptr, col, w, mw), wl, seed)
        del row_ptr, col, w, mw
    graph_desc = f"R-MAT a=.57 b=.19 c=.19 d=.05 seed 0, V={V}, CSR entries={g.E}, max degree={g.max_degree}"
    smp.free()
    g.free()

    # ---- the kernel the roofline target is stated on, and the reference's GPU build beside it
    c2_roof = ref_gpu = None
    if not a.no_side and a.workload != "c2":
        c2_roof, g2 = side_pass_c2(nd, torch, stream, barrier, local, seed, hbm_peak, peak_kind, a.steps)
        if rank == 0 and world == 1:
            ref_gpu = reference_gpu_leg(g2, WORKLOADS["c2"])
        g2.free()
        barrier()

    if rank == 0:
        per_step = total_edges
        line = {
            "metric": "sampled edges/sec", "value": per_step * a.steps / (ms * 1e-3), "unit": "sampled edges/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int32", "data": "synthetic",
            "config": {"workload": f"{a.workload}: {wl['desc']}", "app": APP_NAMES[app], "mode": a.mode,
                       "samples_total": S_total, "samples_rank0": S, "final_sample_size": fs,
                       "sharding": ("one job, contiguous seed ranges of equal expected work (walks that can start weigh 1, the others 1/20), "
                                    "graph replicated per GPU" if bounds else
                                    "one job, contiguous seed ranges of equal counts (src/utils.hpp:26-27), graph replicated per GPU"),
                       "shard_bounds": bounds,
                       "graph": graph_desc,
                       "l2": "working set (graph + sample buffers) larger than L2; no flush between steps",
                       "sampled_edges_per_step": per_step},
            "e2e": None if ms_e2e is None or ms_e2e <= 0 else {
                "value": per_step * a.steps / (ms_e2e * 1e-3), "unit": "sampled edges/s",
                "h2d_bytes_per_step": int(4 * S_total * smp.isz),
                "d2h_bytes_per_step": int(4 * (S_total + e2e_values)) if e2e_sparse else int(S_total * fs * 4),
                "host_result": ("the caller's dense [samples, finalSampleSize] host array, kept from step to step: row lengths and the rows' "
                                "valid prefixes cross PCIe, host threads rewrite the slots that changed (nd_sampler_host_update_*)"
                                if e2e_sparse else "the dense [samples, finalSampleSize] array copied every step"),
                "dense_result_bytes": int(S_total * fs * 4),
                "dense_copy": None if not ms_e2e_dense else {
                    "value": per_step * a.steps / (ms_e2e_dense * 1e-3), "unit": "sampled edges/s",
                    "note": "same leg with the dense array copied every step (PipelinedSampler(sparse_rows=False)), the path d2h_ceiling bounds"},
                "chunks": E2E_CHUNKS, "depth": E2E_DEPTH, "mode": a.mode, "valid_vertices_in_host_result": int(e2e_total),
                "sharding": "equal counts (src/utils.hpp:26-27): the result rows each rank copies out bound this leg",
                "d2h_ceiling_gbs": S_total * fs * 4 / (d2h * 1e-3) / 1e9 if d2h else None,
                "d2h_ceiling_note": "all ranks copying their shard of the result to pinned host memory at once, nothing else running; "
                                    "aggregate GB/s; dense_copy.value <= d2h_ceiling / (4 * final_sample_size) * sampled edges per sample slot"},
            "gpu_launches": int(launches),
            "sample_parallel": None if mode == 2 else {"value": per_step * a.steps / (ms_sp * 1e-3), "unit": "sampled edges/s",
                                                       "note": "same sampler, same samples, nd_mode SampleParallel"},
            "with_gather": None if not ms_gather else {
                "value": per_step * a.steps / (ms_gather * 1e-3), "unit": "sampled edges/s",
                "collective": ("every rank packs its rows' valid prefixes and sends lengths + vertices to rank 0 (NCCL send/recv), which unpacks them "
                               "into the dense [samples, finalSampleSize] array it keeps (nextdoor_b200.dist.PackedRowsGather); a step's transfer runs "
                               "under the next step's sampling (two samplers alternate)" if ms_gather_dense else
                               "every rank sends its dense shard to rank 0 (NCCL send/recv), overlapped with the next step's sampling (two samplers alternate)"),
                "bytes_into_rank0_per_step": int(4 * (S_total - S) + 4 * gather_values) if ms_gather_dense else int((S_total - S) * fs * 4),
                "dense_rows": None if not ms_gather_dense else {
                    "value": per_step * a.steps / (ms_gather_dense * 1e-3), "unit": "sampled edges/s",
                    "bytes_into_rank0_per_step": int((S_total - S) * fs * 4),
                    "floor_ms_at_770_GBps": (S_total - S) * fs * 4 / 770e9 * 1e3,
                    "note": "the same gather with every rank's dense shard sent (nextdoor_b200.dist.gather_samples_start)"}},
            "roofline": roof,
            "c2_next_roofline": c2_roof,
            "reference_gpu": ref_gpu,
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
