"""GPU parity tests of the random-walk apps through the C ABI: bit-exact against the oracle and the
golden fixtures in every execution mode; size-independent properties at the benchmark's sizes."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
MODES = [0, 1, 2]   # TransitParallel, TransitParallel+LB, SampleParallel
WALKS = [0, 1, 2, 3]


def _graph(nd, hg):
    return nd.Graph.from_csr(hg.row_ptr, hg.col, hg.w, hg.max_w)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", ["uniform_walk", "deepwalk", "ppr", "node2vec"])
def test_walks_match_golden(nd, ndo, name, mode):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    zg = np.load(os.path.join(GOLD, "graph_rmat300.npz"))
    g = nd.Graph.from_csr(zg["row_ptr"], zg["col"], zg["w"], zg["max_w"])
    pr = nd.app_params(int(z["app"]), steps=int(z["steps"]), seed=int(z["seed"]))
    s = nd.Sampler(g, pr, num_samples=int(z["S"]), first_sample=int(z["first"]))
    s.sample(mode)
    assert np.array_equal(s.final_samples(), z["out"])
    assert s.stats()["sampled_edges"] == int(z["sampled_edges"])


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("app", WALKS)
def test_walks_match_oracle(nd, ndo, small_graph, app, mode):
    g = _graph(nd, small_graph)
    kw = dict(stop_prob=0.15) if app == 2 else {}
    S, first = 5000, 777          # more samples than vertices: start vertex = index % V
    for steps in (1, 2, 33):
        pr = nd.app_params(app, steps=steps, seed=42, **kw)
        opr = ndo.make_params(app, steps=steps, seed=42, **kw)
        s = nd.Sampler(g, pr, num_samples=S, first_sample=first)
        s.sample(mode)
        exp = ndo.sample(small_graph, opr, S, first=first)
        got = s.final_samples()
        assert np.array_equal(got, exp["out"]), f"app {app} mode {mode} steps {steps}"
        st = s.stats()
        assert st["sampled_edges"] == exp["counters"]["sampled_edges"]
        assert st["live_pairs"] == exp["counters"]["live_pairs"]
        # the events behind the algorithmic-bytes model: tries of the rejection loops
        assert st["weight_tries"] == exp["counters"]["weight_tries"]
        assert st["n2v_tries"] == exp["counters"]["n2v_tries"]
        # a second run of the same sampler gives the same answer
        s.sample(mode)
        assert np.array_equal(s.final_samples(), exp["out"])


def test_uniform_walk_hub_staging(nd, ndo, monkeypatch):
    """ND_WALK_STAGING=1: whole tiles of 256 pairs that stand on one transit are served from the
    transit's adjacency list staged in shared memory (walk_next_hub_kernel), the rest by the
    thread-per-pair kernel.  A star with a ring: a third of all walkers meet on the hub, whose list
    (2999 ids here; 20 000 in the second graph, more than one staged chunk) is streamed in chunks."""
    monkeypatch.setenv("ND_WALK_STAGING", "1")
    for V, S, steps in ((3000, 30_000, 12), (20_001, 60_000, 6)):
        spokes = np.arange(1, V, dtype=np.int32)
        ring_a, ring_b = spokes, np.roll(spokes, -1)
        src = np.concatenate([np.zeros(V - 1, np.int32), spokes, ring_a, ring_b])
        dst = np.concatenate([spokes, np.zeros(V - 1, np.int32), ring_b, ring_a])
        hg = ndo.csr_from_records(src, dst, np.ones(src.shape[0], np.float32), V=V)
        g = _graph(nd, hg)
        pr = nd.app_params(0, steps=steps, seed=17)
        s = nd.Sampler(g, pr, num_samples=S)
        s.sample(1)
        exp = ndo.sample(hg, ndo.make_params(0, steps=steps, seed=17), S)
        assert np.array_equal(s.final_samples(), exp["out"])
        assert s.stats()["sampled_edges"] == exp["counters"]["sampled_edges"]
        live = s.live_pairs()
        assert live[1] == S and live[2] == S          # nobody dies on this graph: the hub holds thousands of pairs


@pytest.mark.parametrize("no_tail", ["0", "1"])
def test_ppr_tail_launch_and_step_loop_agree(nd, ndo, small_graph, monkeypatch, no_tail):
    """PPR in the load-balanced mode finishes the few walks that are still alive with one tail
    launch; ND_WALK_NO_TAIL=1 keeps the step-by-step loop to the end.  Both give the oracle's walks
    and counters."""
    if no_tail == "1":
        monkeypatch.setenv("ND_WALK_NO_TAIL", "1")
    else:
        monkeypatch.delenv("ND_WALK_NO_TAIL", raising=False)
    g = _graph(nd, small_graph)
    pr = nd.app_params(2, steps=60, seed=21, stop_prob=0.15)
    opr = ndo.make_params(2, steps=60, seed=21, stop_prob=0.15)
    S = 20_000
    s = nd.Sampler(g, pr, num_samples=S, first_sample=3)
    s.sample(1)
    exp = ndo.sample(small_graph, opr, S, first=3)
    assert np.array_equal(s.final_samples(), exp["out"])
    st = s.stats()
    assert st["sampled_edges"] == exp["counters"]["sampled_edges"] and st["live_pairs"] == exp["counters"]["live_pairs"]
    assert st["weight_tries"] == exp["counters"]["weight_tries"]


@pytest.mark.parametrize("inline", ["0", "1"])
def test_ppr_tail_beside_the_result_update_over_changing_passes(nd, ndo, small_graph, monkeypatch, inline):
    """The tail launch runs on a second stream beside the result update and writes its walks' rows
    itself (ND_WALK_TAIL_INLINE=1: on the same stream, one after the other).  The result array
    keeps its contents between passes, so passes with different start vertices on one sampler --
    rows that grow and rows that shrink, walks that change sides between the two kernels -- must
    each give the oracle's array; replayed as a CUDA graph on a caller's stream, with the
    hand-over to the tail at several steps, and with the phase timers on."""
    import torch
    monkeypatch.setenv("ND_WALK_TAIL_INLINE", inline)
    g = _graph(nd, small_graph)
    S = 30_000
    rng = np.random.default_rng(4)
    for pairs_floor in ("2000", "12000", "100000"):        # hand-over late, in the middle, after step 0
        monkeypatch.setenv("ND_WALK_TAIL_PAIRS", pairs_floor)
        pr = nd.app_params(2, steps=48, seed=33, stop_prob=0.15)
        opr = ndo.make_params(2, steps=48, seed=33, stop_prob=0.15)
        s = nd.Sampler(g, pr, num_samples=S, first_sample=7)
        st = torch.cuda.Stream()
        s.set_stream(st.cuda_stream)
        for p in range(4):
            init = rng.integers(0, small_graph.V, S).astype(np.int32)
            if p == 2:
                init[::3] = -1                             # a third of the walks never start
            s.set_initial(init)
            if p == 3:
                s.set_profiling(True)
            s.sample(1)
            clean = np.where(init < 0, small_graph.V, init).astype(np.int32)
            exp = ndo.sample(small_graph, opr, S, first=7, initial=clean)
            assert np.array_equal(s.final_samples(), exp["out"]), (pairs_floor, p)
            c = s.stats()
            assert c["sampled_edges"] == exp["counters"]["sampled_edges"], (pairs_floor, p)
            assert c["live_pairs"] == exp["counters"]["live_pairs"], (pairs_floor, p)
        assert s.phase_ms()["tail"][1] == 1                # one tail launch in the timed pass
        s.set_profiling(False)
        s.sample(2)                                        # the sample-parallel mode on the same result array
        assert np.array_equal(s.final_samples(), exp["out"])
        s.free()


@pytest.mark.parametrize("mode", MODES)
def test_node2vec_corrected_comparison(nd, ndo, small_graph, mode):
    g = _graph(nd, small_graph)
    pr = nd.app_params(3, steps=20, seed=9, n2v_ref_compat=0, p=0.5, q=2.0)
    opr = ndo.make_params(3, steps=20, seed=9, n2v_ref_compat=0, p=0.5, q=2.0)
    s = nd.Sampler(g, pr, num_samples=3000)
    s.sample(mode)
    assert np.array_equal(s.final_samples(), ndo.sample(small_graph, opr, 3000)["out"])


@pytest.mark.parametrize("mode", MODES)
def test_explicit_initial_samples_and_edge_cases(nd, ndo, tiny_graph, mode):
    g = _graph(nd, tiny_graph)
    init = np.array([8, 0, 3, 3, 9, 6, 10, -1, 5], np.int32)     # isolated, valid, out of range
    pr = nd.app_params(1, steps=7, seed=3)
    opr = ndo.make_params(1, steps=7, seed=3)
    s = nd.Sampler(g, pr, num_samples=len(init), initial=init)
    s.sample(mode)
    got = s.final_samples()
    clean = np.where((init < 0) | (init >= g.V), g.V, init).astype(np.int32)
    exp = ndo.sample(tiny_graph, opr, len(init), initial=clean)
    assert np.array_equal(got, exp["out"])
    assert (got[0] == g.V).all() and (got[6] == g.V).all() and (got[7] == g.V).all()
    # new seeds on the same sampler
    init2 = np.array([0, 1, 2, 3, 4, 5, 6, 7, 8], np.int32)
    s.set_initial(init2)
    s.sample(mode)
    assert np.array_equal(s.final_samples(), ndo.sample(tiny_graph, opr, 9, initial=init2)["out"])
    # zero samples
    s0 = nd.Sampler(g, pr, num_samples=0)
    s0.sample(mode)
    assert s0.final_samples().shape == (0, 7)


def test_shards_concatenate_to_the_single_gpu_answer(nd, ndo, small_graph):
    """Seed-range sharding (PartStartPointer, src/utils.hpp:26-27): the keyed draws use the global
    sample index, so shards computed separately equal the unsharded run."""
    g = _graph(nd, small_graph)
    pr = nd.app_params(2, steps=30, seed=8, stop_prob=0.15)
    S = 3001
    whole = nd.Sampler(g, pr, num_samples=S)
    whole.sample(1)
    parts = []
    for i in range(4):
        f, c = nd.shard_range(S, i, 4)
        sh = nd.Sampler(g, pr, num_samples=c, first_sample=f)
        sh.sample(1)
        parts.append(sh.final_samples())
    assert np.array_equal(np.concatenate(parts), whole.final_samples())


def test_balanced_seed_ranges_concatenate_to_the_single_gpu_answer(nd, ndo, small_graph):
    """Seed ranges cut where the expected work is equal (walks from vertices without neighbours
    weigh a twentieth): the weights come from the device's row offsets, and the shards still
    concatenate to the unsharded job."""
    import torch
    from nextdoor_b200 import dist as nd_dist
    g = _graph(nd, small_graph)
    S = 5000
    init = (np.arange(S) % small_graph.V).astype(np.int32)
    init[100:900] = -1                                  # a stretch of walks that cannot start
    wts = nd_dist.walk_start_weights(g, torch.from_numpy(init).cuda())
    clean = np.clip(init, 0, small_graph.V - 1)
    has = (np.diff(small_graph.row_ptr)[clean] > 0) & (init >= 0)
    assert np.allclose(wts.cpu().numpy(), np.where(has, 1.0, nd_dist.IDLE_WALK_WEIGHT))
    bounds = nd_dist.balanced_bounds(wts, 4)
    act = [int(has[bounds[r]:bounds[r + 1]].sum()) for r in range(4)]
    assert max(act) - min(act) <= 0.05 * sum(act) + 16
    pr = nd.app_params(2, steps=30, seed=8, stop_prob=0.15)
    whole = nd.Sampler(g, pr, num_samples=S, initial=init)
    whole.sample(1)
    parts = []
    for r in range(4):
        f, c = nd_dist.shard(S, r, 4, bounds)
        sh = nd.Sampler(g, pr, num_samples=c, first_sample=f, initial=init[f:f + c])
        sh.sample(1)
        parts.append(sh.final_samples())
    assert np.array_equal(np.concatenate(parts), whole.final_samples())


@pytest.mark.parametrize("app", [0, 3])
def test_full_size_properties(nd, ndo, app):
    """Benchmark-sized run (2^20 vertices, 16M undirected edges, one 100-step walk per vertex):
    every sampled edge exists in the CSR (check_results.cu:162-299 on all steps), modes agree with
    each other, and a seed subset is bit-exact against the oracle."""
    V, M = 1 << 20, 1 << 24
    g = nd.Graph.rmat(V, M, seed=0)
    row_ptr, col, w, mw = g.to_host()
    hg = ndo.HostGraph(row_ptr, col, w, mw)
    pr = nd.app_params(app, steps=100, seed=0)
    opr = ndo.make_params(app, steps=100, seed=0)
    s = nd.Sampler(g, pr, num_samples=V)
    outs = []
    for mode in (1, 2):
        s.sample(mode)
        outs.append(s.final_samples().copy())
    assert np.array_equal(outs[0], outs[1])
    out = outs[0]
    sub = 20000
    exp = ndo.sample(hg, opr, sub)
    assert np.array_equal(out[:sub], exp["out"])
    init = (np.arange(V) % V).astype(np.int32)
    assert ndo.check_sampled_vertices(hg, opr, V, init, out) == 0
    assert s.stats()["sampled_edges"] == int((out != V).sum())


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("app", [1, 3])
def test_graph_replay_on_user_stream(nd, ndo, small_graph, app, mode):
    """On a caller's (non-default) stream the step loop is captured into a CUDA graph at the first
    sample() and replayed afterwards; new seeds must flow through the replay."""
    import torch
    g = _graph(nd, small_graph)
    pr = nd.app_params(app, steps=25, seed=5)
    opr = ndo.make_params(app, steps=25, seed=5)
    S = 4000
    s = nd.Sampler(g, pr, num_samples=S)
    st = torch.cuda.Stream()
    s.set_stream(st.cuda_stream)
    exp = ndo.sample(small_graph, opr, S)["out"]
    for _ in range(3):
        s.sample(mode)
        assert np.array_equal(s.final_samples(), exp)
    init2 = np.random.default_rng(1).integers(0, small_graph.V, S).astype(np.int32)
    s.set_initial(init2)
    s.sample(mode)
    assert np.array_equal(s.final_samples(), ndo.sample(small_graph, opr, S, initial=init2)["out"])
    assert s.stats()["sampled_edges"] == int((s.final_samples() != small_graph.V).sum())


def test_pipelined_sampler_equals_single_sampler(nd, ndo, small_graph):
    """Seed-range chunks sampled back to back while finished chunks are copied to pinned memory on a second stream."""
    import torch
    g = _graph(nd, small_graph)
    pr = nd.app_params(2, steps=40, seed=12, stop_prob=0.15)
    opr = ndo.make_params(2, steps=40, seed=12, stop_prob=0.15)
    S, first = 10_003, 31
    init = ((np.arange(first, first + S)) % small_graph.V).astype(np.int32)
    st, cst = torch.cuda.Stream(), torch.cuda.Stream()
    pipe = nd.PipelinedSampler(g, pr, S, first_sample=first, initial=init, chunks=3, stream=st.cuda_stream, copy_stream=cst.cuda_stream)
    init_pin = torch.from_numpy(init).pin_memory().numpy()
    out_pin = torch.empty(S * 40, dtype=torch.int32).pin_memory().numpy()
    exp = ndo.sample(small_graph, opr, S, first=first, initial=init)
    for mode in MODES:
        out_pin[:] = -7
        pipe.run(init_pin, out_pin, mode)
        assert np.array_equal(out_pin.reshape(S, 40), exp["out"])
    assert pipe.stats()["sampled_edges"] == exp["counters"]["sampled_edges"]


def test_host_array_updated_by_row_prefixes(nd, ndo, small_graph):
    """nd_sampler_host_update_*: only the rows' valid prefixes cross to the host and only the
    slots that changed are rewritten in the caller's dense array, which must equal the dense copy
    after every pass -- rows growing, shrinking, vanishing; all three modes; the dense fallback
    when most slots are in use; zero samples."""
    g = _graph(nd, small_graph)
    V = small_graph.V
    S, steps = 20_011, 40
    rng = np.random.default_rng(9)
    pr = nd.app_params(2, steps=steps, seed=5, stop_prob=0.15)
    s = nd.Sampler(g, pr, num_samples=S, first_sample=2)
    out = np.empty(S * steps, np.int32)
    nd.host_fill(out, V)
    assert (out == V).all()
    row_len = np.zeros(S, np.int32)
    copied = []
    for p, mode in enumerate((1, 2, 0, 1, 1)):
        init = rng.integers(0, V, S).astype(np.int32)
        if p == 3:
            init[: S // 2] = -1                          # half of the rows become empty
        s.set_initial(init)
        s.sample(mode)
        s.host_update_begin(out, row_len)
        if p % 2:
            s.host_update_fetch()                        # optional middle call
        copied.append(s.host_update_finish())
        dense = s.final_samples()
        assert np.array_equal(out.reshape(S, steps), dense), p
        assert np.array_equal(row_len, (dense != V).sum(axis=1)), p
        assert copied[-1] == int((dense != V).sum()) < S * steps // 4
    s.free()
    # full-length walks: more than half of the slots in use, the dense array is copied as it is
    pr = nd.app_params(0, steps=steps, seed=5)
    s = nd.Sampler(g, pr, num_samples=S)
    s.sample(1)
    s.host_update_begin(out, row_len)
    assert s.host_update_finish() == S * steps
    assert np.array_equal(out.reshape(S, steps), s.final_samples())
    assert np.array_equal(row_len, (s.final_samples() != V).sum(axis=1))
    s.free()
    s0 = nd.Sampler(g, pr, num_samples=0)
    s0.sample(1)
    s0.host_update_begin(out[:0], row_len[:0])
    assert s0.host_update_finish() == 0
    k = nd.Sampler(g, nd.app_params(4, fanout=[3, 2], seed=1), num_samples=10)
    k.sample(1)
    with pytest.raises(nd.NdError):
        k.host_update_begin(out, row_len)                # k-hop rows are not prefixes


@pytest.mark.parametrize("S,steps,stop", [(37, 7, 0.5), (4096, 7, 0.3), (8193, 101, 0.02), (1, 3, 0.5)])
def test_host_array_row_prefixes_odd_sizes(nd, ndo, small_graph, monkeypatch, S, steps, stop):
    """Row lengths that are no multiple of four, fewer rows than one packing chunk, exactly one
    chunk, one row, long rows, a thread count that does not divide the rows: the host array and an
    unpacked device array follow the sampler."""
    import torch
    monkeypatch.setenv("ND_HOST_THREADS", "3" if S > 1 else "5")
    g = _graph(nd, small_graph)
    V = small_graph.V
    pr = nd.app_params(2, steps=steps, seed=2, stop_prob=stop)
    s = nd.Sampler(g, pr, num_samples=S, first_sample=11)
    out = np.full(S * steps, V, np.int32)
    row_len = np.zeros(S, np.int32)
    full = torch.full((S, steps), V, dtype=torch.int32, device="cuda")
    full_len = torch.zeros(S, dtype=torch.int32, device="cuda")
    scratch = torch.empty(nd.rows_scratch_words(S), dtype=torch.int32, device="cuda")
    rng = np.random.default_rng(S)
    for p in range(3):
        s.set_initial(rng.integers(0, V, S).astype(np.int32))
        s.sample(1)
        dense = s.final_samples()
        s.host_update_begin(out, row_len)
        s.host_update_finish()
        assert np.array_equal(out.reshape(S, steps), dense), p
        len_ptr, vals_ptr = s.pack_rows()
        assert s.pack_rows_total() == int((dense != V).sum())
        nd.rows_unpack(0, None, S, steps, V, len_ptr, vals_ptr, full.data_ptr(), full_len.data_ptr(), scratch.data_ptr())
        torch.cuda.synchronize()
        assert np.array_equal(full.cpu().numpy(), dense), p


def test_pipelined_jobs_into_remembered_host_arrays(nd, ndo, small_graph):
    """PipelinedSampler(sparse_rows=True): jobs with changing seeds alternate between two host
    arrays without waiting in between; each array must hold its own job's dense result."""
    import torch
    g = _graph(nd, small_graph)
    pr = nd.app_params(2, steps=40, seed=12, stop_prob=0.15)
    opr = ndo.make_params(2, steps=40, seed=12, stop_prob=0.15)
    S, first = 20_001, 5
    st, cst = torch.cuda.Stream(), torch.cuda.Stream()
    inits = [((np.arange(first, first + S) * k) % small_graph.V).astype(np.int32) for k in (1, 3, 7, 11, 13)]
    inits[2][::2] = -1
    for depth, chunks in ((2, 1), (1, 3), (3, 2)):
        pipe = nd.PipelinedSampler(g, pr, S, first_sample=first, initial=inits[0], chunks=chunks, stream=st.cuda_stream,
                                   copy_stream=cst.cuda_stream, depth=depth, sparse_rows=True)
        pins = [torch.from_numpy(i).pin_memory().numpy() for i in inits]
        outs = [torch.full((S * 40,), -7, dtype=torch.int32).pin_memory().numpy() for _ in range(2)]
        for j, ip in enumerate(pins):
            pipe.run_async(ip, outs[j % 2], 1)
        pipe.wait()
        for j in (len(inits) - 2, len(inits) - 1):       # the last job of each array
            clean = np.where(inits[j] < 0, small_graph.V, inits[j]).astype(np.int32)
            exp = ndo.sample(small_graph, opr, S, first=first, initial=clean)
            assert np.array_equal(outs[j % 2].reshape(S, 40), exp["out"]), (depth, chunks, j)
        assert pipe.values_copied == exp["counters"]["sampled_edges"]
        pipe.forget(outs[0])
        outs[0][:] = -3                                  # the caller scribbles: after forget() the next job refills the array
        pipe.run(pins[0], outs[0], 2)
        assert np.array_equal(outs[0].reshape(S, 40), ndo.sample(small_graph, opr, S, first=first, initial=inits[0])["out"])
        pipe.free()


def test_pipelined_jobs_back_to_back(nd, ndo, small_graph):
    """Jobs enqueued without waiting in between (the next job samples while the previous one's
    last chunk is still copied) land complete and unmixed in their own host buffers."""
    import torch
    g = _graph(nd, small_graph)
    pr = nd.app_params(3, steps=40, seed=12, p=2.0, q=0.5)
    opr = ndo.make_params(3, steps=40, seed=12, p=2.0, q=0.5)
    S, first = 20_001, 5
    st, cst = torch.cuda.Stream(), torch.cuda.Stream()
    inits = [((np.arange(first, first + S) * k) % small_graph.V).astype(np.int32) for k in (1, 3, 7, 11)]
    pipe = nd.PipelinedSampler(g, pr, S, first_sample=first, initial=inits[0], chunks=2, stream=st.cuda_stream,
                               copy_stream=cst.cuda_stream)
    pins = [torch.from_numpy(i).pin_memory().numpy() for i in inits]
    outs = [torch.full((S * 40,), -7, dtype=torch.int32).pin_memory().numpy() for _ in inits]
    for ip, op in zip(pins, outs):
        pipe.run_async(ip, op, 1)
    pipe.wait()
    for i, op in zip(inits, outs):
        exp = ndo.sample(small_graph, opr, S, first=first, initial=i)
        assert np.array_equal(op.reshape(S, 40), exp["out"])
