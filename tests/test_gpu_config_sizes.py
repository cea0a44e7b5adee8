"""GPU parity at the benchmark configurations' own sizes, through the C ABI.

Each test builds the configuration's synthetic graph on the device at full size and checks the
result against the oracle where the oracle finishes in seconds (a prefix or a slice of the
samples) and through size-independent properties on everything: the execution modes agree byte
for byte, every sampled edge exists in the CSR (the condition of the reference's checkers,
src/check_results.cu:162-299), the device's edge counter equals the count of valid vertices.
"""
import numpy as np
import pytest

from test_gpu_collective import _compare_importance

pytestmark = pytest.mark.gpu


def _host(ndo, g):
    row_ptr, col, w, mw = g.to_host()
    return ndo.HostGraph(row_ptr, col, w, mw)


def test_uniform_walk_56944_vertices_whole_output(nd, ndo):
    """Uniform walk, length 100, one walk per vertex on the 56,944-vertex graph: the whole output
    of all three modes against the oracle."""
    V, M = 56944, 400_000
    g = nd.Graph.rmat(V, M, seed=0)
    hg = _host(ndo, g)
    eg = ndo.rmat_graph(V, M, seed=0)
    assert np.array_equal(hg.row_ptr, eg.row_ptr) and np.array_equal(hg.col, eg.col) and np.array_equal(hg.w, eg.w)
    pr = nd.app_params(0, steps=100, seed=0)
    exp = ndo.sample(hg, ndo.make_params(0, steps=100, seed=0), V)
    s = nd.Sampler(g, pr, num_samples=V)
    for mode in (0, 1, 2):
        s.sample(mode)
        assert np.array_equal(s.final_samples(), exp["out"]), f"mode {mode}"
        assert s.stats()["sampled_edges"] == exp["counters"]["sampled_edges"]


def test_ppr_stop15_on_2_24_vertices(nd, ndo):
    """Weighted PPR, stop probability 0.15, one walk per vertex on 2^24 vertices / 2^28
    undirected edges: the edge offsets reach 2^29 and stay inside int32."""
    import torch
    from nextdoor_b200 import dist as nd_dist
    V, M = 1 << 24, 1 << 28
    g = nd.Graph.rmat(V, M, seed=0)
    assert g.E == 2 * M == 1 << 29
    hg = _host(ndo, g)
    assert int(hg.row_ptr[V]) == 1 << 29 and (np.diff(hg.row_ptr) >= 0).all()
    pr = nd.app_params(2, steps=100, seed=0, stop_prob=0.15)
    opr = ndo.make_params(2, steps=100, seed=0, stop_prob=0.15)
    s = nd.Sampler(g, pr, num_samples=V)
    s.sample(1)
    s.sync()
    first = nd_dist.device_samples(s).clone()
    edges_lb = s.stats()["sampled_edges"]
    s.sample(2)
    s.sync()
    second = nd_dist.device_samples(s)
    assert torch.equal(first, second), "TransitParallel+LB and SampleParallel differ"
    assert edges_lb == s.stats()["sampled_edges"] == int((second != V).sum())
    sub = 20000
    exp = ndo.sample(hg, opr, sub)
    assert np.array_equal(first[:sub].cpu().numpy(), exp["out"])
    lo, n = 9_000_000, 1 << 20                    # a slice from the middle of the vertex range
    init = np.arange(lo, lo + n, dtype=np.int32)
    assert ndo.check_sampled_vertices(hg, opr, n, init, first[lo:lo + n].cpu().numpy()) == 0
    mid = ndo.sample(hg, opr, 5000, first=lo, initial=init[:5000])
    assert np.array_equal(first[lo:lo + 5000].cpu().numpy(), mid["out"])


@pytest.mark.parametrize("sort_path", ["0", "1"])
@pytest.mark.parametrize("app", [8, 9])
def test_importance_sampling_on_2_20_vertices(nd, ndo, monkeypatch, app, sort_path):
    """FastGCN (degree^2) and LADIES importance sampling, 2 layers x 64, batches of 64 uniform
    seeds, on 2^20 vertices / 2^24 undirected edges; both union paths."""
    monkeypatch.setenv("ND_COLLECTIVE_SORT", sort_path)
    V, M = 1 << 20, 1 << 24
    g = nd.Graph.rmat(V, M, seed=0)
    hg = _host(ndo, g)
    S = 64 if sort_path == "0" else 8             # the sort pipeline takes seconds per batch at this size
    init = np.random.default_rng(11).integers(0, V, S * 64).astype(np.int32)
    pr = nd.app_params(app, steps=2, fanout=64, batch=64, seed=2)
    opr = ndo.make_params(app, steps=2, fanout=64, batch=64, seed=2)
    s = nd.Sampler(g, pr, num_samples=S, initial=init)
    s.sample(1)
    got, aux = s.final_samples(), s.aux()
    exp = ndo.sample(hg, opr, S, initial=init)
    exp["first"] = 0
    flips = _compare_importance(ndo, hg, opr, S, init, got, aux["prob"], exp)
    print(f"app {app} sort={sort_path}: {flips} CDF-boundary flips of {S * 128} draws")
    assert flips <= 1 + S * 128 // 2000
    assert ndo.check_adjacency(hg, opr, S, init, got, aux["adj_row"], aux["adj_col"]) == 0
