"""GPU parity tests of the collective-neighbourhood apps: the reference's FastGCN / LADIES next()
bit-exactly, the importance-sampling extension with float probabilities at 1e-5 relative and
CDF-boundary index flips counted (a flip is only accepted when the draw lies within the tolerance
of the boundary)."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
RTOL = 1e-5


def _graph(nd, hg):
    return nd.Graph.from_csr(hg.row_ptr, hg.col, hg.w, hg.max_w)


@pytest.mark.parametrize("name", ["fastgcn_ref", "ladies_ref"])
def test_ref_apps_match_golden(nd, name):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    zg = np.load(os.path.join(GOLD, "graph_rmat300.npz"))
    g = nd.Graph.from_csr(zg["row_ptr"], zg["col"], zg["w"], zg["max_w"])
    pr = nd.app_params(int(z["app"]), steps=int(z["steps"]), seed=int(z["seed"]))
    s = nd.Sampler(g, pr, num_samples=int(z["S"]), first_sample=int(z["first"]))
    s.sample(2)
    assert np.array_equal(s.final_samples(), z["out"])
    aux = s.aux()
    assert np.array_equal(aux["adj_row"], z["adj_row"]) and np.array_equal(aux["adj_col"], z["adj_col"])


@pytest.mark.parametrize("app", [6, 7])
@pytest.mark.parametrize("L,B,steps", [(64, 64, 5), (16, 8, 2), (8, 32, 3)])
def test_ref_apps_match_oracle(nd, ndo, small_graph, app, L, B, steps):
    g = _graph(nd, small_graph)
    S = 200
    pr = nd.app_params(app, steps=steps, fanout=L, batch=B, seed=4)
    opr = ndo.make_params(app, steps=steps, fanout=L, batch=B, seed=4)
    s = nd.Sampler(g, pr, num_samples=S, first_sample=9)
    s.sample(1)
    exp = ndo.sample(small_graph, opr, S, first=9)
    assert np.array_equal(s.final_samples(), exp["out"])
    aux = s.aux()
    assert np.array_equal(aux["adj_row"], exp["adj_row"]) and np.array_equal(aux["adj_col"], exp["adj_col"])
    assert s.stats()["sampled_edges"] == exp["counters"]["sampled_edges"]
    assert ndo.check_adjacency(small_graph, opr, S, exp["initial"], s.final_samples(), aux["adj_row"], aux["adj_col"]) == 0


def _compare_importance(ndo, hg, opr, S, init, got, gprob, exp):
    """Returns the number of index flips; raises if a mismatch is not explained by a draw within
    RTOL of a CDF boundary."""
    L = opr.fanout[0]
    eo, ep = exp["out"], exp["prob"].reshape(S, -1)
    gp = gprob.reshape(S, -1)
    flips = 0
    same = got == eo
    assert np.allclose(gp[same], ep[same], rtol=RTOL, atol=0), "probabilities beyond 1e-5 relative"
    bad = np.argwhere(~same)
    first_bad_step = {}
    for s, c in bad:
        step = c // L
        if s in first_bad_step and first_bad_step[s] < step:
            continue          # a later layer of a sample whose earlier layer flipped sees other transits
        first_bad_step.setdefault(s, step)
    for s, step in first_bad_step.items():
        # rebuild the layer's candidates and CDF in float64 and check the draw is at a boundary
        tr = init.reshape(S, -1)[s] if step == 0 else eo[s, (step - 1) * L:step * L]
        cand = sorted({int(v) for t in tr if t != hg.V for v in hg.col[hg.row_ptr[t]:hg.row_ptr[t + 1]]})
        if opr.app == ndo.APP_FASTGCN_IS:
            wt = np.array([float(hg.row_ptr[v + 1] - hg.row_ptr[v]) ** 2 for v in cand])
        else:
            acc = {v: 0.0 for v in cand}
            for t in tr:
                if t == hg.V:
                    continue
                ws = hg.w[hg.row_ptr[t]:hg.row_ptr[t + 1]].astype(np.float64)
                for v, x in zip(hg.col[hg.row_ptr[t]:hg.row_ptr[t + 1]], ws / ws.sum()):
                    acc[int(v)] += x * x
            wt = np.array([acc[v] for v in cand])
        cdf = np.cumsum(wt)
        for j in range(L):
            c = step * L + j
            if got[s, c] == eo[s, c]:
                continue
            u = ndo.lib().ndo_uniform(opr.seed, s + exp["first"], step, j, 0)
            target = float(u) * cdf[-1]
            k = int(np.searchsorted(cdf, target))
            near = min(abs(target - cdf[max(k - 1, 0)]), abs(target - cdf[min(k, len(cdf) - 1)]))
            assert near <= 4 * RTOL * cdf[-1], f"sample {s} layer {step} slot {j}: mismatch away from a CDF boundary"
            assert {int(got[s, c]), int(eo[s, c])} <= {cand[max(k - 1, 0)], cand[min(k, len(cand) - 1)], cand[min(k + 1, len(cand) - 1)]}
            flips += 1
    return flips


@pytest.fixture(params=["bitmap", "bitmap_global", "sort"])
def union_path(request, monkeypatch):
    """The importance samplers build the union as a bitmap with a bit per vertex -- in shared
    memory when it fits, else in global scratch (ND_COLLECTIVE_BITMAP_GLOBAL=1 forces that on small
    graphs) -- or with the radix-sort pipeline (ND_COLLECTIVE_SORT=1)."""
    monkeypatch.setenv("ND_COLLECTIVE_SORT", "1" if request.param == "sort" else "0")
    monkeypatch.setenv("ND_COLLECTIVE_BITMAP_GLOBAL", "1" if request.param == "bitmap_global" else "0")
    return request.param


@pytest.mark.parametrize("app", [8, 9])
@pytest.mark.parametrize("L,B,steps", [(64, 64, 2), (16, 8, 3)])
def test_importance_apps_match_oracle(nd, ndo, small_graph, union_path, app, L, B, steps):
    g = _graph(nd, small_graph)
    S, first = 300, 17
    pr = nd.app_params(app, steps=steps, fanout=L, batch=B, seed=6)
    opr = ndo.make_params(app, steps=steps, fanout=L, batch=B, seed=6)
    rng = np.random.default_rng(1)
    init = rng.integers(0, small_graph.V, S * B).astype(np.int32)
    init[3] = small_graph.V                                    # an invalid transit inside a batch
    init[B:2 * B] = int(np.argmax(small_graph.degree() == 0))   # a batch with an empty union
    s = nd.Sampler(g, pr, num_samples=S, first_sample=first, initial=init)
    s.sample(1)
    exp = ndo.sample(small_graph, opr, S, first=first, initial=init)
    exp["first"] = first
    got = s.final_samples()
    aux = s.aux()
    flips = _compare_importance(ndo, small_graph, opr, S, init, got, aux["prob"], exp)
    print(f"app {app}: {flips} CDF-boundary index flips out of {S * steps * L} draws")
    assert flips <= 1 + S * steps * L // 2000
    assert (got[1] == small_graph.V).all()
    assert ndo.check_adjacency(small_graph, opr, S, init, got, aux["adj_row"], aux["adj_col"]) == 0
    st = s.stats()
    if flips == 0:
        assert st["union_ids"] == exp["counters"]["union_ids"]
        assert st["union_unique"] == exp["counters"]["union_unique"]


@pytest.mark.parametrize("app", [8, 9])
def test_importance_apps_benchmark_shape(nd, ndo, union_path, app):
    """2 layers x 64, batches of 64 uniform seeds on a graph with hubs: chunked candidate buffers,
    every sampled vertex is in the union of the previous layer's neighbours."""
    hg = ndo.rmat_graph(1 << 16, 1 << 20, seed=5)
    g = _graph(nd, hg)
    S = 256
    init = np.random.default_rng(3).integers(0, hg.V, S * 64).astype(np.int32)
    pr = nd.app_params(app, steps=2, fanout=64, batch=64, seed=1)
    opr = ndo.make_params(app, steps=2, fanout=64, batch=64, seed=1)
    s = nd.Sampler(g, pr, num_samples=S, initial=init)
    s.sample(1)
    got = s.final_samples()
    aux = s.aux()
    exp = ndo.sample(hg, opr, S, initial=init)
    exp["first"] = 0
    flips = _compare_importance(ndo, hg, opr, S, init, got, aux["prob"], exp)
    print(f"app {app}: {flips} flips of {S * 128}")
    assert flips <= 1 + S * 128 // 2000
    assert ndo.check_adjacency(hg, opr, S, init, got, aux["adj_row"], aux["adj_col"]) == 0
