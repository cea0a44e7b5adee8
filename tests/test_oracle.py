"""CPU tests of the oracle: pins it to the published Philox known-answer vectors, to the golden
fixtures produced by the reference's own next() bodies, and (where oracle/_ref is built) to those
bodies directly."""
import ctypes as C
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _gold(name):
    return np.load(os.path.join(GOLD, name + ".npz"))


def _gold_graph(ndo):
    z = _gold("graph_rmat300")
    return ndo.HostGraph(z["row_ptr"], z["col"], z["w"], z["max_w"])


def test_philox_known_answers(ndo):
    """Known-answer vectors published with the Philox4x32-10 algorithm (Random123 kat_vectors)."""
    L = ndo.lib()

    def ph(ctr, key):
        c = (C.c_uint32 * 4)(*ctr)
        k = (C.c_uint32 * 2)(*key)
        o = (C.c_uint32 * 4)()
        L.ndo_philox4x32_10(c, k, o)
        return list(o)

    assert ph([0] * 4, [0] * 2) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert ph([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert ph([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]


def test_uniform_range_and_rand_int(ndo):
    L = ndo.lib()
    assert L.ndo_u32_to_uniform(0) > 0.0
    assert L.ndo_u32_to_uniform(0xffffffff) == 1.0
    assert L.ndo_rand_int(1.0, 7) == 6          # u == 1 clamps to n-1 (rand_num_gen.cuh:120)
    assert L.ndo_rand_int(L.ndo_u32_to_uniform(0), 7) == 0
    # lanes of one Philox block are consecutive draws of the same (sample, step, slot)
    a = [L.ndo_draw_u32(9, 3, 2, 1, d) for d in range(8)]
    assert len(set(a)) == 8


@pytest.mark.parametrize("name", ["uniform_walk", "deepwalk", "ppr", "node2vec", "khop", "fastgcn_ref", "ladies_ref"])
def test_oracle_matches_golden(ndo, name):
    z = _gold(name)
    g = _gold_graph(ndo)
    app, steps, S = int(z["app"]), int(z["steps"]), int(z["S"])
    pr = ndo.make_params(app, steps=None if app == ndo.APP_KHOP else steps, seed=int(z["seed"]))
    r = ndo.sample(g, pr, S, first=int(z["first"]))
    assert np.array_equal(r["out"], z["out"])
    assert r["counters"]["sampled_edges"] == int(z["sampled_edges"])
    if "adj_row" in z:
        assert np.array_equal(r["adj_row"], z["adj_row"])
        assert np.array_equal(r["adj_col"], z["adj_col"])


def test_oracle_loader_matches_golden(ndo):
    z = _gold("loader_rmat300")
    g = ndo.csr_from_records(z["src"], z["dst"], z["w"])
    assert g.V == z["row_ptr"].shape[0] - 1 == 299   # vertex count = max id + 1 (graph.hpp:131-142)
    assert np.array_equal(g.row_ptr, z["row_ptr"])
    assert np.array_equal(g.col, z["col"])
    assert np.array_equal(g.w, z["wout"])
    assert np.array_equal(g.max_w, z["max_w"])


@pytest.mark.parametrize("app", [0, 1, 2, 3, 4, 6, 7])
def test_oracle_matches_reference_bodies(ndo, small_graph, app):
    if not ndo.ref_available():
        pytest.skip("oracle/_ref not built (reference tree absent)")
    S = 6 if app >= 6 else 500
    steps = {0: 37, 1: 37, 2: 100, 3: 37, 4: 2, 6: 3, 7: 5}[app]
    pr = ndo.make_params(app, steps=None if app == 4 else steps, seed=77)
    a = ndo.sample(small_graph, pr, S, first=123)
    r = ndo.ref_sample(small_graph, app, steps, S, first=123, seed=77)
    assert np.array_equal(a["out"], r["out"])
    assert a["counters"]["sampled_edges"] == r["sampled_edges"]
    if app >= 6:
        assert np.array_equal(a["adj_row"], r["adj_row"]) and np.array_equal(a["adj_col"], r["adj_col"])


def test_tiny_graph_walks_by_hand(ndo, tiny_graph):
    g = tiny_graph
    pr = ndo.make_params(ndo.APP_UNIFORM_WALK, steps=6, seed=1)
    r = ndo.sample(g, pr, 10)
    out = r["out"]
    assert (out[8] == g.V).all() and (out[9] == g.V).all()      # isolated: nothing sampled, INVALID = V
    assert set(out[0]) <= {0, 1, 2} and out[0][0] == 1           # vertex 0 has the single neighbour 1
    assert set(out[6]) <= {6, 7}
    assert ndo.check_sampled_vertices(g, pr, 10, r["initial"], out) == 0
    bad = out.copy()
    bad[0][0] = 4                                                  # 0-4 is not an edge
    assert ndo.check_sampled_vertices(g, pr, 10, r["initial"], bad) > 0


def test_ppr_stop_probability(ndo, small_graph):
    pr = ndo.make_params(ndo.APP_PPR, steps=100, stop_prob=0.15, seed=3)
    r = ndo.sample(small_graph, pr, 2000)
    deg = small_graph.degree()[:2000]
    lens = (r["out"] != small_graph.V).sum(1)
    assert (lens[deg == 0] == 0).all()
    live = lens[deg > 0]
    # a walk that never hits a dead end survives a step with probability 0.85
    assert 3.0 < live.mean() < 7.0
    assert ndo.check_sampled_vertices(small_graph, pr, 2000, r["initial"], r["out"]) == 0


def test_khop_distinct_properties(ndo, small_graph):
    g = small_graph
    pr = ndo.make_params(ndo.APP_KHOP_DISTINCT, fanout=[25, 10], seed=5)
    r = ndo.sample(g, pr, 300)
    out, hop = r["out"], r["hop_counts"].reshape(300, 2)
    for s in range(300):
        for off, n, c in ((0, 25, hop[s, 0]), (25, 250, hop[s, 1])):
            seg = out[s, off:off + n]
            assert (seg[c:] == g.V).all()
            assert (np.diff(seg[:c]) > 0).all()                    # ascending and unique
        d = g.degree()[s]
        assert hop[s, 0] == min(len(set(g.col[g.row_ptr[s]:g.row_ptr[s + 1]])), 25) or d > 25
    assert ndo.check_sampled_vertices(g, pr, 300, r["initial"], out) == 0


def test_importance_sampling_properties(ndo, small_graph):
    g = small_graph
    for app in (ndo.APP_FASTGCN_IS, ndo.APP_LADIES_IS):
        pr = ndo.make_params(app, steps=2, fanout=16, batch=8, seed=2)
        r = ndo.sample(g, pr, 50)
        assert ndo.check_adjacency(g, pr, 50, r["initial"], r["out"], r["adj_row"], r["adj_col"]) == 0
        out = r["out"]
        init = r["initial"].reshape(50, 8)
        for s in range(50):
            union = set()
            for t in init[s]:
                union |= set(g.col[g.row_ptr[t]:g.row_ptr[t + 1]])
            lay0 = out[s, :16]
            assert all((v in union) or v == g.V for v in lay0)
        p = r["prob"]
        assert ((p >= 0) & (p <= 1)).all()


def test_invert_map_and_distinct(ndo):
    rng = np.random.default_rng(0)
    keys = rng.integers(0, 50, 1000).astype(np.int32)
    keys[::7] = 50
    vals = np.arange(1000, dtype=np.int32)
    ko, vo = ndo.invert_map(keys, vals, 50)
    live = keys != 50
    order = np.argsort(keys[live], kind="stable")
    assert np.array_equal(ko, keys[live][order]) and np.array_equal(vo, vals[live][order])
    seg = np.array([5, 3, 50, 3, 9, 5, -1], np.int32)
    n = ndo.lib().ndo_distinct(seg.ctypes.data_as(C.c_void_p), 7, 50)
    assert n == 3 and list(seg) == [3, 5, 9, 50, 50, 50, 50]


def test_partition_covers_graph(ndo, small_graph):
    g = small_graph
    for budget in (4096, 20000, 10 ** 9):
        fv, lv, fe, le = ndo.partition(g, budget)
        assert fv[0] == 0 and lv[-1] == g.V - 1 and fe[0] == 0 and le[-1] == g.E - 1
        assert (fe[1:] == le[:-1] + 1).all()
        nbytes = (le - fe + 1) * 4 + (lv - fv + 1) * 16
        assert (nbytes <= budget + 16).all()
    fv, lv, fe, le = ndo.partition(g, 10 ** 9)
    assert len(fv) == 1


def test_rmat_is_deterministic_and_symmetric(ndo):
    s1, d1, w1 = ndo.rmat_records(1000, 5000, seed=4)
    s2, d2, w2 = ndo.rmat_records(1000, 5000, seed=4)
    assert np.array_equal(s1, s2) and np.array_equal(d1, d2) and np.array_equal(w1, w2)
    assert np.array_equal(s1[0::2], d1[1::2]) and np.array_equal(d1[0::2], s1[1::2])
    assert (s1 != d1).all() and s1.max() < 1000 and (w1 >= 1).all() and (w1 < 5).all()
    s3, _, _ = ndo.rmat_records(1000, 5000, seed=5)
    assert not np.array_equal(s1, s3)
