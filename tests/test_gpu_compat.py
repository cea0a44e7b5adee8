"""GPU tests of the source-compatibility layer (include/nextdoor/): applications written against the
reference's App struct contract, compiled unchanged through those headers, must produce the oracle's
samples bit for bit in both kernel types.  Where the reference tree was present at build time the
reference's OWN application files (randomWalks.cu, khop.cu, example/uniformRandWalk.cu) are part of
the test library too."""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
OWN = os.path.join(HERE, "apps", "libnd_compat_apps.so")
WITH_REF = os.path.join(HERE, "apps", "_ref", "libnd_compat_ref.so")
KERNELS = [("TransitParallel", 0), ("TransitParallel", 1), ("SampleParallel", 0)]


@pytest.fixture(scope="module")
def world(ndo, tmp_path_factory):
    src, dst, w = ndo.rmat_records(1500, 9000, seed=8)
    path = str(tmp_path_factory.mktemp("compat") / "graph.bin")
    ndo.write_edge_list_binary(path, src, dst, w)
    return path, ndo.csr_from_records(src, dst, w)   # vertex count = max id + 1, as the loader decides


def _lib(path):
    L = C.CDLL(path)
    L.ndc_run.restype = C.c_int
    L.ndc_run.argtypes = [C.c_int, C.c_char_p, C.c_char_p, C.c_int, C.c_void_p, C.c_int64, C.POINTER(C.c_int64),
                          C.POINTER(C.c_int), C.c_void_p, C.c_void_p]
    return L


def _run(L, which, path, kernel, lb, cap, adj=None):
    out = np.empty(cap, np.int32)
    n, fs = C.c_int64(0), C.c_int(0)
    ar = ac = None
    if adj:
        ar, ac = np.empty(adj, np.int32), np.empty(adj, np.int32)
    rc = L.ndc_run(which, path.encode(), kernel.encode(), lb, out.ctypes.data, cap, C.byref(n), C.byref(fs),
                   ar.ctypes.data if adj else None, ac.ctypes.data if adj else None)
    assert rc == 0, f"ndc_run({which}) failed with {rc}"
    return out[:n.value].reshape(-1, fs.value), ar, ac


@pytest.mark.parametrize("kernel,lb", KERNELS)
def test_own_apps_match_oracle(ndo, world, kernel, lb):
    path, hg = world
    L = _lib(OWN)
    V = hg.V
    cases = [
        (0, ndo.make_params(ndo.APP_UNIFORM_WALK, steps=40), 3 * V + 7),
        (1, ndo.make_params(ndo.APP_DEEPWALK, steps=30), 3 * V + 7),
        (2, ndo.make_params(ndo.APP_NODE2VEC, steps=25, p=0.5, q=2.0, n2v_ref_compat=0), 3 * V + 7),
        (3, ndo.make_params(ndo.APP_KHOP, fanout=[4, 3, 2]), V),
    ]
    for which, pr, S in cases:
        fs = ndo.final_sample_size(pr)
        got, _, _ = _run(L, which, path, kernel, lb, S * fs)
        exp = ndo.sample(hg, pr, S)["out"]
        assert got.shape == exp.shape
        assert np.array_equal(got, exp), f"app {which} kernel {kernel} lb {lb}"


@pytest.mark.parametrize("kernel,lb", KERNELS)
def test_explicit_transits_app(ndo, world, kernel, lb):
    """hasExplicitTransits / stepTransits: the next transit comes from the sample's own state.  The
    expected walks are restated here from the app's definition with the oracle's keyed draws."""
    path, hg = world
    L = _lib(OWN)
    V, steps, INV = hg.V, 12, hg.V
    got, _, _ = _run(L, 5, path, kernel, lb, V * steps)
    u = ndo.lib().ndo_uniform
    ri = ndo.lib().ndo_rand_int
    exp = np.full((V, steps), INV, np.int32)
    for s in range(V):
        roots = [(s * 7 + i * 13) % V for i in range(4)]
        last, transit = 0, roots[0]
        for step in range(steps):
            draw = 0
            rs, deg = hg.row_ptr[transit], hg.row_ptr[transit + 1] - hg.row_ptr[transit]
            if deg > 0:
                if deg == 1:
                    v = int(hg.col[rs])
                else:
                    v = int(hg.col[rs + ri(u(0, s, step, 0, draw), int(deg))])
                    draw += 1
                if step > 0:
                    roots[last] = v
                exp[s, step] = v
            if step < steps - 1:   # stepTransits draws from the pair's stream at a fixed offset (1 << 16)
                last = ri(u(0, s, step, 0, 1 << 16), 4)
                transit = roots[last]
    assert np.array_equal(got, exp)


def test_reference_multirw_modes_agree(ndo, world):
    """The reference's multiRW app (explicit transits, samples seeded with rand()) compiled unchanged:
    no oracle restates it, so the check is that its three execution modes produce the same walks and
    that every step is an edge of the graph from one of the sample's roots."""
    if not os.path.exists(WITH_REF):
        pytest.skip("built without the reference tree")
    path, hg = world
    L = _lib(WITH_REF)
    outs = [_run(L, 15, path, k, lb, hg.V * 100)[0] for k, lb in KERNELS]
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
    assert (outs[0] != hg.V).sum() > hg.V * 50


def test_own_collective_app_matches_oracle(ndo, world):
    path, hg = world
    L = _lib(OWN)
    pr = ndo.make_params(ndo.APP_FASTGCN_REF, steps=2, fanout=8, batch=8)
    S = 500
    got, ar, ac = _run(L, 4, path, "SampleParallel", 0, S * 16, adj=S * 128)
    exp = ndo.sample(hg, pr, S)
    assert np.array_equal(got, exp["out"])
    assert np.array_equal(ar, exp["adj_row"]) and np.array_equal(ac, exp["adj_col"])


@pytest.mark.parametrize("kernel,lb", KERNELS)
def test_reference_app_files_drop_in(ndo, world, kernel, lb):
    if not os.path.exists(WITH_REF):
        pytest.skip("built without the reference tree")
    path, hg = world
    L = _lib(WITH_REF)
    V = hg.V
    cases = [(10, ndo.APP_UNIFORM_WALK, V, None), (11, ndo.APP_DEEPWALK, 100 * V, None), (12, ndo.APP_PPR, 100 * V, None),
             (13, ndo.APP_NODE2VEC, 100 * V, None), (14, ndo.APP_KHOP, V, None),
             (16, ndo.APP_KHOP, V, [10, 25])]   # LayerSamplingApp = k-hop with fan-outs 10 then 25 (layerSampling.cu:3-8)
    for which, app, S, fan in cases:
        pr = ndo.make_params(app, fanout=fan)          # the reference's compile-time constants
        fs = ndo.final_sample_size(pr)
        got, _, _ = _run(L, which, path, kernel, lb, S * fs)
        exp = ndo.sample(hg, pr, S)["out"]
        assert np.array_equal(got, exp), f"reference app {which} kernel {kernel} lb {lb}"


def test_app_main_command_line(ndo, world, capfd):
    path, hg = world
    L = _lib(OWN)
    args = [b"app", b"-g", path.encode(), b"-t", b"edge-list", b"-f", b"binary", b"-n", b"1", b"-k", b"TransitParallel", b"-l"]
    argv = (C.c_char_p * len(args))(*args)
    assert L.ndc_app_main(len(args), argv) == 0
    outp = capfd.readouterr().out
    pr = ndo.make_params(ndo.APP_UNIFORM_WALK, steps=40)
    exp = ndo.sample(hg, pr, 3 * hg.V + 7)["counters"]["sampled_edges"]
    assert f"totalSampledVertices {exp}" in outp
    bad = [b"app", b"-g", b"/nonexistent.bin", b"-t", b"edge-list", b"-f", b"binary"]
    assert L.ndc_app_main(len(bad), (C.c_char_p * len(bad))(*bad)) == 0
    assert "not found" in capfd.readouterr().out


def _run_subgraph(L, fn, path, kernel, lb, hg):
    """Runs one of the reference's two subgraph apps and returns, per sample, its 32 vertices and
    the (row, col) pairs it appended to the COO side buffers."""
    f = getattr(L, fn)
    f.restype = C.c_int
    f.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p,
                  C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]
    max_s = hg.V  # both apps take about V/4 samples
    cap = int(hg.E) * 9
    rows, cols = np.full(cap, -1, np.int32), np.full(cap, -1, np.int32)
    pos, ln, verts = np.zeros(max_s, np.int32), np.zeros(max_s, np.int32), np.zeros(max_s * 32, np.int32)
    n = C.c_int64(0)
    rc = f(path.encode(), kernel.encode(), lb, cap, rows.ctypes.data, cols.ctypes.data, max_s, pos.ctypes.data,
           ln.ctypes.data, verts.ctypes.data, C.byref(n))
    assert rc == 0, f"{fn} failed with {rc}"
    S = n.value
    return S, verts[:S * 32].reshape(S, 32), [(rows[pos[i]:pos[i] + ln[i]], cols[pos[i]:pos[i] + ln[i]]) for i in range(S)]


@pytest.mark.skipif(not os.path.exists(WITH_REF), reason="built without the reference tree")
@pytest.mark.parametrize("kernel,lb", KERNELS)
def test_reference_mvs_app(world, kernel, lb):
    """src/apps/mvs/mvsSampling.cu compiled unchanged: every sample collects exactly the edges of
    its 32 batch vertices (what the reference's own checker, src/tests/multiGPU/mvs.cu:11-110, asks)."""
    path, hg = world
    L = C.CDLL(WITH_REF)
    S, verts, coo = _run_subgraph(L, "ndc_run_mvs", path, kernel, lb, hg)
    assert S == min(1500000, (hg.V * 8 + 31) // 32)
    for s in range(S):
        assert np.array_equal(verts[s], (s * 32 + np.arange(32)) % hg.V)
        exp = sorted((int(v), int(c)) for v in verts[s] for c in hg.col[hg.row_ptr[v]:hg.row_ptr[v + 1]])
        got = sorted(zip(coo[s][0].tolist(), coo[s][1].tolist()))
        assert got == exp, f"sample {s}"


@pytest.mark.skipif(not os.path.exists(WITH_REF), reason="built without the reference tree")
@pytest.mark.parametrize("kernel,lb", KERNELS)
def test_reference_clustergcn_app(world, kernel, lb):
    """src/apps/clustergcn/clusterGCNSampling.cu compiled unchanged (explicit transits, positions
    claimed with atomics in stepTransits): every sample holds the subgraph induced by its two
    clusters of 16 vertices, one entry per (v1, v2) pair that is an edge."""
    path, hg = world
    L = C.CDLL(WITH_REF)
    S, verts, coo = _run_subgraph(L, "ndc_run_cluster", path, kernel, lb, hg)
    n_clusters = hg.V // 16
    assert S == min(2000000, (hg.V * 8 + 31) // 32)
    spans = []
    for s in range(S):
        cl = [(s * 2 + i) % n_clusters for i in range(2)]
        assert np.array_equal(verts[s], np.concatenate([c * 16 + np.arange(16) for c in cl]))
        exp = sorted((int(v1), int(v2)) for v1 in verts[s] for v2 in verts[s]
                     if v2 in set(hg.col[hg.row_ptr[v1]:hg.row_ptr[v1 + 1]].tolist()))
        got = sorted(zip(coo[s][0].tolist(), coo[s][1].tolist()))
        assert got == exp, f"sample {s}"
