"""GPU parity tests of the single operators behind the C ABI: keyed Philox draws, the map
inversion (radix sort), the dedup kernel, and the device graph pipeline (R-MAT generator, CSR
build from edge records, partitioner).  Bit-exact against the oracle."""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_philox_draws_match_oracle(nd, ndo):
    import torch
    rng = np.random.default_rng(0)
    n = 5000
    t4 = rng.integers(0, 2 ** 32, size=(n, 4), dtype=np.uint64).astype(np.uint32)
    t4[:, 3] %= 11
    t4[0] = (0, 0, 0, 0)
    t4[1] = (0xffffffff, 0xffffffff, 0xffffffff, 7)
    d_t = _dev(t4.view(np.int32))
    d_o = torch.empty(n, dtype=torch.float32, device="cuda")
    seed = 0x1234567887654321
    nd.check(nd.lib.nd_philox_uniform(0, seed, n, d_t.data_ptr(), d_o.data_ptr()))
    got = d_o.cpu().numpy()
    L = ndo.lib()
    exp = np.array([L.ndo_uniform(seed, int(a), int(b), int(c), int(d)) for a, b, c, d in t4], np.float32)
    assert np.array_equal(got, exp)


@pytest.mark.parametrize("n,vmax", [(1, 5), (100, 3), (2048, 70000), (2049, 2 ** 16), (50_000, 2 ** 20),
                                    (1_000_003, 2 ** 20), (6_000_000, 2 ** 24)])
def test_invert_map_matches_oracle(nd, ndo, n, vmax):
    import torch
    rng = np.random.default_rng(n)
    keys = rng.integers(0, vmax, n).astype(np.int32)
    # skew: a hub, plus dead pairs that must vanish
    keys[rng.random(n) < 0.2] = vmax // 3
    keys[rng.random(n) < 0.1] = vmax
    vals = rng.permutation(n).astype(np.int32)
    ek, ev = ndo.invert_map(keys, vals, vmax)
    dk, dv = _dev(keys), _dev(vals)
    ok, ov = torch.empty_like(dk), torch.empty_like(dv)
    live = C.c_int64(-1)
    nd.check(nd.lib.nd_invert_map(0, n, dk.data_ptr(), dv.data_ptr(), vmax, ok.data_ptr(), ov.data_ptr(), C.byref(live)))
    assert live.value == ek.shape[0]
    assert np.array_equal(ok.cpu().numpy()[:live.value], ek)
    assert np.array_equal(ov.cpu().numpy()[:live.value], ev)      # stable: equal keys keep their order


def test_stream_ordered_inverter_matches_oracle(nd, ndo):
    """nd_inverter_run: the scratch allocated once, calls of different sizes back to back on a
    caller stream without any wait in between, the live count read from the device afterwards."""
    import torch
    vmax, cap = 5000, 300_000
    inv = C.c_void_p()
    nd.check(nd.lib.nd_inverter_create(0, cap, vmax, C.byref(inv)))
    st = torch.cuda.Stream()
    rng = np.random.default_rng(3)
    jobs = []
    with torch.cuda.stream(st):
        for n in (cap, 1, 77_777, 2048):
            keys = rng.integers(0, vmax + 1, n).astype(np.int32)      # vmax itself = dead pairs
            vals = rng.permutation(n).astype(np.int32)
            dk, dv = _dev(keys), _dev(vals)
            ok, ov = torch.empty_like(dk), torch.empty_like(dv)
            d_live = C.c_void_p()
            nd.check(nd.lib.nd_inverter_run(inv, st.cuda_stream, n, dk.data_ptr(), dv.data_ptr(), ok.data_ptr(), ov.data_ptr(),
                                            C.byref(d_live)))
            live = torch.empty(1, dtype=torch.int32, device="cuda")   # the count of THIS run, copied in stream order
            src = torch.as_tensor(_DevInt(d_live.value), device="cuda")
            live.copy_(src)
            jobs.append((keys, vals, ok, ov, live, dk, dv))
    st.synchronize()
    for keys, vals, ok, ov, live, _, _ in jobs:
        ek, ev = ndo.invert_map(keys, vals, vmax)
        n_live = int(live.item())
        assert n_live == ek.shape[0]
        assert np.array_equal(ok.cpu().numpy()[:n_live], ek) and np.array_equal(ov.cpu().numpy()[:n_live], ev)
    assert nd.lib.nd_inverter_run(inv, st.cuda_stream, cap + 1, 1, 1, 1, 1, None) != 0      # beyond the capacity: refused
    nd.check(nd.lib.nd_inverter_destroy(inv))


class _DevInt:
    """One int32 in device memory owned by the library, as a CUDA array."""

    def __init__(self, ptr):
        self.__cuda_array_interface__ = {"shape": (1,), "typestr": "<i4", "data": (int(ptr), False), "version": 3}


def test_sampler_reports_its_kernel_and_live_pairs(nd, ndo, small_graph):
    g = nd.Graph.from_csr(small_graph.row_ptr, small_graph.col, small_graph.w, small_graph.max_w)
    pr = nd.app_params(0, steps=10, seed=1)
    s = nd.Sampler(g, pr, num_samples=3000)
    buf = C.create_string_buffer(128)
    names = []
    for mode in (0, 1, 2):
        nd.check(nd.lib.nd_sampler_next_kernel(s._h, mode, buf, 128))
        names.append(buf.value.decode())
    assert names == ["walk_next_tp_kernel<uniform walk>", "walk_next_count_kernel<uniform walk>", "walk_sp_kernel<uniform walk>"]
    s.sample(1)
    live = s.live_pairs()
    exp = ndo.sample(small_graph, ndo.make_params(0, steps=10, seed=1), 3000)
    assert int(live.sum()) == exp["counters"]["live_pairs"]
    deg = small_graph.degree()
    assert live[0] == 3000 and live[1] == int((deg[np.arange(3000) % small_graph.V] > 0).sum())


def test_invert_map_all_dead_and_empty(nd):
    import torch
    live = C.c_int64(-1)
    nd.check(nd.lib.nd_invert_map(0, 0, None, None, 10, None, None, C.byref(live)))
    assert live.value == 0
    k = torch.full((300,), 10, dtype=torch.int32, device="cuda")
    v = torch.arange(300, dtype=torch.int32, device="cuda")
    ok, ov = torch.empty_like(k), torch.empty_like(v)
    nd.check(nd.lib.nd_invert_map(0, 300, k.data_ptr(), v.data_ptr(), 10, ok.data_ptr(), ov.data_ptr(), C.byref(live)))
    assert live.value == 0


@pytest.mark.parametrize("seg_len", [1, 25, 32, 250, 275, 1000])
def test_distinct_segments_match_oracle(nd, ndo, seg_len):
    import torch
    rng = np.random.default_rng(seg_len)
    nseg, inv = 777, 5000
    data = rng.integers(0, 60 if seg_len > 8 else 3, (nseg, seg_len)).astype(np.int32) * 83 % inv
    data[rng.random((nseg, seg_len)) < 0.15] = inv
    data[0, :] = inv                       # empty segment
    data[1, :] = 7                         # one value repeated
    exp = data.copy()
    cnt = np.array([ndo.lib().ndo_distinct(exp[i].ctypes.data_as(C.c_void_p), seg_len, inv) for i in range(nseg)], np.int32)
    d = _dev(data)
    dc = torch.zeros(nseg, dtype=torch.int32, device="cuda")
    nd.check(nd.lib.nd_distinct_segments(0, d.data_ptr(), nseg, seg_len, inv, dc.data_ptr()))
    assert np.array_equal(d.cpu().numpy(), exp)
    assert np.array_equal(dc.cpu().numpy(), cnt)


@pytest.mark.parametrize("V,M", [(300, 1500), (56944, 400_000), (1 << 17, 1 << 20)])
def test_rmat_graph_matches_oracle(nd, ndo, V, M):
    g = nd.Graph.rmat(V, M, seed=0)
    eg = ndo.rmat_graph(V, M, seed=0)
    assert (g.V, g.E) == (eg.V, eg.E)
    row_ptr, col, w, mw = g.to_host()
    assert np.array_equal(row_ptr, eg.row_ptr)
    assert np.array_equal(col, eg.col)
    assert np.array_equal(w, eg.w)
    assert np.array_equal(mw, eg.max_w)
    assert g.max_degree == int(eg.degree().max())


def test_csr_from_records_matches_reference_loader(nd, ndo, tmp_path):
    """Golden CSR produced by the reference's own host loader from shuffled records with duplicates."""
    z = np.load(os.path.join(GOLD, "loader_rmat300.npz"))
    g = nd.Graph.from_edge_records(z["src"], z["dst"], z["w"])
    row_ptr, col, w, mw = g.to_host()
    assert g.V == 299
    assert np.array_equal(row_ptr, z["row_ptr"]) and np.array_equal(col, z["col"])
    assert np.array_equal(w, z["wout"]) and np.array_equal(mw, z["max_w"])
    # and through the file loader (12-byte records, src/graph.hpp:126-129)
    path = str(tmp_path / "edges.bin")
    ndo.write_edge_list_binary(path, z["src"], z["dst"], z["w"])
    g2 = nd.Graph.load(path)
    assert np.array_equal(g2.to_host()[1], z["col"])
    with pytest.raises(nd.NdError) as e:
        nd.Graph.load(str(tmp_path / "missing.bin"))
    assert e.value.code == 3 and "not found" in str(e.value)


def test_csr_upload_computes_max_weight(nd, ndo, small_graph):
    g = nd.Graph.from_csr(small_graph.row_ptr, small_graph.col, small_graph.w)   # max_w left to the device
    assert np.array_equal(g.to_host()[3], small_graph.max_w)
    with pytest.raises(nd.NdError):
        nd.Graph.from_csr(np.array([1, 2], np.int32), np.array([0], np.int32), np.ones(1, np.float32))


def test_negative_weights_sort_like_the_reference(nd, ndo):
    src = np.array([0, 0, 0, 1, 0], np.int32)
    dst = np.array([1, 1, 1, 0, 1], np.int32)
    w = np.array([2.0, -1.0, 0.5, 1.0, -3.0], np.float32)
    g = nd.Graph.from_edge_records(src, dst, w)
    eg = ndo.csr_from_records(src, dst, w)
    _, col, wo, mw = g.to_host()
    assert np.array_equal(wo, eg.w) and list(wo[:4]) == [-3.0, -1.0, 0.5, 2.0]
    assert np.array_equal(mw, eg.max_w)


@pytest.mark.parametrize("budget", [100, 4096, 50_000, 10 ** 9])
def test_partition_matches_oracle(nd, ndo, small_graph, budget):
    g = nd.Graph.from_csr(small_graph.row_ptr, small_graph.col, small_graph.w, small_graph.max_w)
    got = g.partition(budget, max_parts=100000)
    exp = ndo.partition(small_graph, budget, max_parts=100000)
    for a, b in zip(got, exp):
        assert np.array_equal(a, b)


def test_text_loaders_match_reference_loaders(nd, tmp_path):
    """Golden CSRs produced by the reference's own text loaders (edge list: topology only, weights
    stored as 0; adjacency list: vertices renumbered by line, a vertex without edges still counts)."""
    z = np.load(os.path.join(GOLD, "loader_text.npz"))
    for kind, gtype, key in (("edge", "edge-list", "e_"), ("adj", "adj-list", "a_")):
        path = str(tmp_path / f"{kind}.txt")
        with open(path, "wb") as f:
            f.write(z[f"{kind}_txt"].tobytes())
        g = nd.Graph.load(path, gtype, "text")
        row_ptr, col, w, mw = g.to_host()
        assert np.array_equal(row_ptr, z[key + "row_ptr"]), kind
        assert np.array_equal(col, z[key + "col"]) and np.array_equal(w, z[key + "w"]) and np.array_equal(mw, z[key + "max_w"])
    with pytest.raises(nd.NdError) as e:
        nd.Graph.load(str(tmp_path / "edge.txt"), "adj-list", "binary")
    assert "not supported" in str(e.value)
    with pytest.raises(nd.NdError) as e:
        nd.Graph.load(str(tmp_path / "edge.txt"), "matrix-market", "text")
    assert "Incorrect graph file type" in str(e.value)


def test_random_gather_probe_reports_a_rate():
    """The measurement aid of bench.py (bench_probe.cu, its own small library)."""
    import ctypes as C
    import bench
    probe = C.CDLL(bench.build_probe())
    probe.nd_bench_random_gather.argtypes = [C.c_int, C.c_int64, C.c_int64, C.c_int, C.POINTER(C.c_double)]
    small, large = C.c_double(0), C.c_double(0)
    assert probe.nd_bench_random_gather(0, 8 << 20, 1 << 22, 3, C.byref(small)) == 0     # L2-resident array
    assert probe.nd_bench_random_gather(0, 1 << 30, 1 << 22, 3, C.byref(large)) == 0     # 1 GiB: DRAM
    assert small.value > large.value > 1e9
    assert probe.nd_bench_random_gather(0, 0, 1, 1, C.byref(small)) != 0                 # bad argument is an error, not a crash
