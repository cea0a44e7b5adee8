"""ctypes bindings of the CPU oracle (oracle/nd_oracle.c) and of the host build of the
reference's own app sources (oracle/_ref/libnd_ref.so).

TEST INFRASTRUCTURE ONLY: tests, the smoke check and the CPU-baseline leg of the benchmark may
import this module; the product package must not.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE_TREE = os.environ.get("NEXTDOOR_REFERENCE", "/root/reference")  # where the upstream sources lie, if present
ORACLE_SO = os.path.join(HERE, "libnd_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libnd_ref.so")

APP_UNIFORM_WALK, APP_DEEPWALK, APP_PPR, APP_NODE2VEC, APP_KHOP, APP_KHOP_DISTINCT = range(6)
APP_FASTGCN_REF, APP_LADIES_REF, APP_FASTGCN_IS, APP_LADIES_IS = 6, 7, 8, 9
MAX_FANOUT = 8


class Params(C.Structure):
    _fields_ = [
        ("app", C.c_int32),
        ("steps", C.c_int32),
        ("fanout", C.c_int32 * MAX_FANOUT),
        ("batch", C.c_int32),
        ("n2v_ref_compat", C.c_int32),
        ("p", C.c_float),
        ("q", C.c_float),
        ("stop_prob", C.c_float),
        ("seed", C.c_uint64),
    ]


class Graph(C.Structure):
    _fields_ = [
        ("V", C.c_int32),
        ("E", C.c_int64),
        ("row_ptr", C.c_void_p),
        ("col", C.c_void_p),
        ("w", C.c_void_p),
        ("max_w", C.c_void_p),
    ]


class Counters(C.Structure):
    _fields_ = [(n, C.c_int64) for n in (
        "sampled_edges", "next_calls", "weight_tries", "n2v_tries", "n2v_probes", "live_pairs",
        "union_ids", "union_unique")]

    def as_dict(self):
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


def make_params(app, steps=None, fanout=None, batch=64, p=2.0, q=0.5, stop_prob=0.01, seed=0,
                n2v_ref_compat=1):
    """Defaults are the reference's compile-time constants (randomWalks.cu:4,105,149-150;
    khop.cu:3-8; fastgcnSampling.cu:1-4)."""
    pr = Params()
    pr.app = app
    if app <= APP_NODE2VEC:
        pr.steps = 100 if steps is None else steps
        pr.fanout[0] = 1
    elif app in (APP_KHOP, APP_KHOP_DISTINCT):
        fan = list(fanout) if fanout is not None else [25, 10]
        pr.steps = len(fan) if steps is None else steps
        for i, f in enumerate(fan):
            pr.fanout[i] = f
    else:
        pr.steps = 5 if steps is None else steps
        pr.fanout[0] = 64 if fanout is None else (fanout if isinstance(fanout, int) else fanout[0])
    pr.batch = batch
    pr.p, pr.q, pr.stop_prob = p, q, stop_prob
    pr.seed = seed
    pr.n2v_ref_compat = n2v_ref_compat
    return pr


def build(force=False):
    """Compile the oracle (and, where the reference tree is present, oracle/_ref)."""
    if force or not os.path.exists(ORACLE_SO) or \
            os.path.getmtime(ORACLE_SO) < os.path.getmtime(os.path.join(HERE, "nd_oracle.c")):
        subprocess.run(["make", "-C", HERE, "libnd_oracle.so"], check=True, capture_output=True)
    if os.path.isdir(os.path.join(REFERENCE_TREE, "src")):
        subprocess.run(["make", "-C", HERE, "ref", "REF=" + REFERENCE_TREE], check=True, capture_output=True)
        # the reference's GPU code for sm_100 (timed beside the library by ref_gpu/run_ref_gpu.py);
        # a measurement leg only, so a compiler failure here does not fail the build
        subprocess.run(["make", "-C", HERE, "ref_gpu", "REF=" + REFERENCE_TREE], check=False, capture_output=True)


_lib = None
_ref = None


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_SO):
            build()
        L = C.CDLL(ORACLE_SO)
        L.ndo_uniform.restype = C.c_float
        L.ndo_uniform.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]
        L.ndo_draw_u32.restype = C.c_uint32
        L.ndo_draw_u32.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]
        L.ndo_u32_to_uniform.restype = C.c_float
        L.ndo_u32_to_uniform.argtypes = [C.c_uint32]
        L.ndo_rand_int.restype = C.c_int32
        L.ndo_rand_int.argtypes = [C.c_float, C.c_int32]
        L.ndo_rmat_records.argtypes = [C.c_int32, C.c_int64, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p]
        L.ndo_csr_from_records.restype = C.c_int32
        L.ndo_csr_from_records.argtypes = [C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                           C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.ndo_partition.argtypes = [C.c_int32, C.c_void_p, C.c_int64, C.c_int32] + [C.c_void_p] * 5
        L.ndo_final_sample_size.restype = C.c_int32
        L.ndo_initial_sample_size.restype = C.c_int32
        L.ndo_sample.restype = C.c_int
        L.ndo_sample.argtypes = [C.POINTER(Graph), C.POINTER(Params), C.c_int64, C.c_int64] + \
            [C.c_void_p] * 6 + [C.POINTER(Counters), C.c_int]
        L.ndo_invert_map.restype = C.c_int64
        L.ndo_invert_map.argtypes = [C.c_int64, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]
        L.ndo_distinct.restype = C.c_int32
        L.ndo_distinct.argtypes = [C.c_void_p, C.c_int32, C.c_int32]
        L.ndo_check_sampled_vertices.restype = C.c_int64
        L.ndo_check_sampled_vertices.argtypes = [C.POINTER(Graph), C.POINTER(Params), C.c_int64, C.c_void_p, C.c_void_p]
        L.ndo_check_adjacency.restype = C.c_int64
        L.ndo_check_adjacency.argtypes = [C.POINTER(Graph), C.POINTER(Params), C.c_int64] + [C.c_void_p] * 4
        L.ndo_max_threads.restype = C.c_int
        _lib = L
    return _lib


def ref_available():
    return os.path.exists(REF_SO)


def ref():
    """The reference's own next() bodies on the host (None where it was not built)."""
    global _ref
    if _ref is None and ref_available():
        R = C.CDLL(REF_SO)
        R.ref_sample.restype = C.c_int
        R.ref_sample.argtypes = [C.c_int32] + [C.c_void_p] * 4 + [C.c_int, C.c_int, C.c_int64, C.c_int64,
                                                                   C.c_uint64] + [C.c_void_p] * 5 + [C.c_int]
        R.ref_load_edge_list_binary.restype = C.c_int
        R.ref_load_edge_list_binary.argtypes = [C.c_char_p] + [C.c_void_p] * 6
        R.ref_max_threads.restype = C.c_int
        _ref = R
    return _ref


class HostGraph:
    """CSR on the host: row_ptr[V+1] (exclusive ends), col[E], w[E], max_w[V]."""

    def __init__(self, row_ptr, col, w, max_w):
        self.row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
        self.col = np.ascontiguousarray(col, dtype=np.int32)
        self.w = np.ascontiguousarray(w, dtype=np.float32)
        self.max_w = np.ascontiguousarray(max_w, dtype=np.float32)
        self.V = int(self.row_ptr.shape[0] - 1)
        self.E = int(self.col.shape[0])

    def cgraph(self):
        g = Graph()
        g.V, g.E = self.V, self.E
        g.row_ptr, g.col, g.w, g.max_w = _p(self.row_ptr), _p(self.col), _p(self.w), _p(self.max_w)
        return g

    def degree(self):
        return np.diff(self.row_ptr)


def rmat_records(V, M, seed=0):
    src = np.empty(2 * M, np.int32)
    dst = np.empty(2 * M, np.int32)
    w = np.empty(2 * M, np.float32)
    lib().ndo_rmat_records(V, M, seed, _p(src), _p(dst), _p(w))
    return src, dst, w


def csr_from_records(src, dst, w, V=0):
    src = np.ascontiguousarray(src, np.int32)
    dst = np.ascontiguousarray(dst, np.int32)
    w = np.ascontiguousarray(w, np.float32)
    n = src.shape[0]
    if V <= 0:
        V = lib().ndo_csr_from_records(n, _p(src), _p(dst), _p(w), 0, None, None, None, None)
    row_ptr = np.empty(V + 1, np.int32)
    col = np.empty(n, np.int32)
    wo = np.empty(n, np.float32)
    mw = np.empty(V, np.float32)
    lib().ndo_csr_from_records(n, _p(src), _p(dst), _p(w), V, _p(row_ptr), _p(col), _p(wo), _p(mw))
    return HostGraph(row_ptr, col, wo, mw)


def rmat_graph(V, M, seed=0):
    return csr_from_records(*rmat_records(V, M, seed), V=V)


def write_edge_list_binary(path, src, dst, w):
    """12-byte records {int32 src, int32 dst, float32 w}: the format of src/graph.hpp:126-129."""
    rec = np.empty(src.shape[0], dtype=[("s", "<i4"), ("d", "<i4"), ("w", "<f4")])
    rec["s"], rec["d"], rec["w"] = src, dst, w
    rec.tofile(path)


def final_sample_size(params):
    return int(lib().ndo_final_sample_size(C.byref(params)))


def initial_sample_size(params):
    return int(lib().ndo_initial_sample_size(C.byref(params)))


def default_initial(params, V, S, first=0):
    """initialSample of the reference apps: walks/k-hop start sample i at vertex i % V
    (randomWalks.cu:34, khop.cu:47); collective batches take consecutive ids
    (fastgcnSampling.cu:80-82)."""
    isz = initial_sample_size(params)
    idx = np.arange(first, first + S, dtype=np.int64)
    if isz == 1:
        return (idx % V).astype(np.int32)
    return ((idx[:, None] * isz + np.arange(isz)[None, :]) % V).astype(np.int32).reshape(-1)


def sample(g: HostGraph, params, S, first=0, initial=None, threads=0, want_adj=True):
    """Returns dict(out, adj_row, adj_col, prob, hop_counts, counters)."""
    fs = final_sample_size(params)
    if initial is None:
        initial = default_initial(params, g.V, S, first)
    initial = np.ascontiguousarray(initial, np.int32)
    out = np.empty(S * fs, np.int32)
    collective = params.app >= APP_FASTGCN_REF
    adj_row = adj_col = prob = hop = None
    if collective and want_adj:
        L, B = params.fanout[0], params.batch
        n = S * params.steps * max(L, B) * L
        adj_row = np.empty(n, np.int32)
        adj_col = np.empty(n, np.int32)
    if collective:
        prob = np.zeros(S * fs, np.float32)
    if params.app == APP_KHOP_DISTINCT:
        hop = np.zeros(S * params.steps, np.int32)
    ctr = Counters()
    cg = g.cgraph()
    rc = lib().ndo_sample(C.byref(cg), C.byref(params), S, first, _p(initial), _p(out), _p(adj_row),
                          _p(adj_col), _p(prob), _p(hop), C.byref(ctr), threads)
    if rc != 0:
        raise RuntimeError(f"ndo_sample failed: {rc}")
    return dict(out=out.reshape(S, fs), adj_row=adj_row, adj_col=adj_col, prob=prob,
                hop_counts=hop, counters=ctr.as_dict(), initial=initial)


def ref_sample(g: HostGraph, app, steps, S, first=0, seed=0, initial=None, threads=0, fs=None):
    R = ref()
    if R is None:
        raise RuntimeError("oracle/_ref is not built")
    pr = make_params(app, steps=steps if app not in (APP_KHOP,) else None, seed=seed)
    if fs is None:
        fs = final_sample_size(pr)
    if initial is None:
        initial = default_initial(pr, g.V, S, first)
    initial = np.ascontiguousarray(initial, np.int32)
    out = np.empty(S * fs, np.int32)
    adj_row = adj_col = None
    if app in (APP_FASTGCN_REF, APP_LADIES_REF):
        adj_row = np.empty(S * steps * 64 * 64, np.int32)
        adj_col = np.empty(S * steps * 64 * 64, np.int32)
    e = C.c_int64(0)
    rc = R.ref_sample(g.V, _p(g.row_ptr), _p(g.col), _p(g.w), _p(g.max_w), app, steps, S, first, seed,
                      _p(initial), _p(out), _p(adj_row), _p(adj_col), C.addressof(e), threads)
    if rc != 0:
        raise RuntimeError(f"ref_sample failed: {rc}")
    return dict(out=out.reshape(S, fs), adj_row=adj_row, adj_col=adj_col, sampled_edges=int(e.value))


def ref_load_edge_list_binary(path):
    R = ref()
    V = C.c_int32(0)
    E = C.c_int64(0)
    R.ref_load_edge_list_binary(path.encode(), C.addressof(V), C.addressof(E), None, None, None, None)
    row_ptr = np.empty(V.value + 1, np.int32)
    col = np.empty(E.value, np.int32)
    w = np.empty(E.value, np.float32)
    mw = np.empty(V.value, np.float32)
    R.ref_load_edge_list_binary(path.encode(), C.addressof(V), C.addressof(E), _p(row_ptr), _p(col), _p(w), _p(mw))
    return HostGraph(row_ptr, col, w, mw)


def ref_load_text(path, kind):
    """kind 1: text edge list, 2: text adjacency list -- through the reference's own loaders."""
    R = ref()
    R.ref_load_text.restype = C.c_int
    R.ref_load_text.argtypes = [C.c_char_p, C.c_int] + [C.c_void_p] * 6
    V = C.c_int32(0)
    E = C.c_int64(0)
    R.ref_load_text(path.encode(), kind, C.addressof(V), C.addressof(E), None, None, None, None)
    row_ptr = np.empty(V.value + 1, np.int32)
    col = np.empty(E.value, np.int32)
    w = np.empty(E.value, np.float32)
    mw = np.empty(V.value, np.float32)
    R.ref_load_text(path.encode(), kind, C.addressof(V), C.addressof(E), _p(row_ptr), _p(col), _p(w), _p(mw))
    return HostGraph(row_ptr, col, w, mw)


def invert_map(keys, vals, invalid):
    keys = np.ascontiguousarray(keys, np.int32)
    vals = np.ascontiguousarray(vals, np.int32)
    ko = np.empty_like(keys)
    vo = np.empty_like(vals)
    n = lib().ndo_invert_map(keys.shape[0], _p(keys), _p(vals), invalid, _p(ko), _p(vo))
    return ko[:n], vo[:n]


def check_sampled_vertices(g, params, S, initial, out):
    cg = g.cgraph()
    out = np.ascontiguousarray(out, np.int32)
    initial = np.ascontiguousarray(initial, np.int32)
    return int(lib().ndo_check_sampled_vertices(C.byref(cg), C.byref(params), S, _p(initial), _p(out)))


def check_adjacency(g, params, S, initial, out, adj_row, adj_col):
    cg = g.cgraph()
    return int(lib().ndo_check_adjacency(C.byref(cg), C.byref(params), S, _p(np.ascontiguousarray(initial, np.int32)),
                                         _p(np.ascontiguousarray(out, np.int32)), _p(adj_row), _p(adj_col)))


def partition(g, budget, max_parts=4096):
    fv = np.zeros(max_parts, np.int32)
    lv = np.zeros(max_parts, np.int32)
    fe = np.zeros(max_parts, np.int64)
    le = np.zeros(max_parts, np.int64)
    n = C.c_int32(0)
    lib().ndo_partition(g.V, _p(g.row_ptr), budget, max_parts, _p(fv), _p(lv), _p(fe), _p(le), C.addressof(n))
    k = n.value
    return fv[:k], lv[:k], fe[:k], le[:k]
