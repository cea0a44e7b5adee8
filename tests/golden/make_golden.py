"""Generates the golden fixtures of tests/golden from the reference's OWN next() bodies compiled
for the host (oracle/_ref, which needs the reference tree at build time).  The fixtures are
self-contained: they hold the graph, the seeds and the outputs, so the tests need neither the
reference nor this script at run time.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import ndo  # noqa: E402

ndo.build()
assert ndo.ref_available(), "oracle/_ref is not built (reference tree absent?)"

g = ndo.rmat_graph(300, 1500, seed=3)
graph = dict(row_ptr=g.row_ptr, col=g.col, w=g.w, max_w=g.max_w)
np.savez_compressed(os.path.join(HERE, "graph_rmat300.npz"), **graph)

SEED = 11
cases = {
    "uniform_walk": (ndo.APP_UNIFORM_WALK, 20, 300),
    "deepwalk": (ndo.APP_DEEPWALK, 20, 300),
    "ppr": (ndo.APP_PPR, 100, 300),       # stop probability 0.01 is compiled into the reference
    "node2vec": (ndo.APP_NODE2VEC, 20, 300),
    "khop": (ndo.APP_KHOP, 2, 64),         # fan-out 25 then 10 is compiled into the reference
    "fastgcn_ref": (ndo.APP_FASTGCN_REF, 2, 2),
    "ladies_ref": (ndo.APP_LADIES_REF, 3, 2),
}
for name, (app, steps, S) in cases.items():
    r = ndo.ref_sample(g, app, steps, S, first=5, seed=SEED)
    out = dict(app=app, steps=steps, S=S, first=5, seed=SEED, out=r["out"], sampled_edges=r["sampled_edges"])
    if r["adj_row"] is not None:
        out["adj_row"], out["adj_col"] = r["adj_row"], r["adj_col"]
    np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **out)
    print(name, r["out"].shape, r["sampled_edges"])

# the reference's host loader on a binary edge list (duplicates, unsorted records)
src, dst, w = ndo.rmat_records(300, 1500, seed=3)
perm = np.random.default_rng(0).permutation(src.shape[0])
path = os.path.join(HERE, "_tmp_edges.bin")
ndo.write_edge_list_binary(path, src[perm], dst[perm], w[perm])
lg = ndo.ref_load_edge_list_binary(path)
os.remove(path)
np.savez_compressed(os.path.join(HERE, "loader_rmat300.npz"), src=src[perm], dst=dst[perm], w=w[perm],
                    row_ptr=lg.row_ptr, col=lg.col, wout=lg.w, max_w=lg.max_w)
print("loader", lg.V, lg.E)

# the reference's text loaders.  The edge-list file lists every vertex's edges in ascending
# neighbour order and names the largest id first (the reference neither sorts this format nor
# grows its vertex array for an id equal to the current size, src/graph.hpp:196-210).
rng = np.random.default_rng(4)
pairs = sorted({(int(a), int(b)) for a, b in rng.integers(0, 40, (300, 2)) if a != b})
pairs = [(39, 0)] + [p for p in pairs if p != (39, 0)]
# The file ends with a zero-weight triple: both loaders stop reading there (src/graph.hpp:199-202),
# which also keeps the reference from parsing past its unterminated read buffer (:171-178).
edge_txt = "".join(f"{a} {b} 1.5\n" for a, b in pairs) + "0 0 0\n"
path = os.path.join(HERE, "_tmp_edges.txt")
open(path, "w").write(edge_txt)
lg = ndo.ref_load_text(path, 1)
os.remove(path)
ids = [100 + 7 * i for i in range(25)]          # arbitrary ids, renumbered by line order
lines = []
for i, vid in enumerate(ids):
    nb = sorted(set(int(x) for x in rng.integers(0, 25, int(rng.integers(0, 6)))) - {i})
    lines.append(str(vid) + "".join(f" {ids[j]} {1 + 0.25 * ((i + j) % 9)}" for j in nb))
adj_txt = "\n".join(lines) + "\n"
path = os.path.join(HERE, "_tmp_adj.txt")
open(path, "w").write(adj_txt)
ag = ndo.ref_load_text(path, 2)
os.remove(path)
np.savez_compressed(os.path.join(HERE, "loader_text.npz"),
                    edge_txt=np.frombuffer(edge_txt.encode(), np.uint8), e_row_ptr=lg.row_ptr, e_col=lg.col, e_w=lg.w, e_max_w=lg.max_w,
                    adj_txt=np.frombuffer(adj_txt.encode(), np.uint8), a_row_ptr=ag.row_ptr, a_col=ag.col, a_w=ag.w, a_max_w=ag.max_w)
print("text loaders", lg.V, lg.E, ag.V, ag.E)
