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
