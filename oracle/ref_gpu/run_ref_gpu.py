"""Times the reference's own GPU build (oracle/_ref/ref_gpu_*, made by `make -C oracle ref_gpu`
from the reference's sources) on the synthetic graph of a bench workload.  Measurement
infrastructure, not part of the product.

The graph is generated on the GPU by the library's R-MAT generator, written as the reference's
binary edge list (12-byte records src, dst, weight -- src/graph.hpp:106-159), and each binary is
run as its own process; the figure reported is the reference's own "End to end time" print
(src/nextdoor.cu:2965, :3194: the step loop only) and its totalSampledVertices (:3299).

usage: python oracle/ref_gpu/run_ref_gpu.py [--workload c1|c2|c2u|c2d] [--timeout 300]
"""
import argparse
import json
import os
import re
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

BIN = {0: "ref_gpu_uniform", 1: "ref_gpu_deepwalk", 2: "ref_gpu_ppr", 3: "ref_gpu_node2vec", 4: "ref_gpu_khop"}


def write_edge_list(g, path):
    row_ptr, col, w, _ = g.to_host()
    src = np.repeat(np.arange(g.V, dtype=np.int32), np.diff(row_ptr))
    rec = np.empty(src.shape[0], dtype=[("s", "<i4"), ("d", "<i4"), ("w", "<f4")])
    rec["s"], rec["d"], rec["w"] = src, col, w
    rec.tofile(path)
    return src.shape[0]


def main():
    import bench
    from nextdoor_b200 import api as nd
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--timeout", type=int, default=300)
    a = ap.parse_args()
    wl = bench.WORKLOADS[a.workload]
    g = nd.Graph.rmat(wl["V"], wl["M"], 0, device=0)
    out = {"workload": a.workload, "V": g.V, "E": g.E, "runs": []}
    exe = os.path.join(ROOT, "oracle", "_ref", BIN[wl["app"]])
    if not os.path.exists(exe):
        print(json.dumps({"unavailable": f"{exe} not built"}))
        return
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "graph.bin")
        out["records"] = write_edge_list(g, path)
        del g
        for kernel, lb in (("TransitParallel", 0), ("TransitParallel", 1), ("SampleParallel", 0)):
            try:
                r = subprocess.run([exe, path, kernel, str(lb), "1"], capture_output=True, text=True, timeout=a.timeout)
            except subprocess.TimeoutExpired:
                out["runs"].append({"kernel": kernel, "lb": lb, "error": "timeout"})
                break  # do not start another run after one that did not end
            txt = r.stdout
            t = re.search(r"End to end time ([0-9.eE+-]+) secs", txt)
            n = re.search(r"totalSampledVertices (\d+)", txt)
            run = {"kernel": kernel, "lb": lb, "rc": r.returncode}
            if t and n and r.returncode == 0:
                run["end_to_end_s"] = float(t.group(1))
                run["sampled_vertices"] = int(n.group(1))
                run["edges_per_s"] = int(n.group(1)) / float(t.group(1)) if float(t.group(1)) > 0 else None
            else:
                run["error"] = (r.stderr or txt)[-300:]
            out["runs"].append(run)
            if r.returncode != 0:
                break  # a failed run of the reference is not repeated in another mode
    print(json.dumps(out))


if __name__ == "__main__":
    main()
