"""GPU tests of sampling over a PARTITIONED graph (nextdoor_b200.partitioned, nd_walk_step): the
result must equal the replicated sampler's / the oracle's bit for bit for any number of ranks,
because every draw is keyed by (global sample, step)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
APPS = [(0, {}), (1, {}), (2, {"stop_prob": 0.15})]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("app,extra", APPS)
def test_one_rank_equals_sampler_and_oracle(nd, ndo, app, extra):
    """world = 1: no routing, only nd_walk_step driven step by step."""
    from nextdoor_b200 import partitioned as ndp
    hg = ndo.rmat_graph(3000, 20000, seed=11)
    S, steps = 5000, 25
    pr = nd.app_params(app, steps=steps, seed=4, **extra)
    bounds = ndp.split_bounds(hg.row_ptr, 1)
    rp, col, w = ndp.local_rows(hg.row_ptr, hg.col, hg.w, 0, hg.V)
    walker = ndp.PartitionedWalker(rp, col, w, bounds, pr)
    out, first = walker.run(S)
    exp = ndo.sample(hg, ndo.make_params(app, steps=steps, seed=4, **extra), S)["out"]
    assert first == 0 and np.array_equal(out.cpu().numpy(), exp)
    g = nd.Graph.from_csr(hg.row_ptr, hg.col, hg.w, hg.max_w)
    smp = nd.Sampler(g, pr, num_samples=S)
    smp.sample(1)
    assert np.array_equal(smp.final_samples(), exp)


def _worker(rank, world, port, backend, app, extra, total, steps, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dev = rank if backend == "nccl" else 0      # gloo: the ranks share GPU 0, collectives go through host memory
    torch.cuda.set_device(dev)
    if backend == "nccl":
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", dev))
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    from nextdoor_b200 import api as nd
    from nextdoor_b200 import partitioned as ndp
    from oracle import ndo
    hg = ndo.rmat_graph(4000, 30000, seed=13)
    bounds = ndp.split_bounds(hg.row_ptr, world)
    rp, col, w = ndp.local_rows(hg.row_ptr, hg.col, hg.w, int(bounds[rank]), int(bounds[rank + 1]))
    pr = nd.app_params(app, steps=steps, seed=21, **extra)
    walker = ndp.PartitionedWalker(rp, col, w, bounds, pr, device=f"cuda:{dev}")
    init = (np.arange(total) * 13 % hg.V).astype(np.int32)
    out, first = walker.run(total, initial=init)
    exp = ndo.sample(hg, ndo.make_params(app, steps=steps, seed=21, **extra), total, initial=init)["out"]
    ok = bool(np.array_equal(out.cpu().numpy(), exp[first:first + out.shape[0]]))
    oks = [None] * world
    dist.all_gather_object(oks, ok)
    if rank == 0:
        ret["ok"] = all(oks)
        ret["entries"] = [int(bounds[r + 1] - bounds[r]) for r in range(world)]
    dist.destroy_process_group()


@pytest.mark.parametrize("app,extra", APPS)
def test_two_ranks_on_one_gpu(app, extra):
    """Two processes share GPU 0, each holding half of the graph's rows; the all-to-all runs over
    gloo through host memory."""
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), "gloo", app, extra, 6001, 20, ret), nprocs=2, join=True)
    assert ret["ok"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_nccl():
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), "nccl", 1, {}, 20001, 30, ret), nprocs=2, join=True)
    assert ret["ok"]
