"""A sharded walk job gathered on one rank by row prefixes (nextdoor_b200.dist.PackedRowsGather):
the packing and unpacking kernels on one GPU, then two ranks -- as two processes sharing GPU 0 over
gloo (transfers through host memory), and over NCCL where the box has two GPUs."""
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


def test_pack_and_unpack_round_trip_over_changing_passes(nd, ndo, small_graph):
    """nd_sampler_pack_rows -> nd_rows_unpack into a second dense array that is kept from pass to
    pass: it must equal the sampler's own result array after every pass (rows growing, shrinking
    and vanishing), and the packed total must be the number of sampled vertices."""
    g = nd.Graph.from_csr(small_graph.row_ptr, small_graph.col, small_graph.w, small_graph.max_w)
    V, S, steps = small_graph.V, 20_011, 40
    pr = nd.app_params(2, steps=steps, seed=5, stop_prob=0.15)
    s = nd.Sampler(g, pr, num_samples=S, first_sample=4)
    full = torch.full((S, steps), V, dtype=torch.int32, device="cuda")
    full_len = torch.zeros(S, dtype=torch.int32, device="cuda")
    scratch = torch.empty(nd.rows_scratch_words(S), dtype=torch.int32, device="cuda")
    rng = np.random.default_rng(3)
    for p, mode in enumerate((1, 2, 0, 1)):
        init = rng.integers(0, V, S).astype(np.int32)
        if p == 2:
            init[S // 3:] = -1
        s.set_initial(init)
        s.sample(mode)
        len_ptr, vals_ptr = s.pack_rows()
        total = s.pack_rows_total()
        dense = s.final_samples()
        assert total == int((dense != V).sum()) == s.stats()["sampled_edges"]
        nd.rows_unpack(0, None, S, steps, V, len_ptr, vals_ptr, full.data_ptr(), full_len.data_ptr(), scratch.data_ptr())
        torch.cuda.synchronize()
        assert np.array_equal(full.cpu().numpy(), dense), p
        assert np.array_equal(full_len.cpu().numpy(), (dense != V).sum(axis=1)), p
    k = nd.Sampler(g, nd.app_params(4, fanout=[3, 2], seed=1), num_samples=10)
    k.sample(1)
    with pytest.raises(nd.NdError):
        k.pack_rows()


def _worker(rank, world, port, backend, balanced, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dev = rank if backend == "nccl" else 0      # gloo: the ranks share GPU 0
    torch.cuda.set_device(dev)
    if backend == "nccl":
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", dev))
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    from nextdoor_b200 import api as nd
    from nextdoor_b200 import dist as nd_dist
    from oracle import ndo
    hg = ndo.rmat_graph(4000, 30000, seed=13)
    g = nd.Graph.from_csr(hg.row_ptr, hg.col, hg.w, hg.max_w, device=dev)
    total, steps = 30_001, 30
    pr = nd.app_params(2, steps=steps, seed=21, stop_prob=0.15)
    opr = ndo.make_params(2, steps=steps, seed=21, stop_prob=0.15)
    ok = True
    gather = None
    for p in range(3):                                   # three jobs with different seeds into the same gathered array
        init = ((np.arange(total) * (3 + 4 * p)) % hg.V).astype(np.int32)
        if p == 1:
            init[::2] = -1
        bounds = None
        if balanced:
            bounds = nd_dist.balanced_bounds(nd_dist.walk_start_weights(g, torch.from_numpy(init).cuda()), world)
            gather = None                                # the cut moves with the seeds: a new gathered array per job
        if gather is None:
            gather = nd_dist.PackedRowsGather(total, steps, hg.V, dst=0, bounds=bounds)
        f, c = nd_dist.shard(total, rank, world, bounds)
        smp = nd.Sampler(g, pr, num_samples=c, first_sample=f, initial=init[f:f + c])
        smp.sample(1, sync=False)
        gather.finish(gather.start(smp))
        if rank == 0:
            clean = np.where(init < 0, hg.V, init).astype(np.int32)
            exp = ndo.sample(hg, opr, total, initial=clean)
            ok = ok and bool(np.array_equal(gather.full.cpu().numpy(), exp["out"]))
            ok = ok and gather.values_moved == exp["counters"]["sampled_edges"]
        smp.free()
    oks = [None] * world
    dist.all_gather_object(oks, ok)
    if rank == 0:
        ret["ok"] = all(oks)
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("balanced", [False, True])
def test_two_ranks_on_one_gpu(balanced):
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), "gloo", balanced, ret), nprocs=2, join=True)
    assert ret["ok"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_nccl():
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), "nccl", True, ret), nprocs=2, join=True)
    assert ret["ok"]
