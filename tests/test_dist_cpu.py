"""World-size-2 test of the multi-rank host logic on CPU (gloo): shard ranges follow the
reference's rule, and the gathered shards equal the unsharded job.  The per-rank sampling is done
by the oracle here (no GPU in this test); the same plumbing runs over NCCL on the GPUs."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, total, fs_steps, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nextdoor_b200 import dist as nd_dist
    from oracle import ndo
    g = ndo.rmat_graph(500, 2500, seed=2)
    pr = ndo.make_params(ndo.APP_DEEPWALK, steps=fs_steps, seed=3)
    first, count = nd_dist.shard(total, rank, world)
    local = ndo.sample(g, pr, count, first=first)["out"]
    full = nd_dist.all_gather_samples(torch.from_numpy(local.copy()), total)
    one = nd_dist.gather_samples_to(torch.from_numpy(local.copy()), total, dst=0)     # the gather the benchmark times
    assert (one is None) == (rank != 0)
    # the same job cut where the work is balanced: walks from vertices without neighbours weigh little
    init = np.arange(total) % g.V
    has = np.diff(g.row_ptr)[init] > 0
    bounds = nd_dist.balanced_bounds(torch.from_numpy(np.where(has, 1.0, 1.0 / 16)), world)
    bf, bc = nd_dist.shard(total, rank, world, bounds)
    blocal = ndo.sample(g, pr, bc, first=bf)["out"]
    bfull = nd_dist.all_gather_samples(torch.from_numpy(blocal.copy()), total, bounds=bounds)
    bone = nd_dist.gather_samples_to(torch.from_numpy(blocal.copy()), total, dst=0, bounds=bounds)
    if rank == 0:
        whole = ndo.sample(g, pr, total)["out"]
        ret["ok"] = bool(np.array_equal(full.numpy(), whole)) and bool(np.array_equal(one.numpy(), whole))
        ret["ok_balanced"] = bool(np.array_equal(bfull.numpy(), whole)) and bool(np.array_equal(bone.numpy(), whole))
        ret["ranges"] = [nd_dist.shard(total, r, world) for r in range(world)]
        ret["bounds"] = list(bounds)
        ret["active"] = [int(has[bounds[r]:bounds[r + 1]].sum()) for r in range(world)]
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_ranks_gather_equals_single_job():
    from nextdoor_b200 import build
    build.build()
    for total in (1001, 1000):       # uneven: the last rank takes the remainder
        mgr = mp.Manager()
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, _free_port(), total, 12, ret), nprocs=2, join=True)
        assert ret["ok"]
        (f0, c0), (f1, c1) = ret["ranges"]
        assert (f0, c0) == (0, total // 2) and (f1, c1) == (total // 2, total - total // 2)
        assert ret["ok_balanced"]
        b, act = ret["bounds"], ret["active"]
        assert b[0] == 0 and b[2] == total and 0 < b[1] < total
        assert abs(act[0] - act[1]) <= 0.1 * sum(act) + 16      # the R-MAT ids put the isolated vertices at the high end


def test_balanced_bounds_edge_cases():
    from nextdoor_b200 import build
    build.build()
    from nextdoor_b200 import dist as nd_dist
    assert nd_dist.balanced_bounds(torch.ones(8), 4) == [0, 2, 4, 6, 8]
    assert nd_dist.balanced_bounds(torch.ones(0), 3) == [0, 0, 0, 0]
    assert nd_dist.balanced_bounds(torch.zeros(9), 3) == [0, 3, 6, 9]             # no weight at all: the equal ranges
    assert nd_dist.balanced_bounds(torch.tensor([0., 0, 0, 5, 0, 0]), 2) == [0, 4, 6]  # one heavy sample: it stays whole
    b = nd_dist.balanced_bounds(torch.tensor([1., 1, 1, 1, 0, 0, 0, 0, 0, 0]), 4)
    assert b == [0, 1, 2, 3, 10]
    w = torch.rand(1000, dtype=torch.float64)
    b = nd_dist.balanced_bounds(w, 7)
    assert b[0] == 0 and b[-1] == 1000 and all(x <= y for x, y in zip(b, b[1:]))
    sums = [float(w[b[i]:b[i + 1]].sum()) for i in range(7)]
    assert max(sums) - min(sums) <= 2.0                                            # within two samples' weight
    assert nd_dist.shard(1000, 3, 7, b) == (b[3], b[4] - b[3])


class _CpuOps:
    """The four device operations of nextdoor_b200.partitioned restated on CPU tensors, next()
    from the oracle's keyed draws (uniform walk), so that PartitionedWalker.run -- the routing code
    the GPUs run -- is driven without a GPU."""

    def __init__(self, ndo, rp, col, bounds, rank, seed):
        self.ndo, self.rp, self.col, self.bounds, self.rank, self.seed = ndo, rp, col, bounds, rank, seed

    def step_packed(self, step, wk):
        u, ri = self.ndo.lib().ndo_uniform, self.ndo.lib().ndo_rand_int
        out = torch.empty_like(wk)
        for i, x in enumerate(wk.tolist()):
            s, t = (x >> 32) & 0xffffffff, x & 0xffffffff
            assert self.bounds[self.rank] <= t < self.bounds[self.rank + 1], "a walker was routed to a rank that does not own its vertex"
            deg = int(self.rp[t + 1] - self.rp[t])
            out[i] = ((s << 32) | int(self.col[self.rp[t] + ri(u(self.seed, s, step, 0, 0), deg)])) if deg > 0 else -1
        return out

    @staticmethod
    def _dest(wk, by_sample, bounds):
        live = wk != -1
        key = ((wk >> 32) & 0xffffffff) if by_sample else (wk & 0xffffffff)
        return live, torch.bucketize(key, bounds[1:-1].contiguous(), right=True)

    def route_count(self, wk, by_sample, bounds, counts):
        live, dest = self._dest(wk, by_sample, bounds)
        counts.copy_(torch.bincount(dest[live], minlength=counts.shape[0]))

    def route_scatter(self, wk, by_sample, bounds, counts, n_out):
        live, dest = self._dest(wk, by_sample, bounds)
        out = wk[live][torch.argsort(dest[live], stable=True)]
        assert out.shape[0] == n_out
        return out

    def records_store(self, mine, step, first, count, steps, out):
        s, v = (mine >> 32) & 0xffffffff, mine & 0xffffffff
        assert bool(((s >= first) & (s < first + count)).all()), "a record arrived at a rank that is not its sample's home"
        out[s - first, step] = v.to(torch.int32)


def _partitioned_worker(rank, world, port, total, steps, ret):
    """The routing and bookkeeping of the partitioned walker over gloo."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nextdoor_b200 import api as nd
    from nextdoor_b200 import partitioned as ndp
    from oracle import ndo
    g = ndo.rmat_graph(300, 1500, seed=4)
    seed = 9
    bounds = ndp.split_bounds(g.row_ptr, world)
    rp, col, w = ndp.local_rows(g.row_ptr, g.col, g.w, int(bounds[rank]), int(bounds[rank + 1]))
    pr = nd.app_params(nd.APP_UNIFORM_WALK, steps=steps, seed=seed)
    walker = ndp.PartitionedWalker(rp, col, w, bounds, pr, device="cpu", ops=_CpuOps(ndo, rp, col, bounds, rank, seed))
    init = (np.arange(total) * 7 % g.V).astype(np.int32)
    init[5] = g.V          # an invalid seed: its row stays invalid
    out, first = walker.run(total, initial=init)
    exp = ndo.sample(g, ndo.make_params(ndo.APP_UNIFORM_WALK, steps=steps, seed=seed), total, initial=init)["out"]
    ok = np.array_equal(out.numpy(), exp[first:first + out.shape[0]])
    oks = [None] * world
    dist.all_gather_object(oks, bool(ok))
    if rank == 0:
        ret["ok"] = all(oks)
        ret["sent"] = walker.bytes_sent
    dist.destroy_process_group()


def test_partitioned_walk_two_ranks_equals_replicated_job():
    from nextdoor_b200 import build
    build.build()
    for world in (2, 3):
        mgr = mp.Manager()
        ret = mgr.dict()
        mp.spawn(_partitioned_worker, args=(world, _free_port(), 257, 15, ret), nprocs=world, join=True)
        assert ret["ok"]
        assert ret["sent"] > 0


def test_partition_helpers_cover_the_graph_exactly():
    """split_bounds / local_rows: the ranges tile [0, V), every CSR entry lands in exactly one
    part, and a part's rows are the graph's rows with the foreign rows empty."""
    sys.path.insert(0, ROOT)
    from nextdoor_b200 import partitioned as ndp
    from oracle import ndo
    g = ndo.rmat_graph(700, 5000, seed=6)
    for parts in (1, 2, 3, 8):
        b = ndp.split_bounds(g.row_ptr, parts)
        assert b[0] == 0 and b[-1] == g.V and (np.diff(b) >= 0).all()
        total = 0
        for r in range(parts):
            rp, col, w = ndp.local_rows(g.row_ptr, g.col, g.w, int(b[r]), int(b[r + 1]))
            assert rp.shape[0] == g.V + 1 and rp[0] == 0 and rp[-1] == col.shape[0] == w.shape[0]
            deg = np.diff(rp)
            assert (deg[: b[r]] == 0).all() and (deg[b[r + 1]:] == 0).all()
            assert np.array_equal(deg[b[r]: b[r + 1]], np.diff(g.row_ptr)[b[r]: b[r + 1]])
            assert np.array_equal(col, g.col[g.row_ptr[b[r]]: g.row_ptr[b[r + 1]]])
            total += col.shape[0]
        assert total == g.E
        sizes = [int(g.row_ptr[b[r + 1]] - g.row_ptr[b[r]]) for r in range(parts)]
        assert max(sizes) - min(sizes) <= 2 * int(np.diff(g.row_ptr).max())   # balanced up to one hub list
