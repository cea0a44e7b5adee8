"""Multi-GPU plumbing of the sampling path: one process per GPU, graph replicated, samples
sharded by seed range, and only the final sample gather crossing NVLink (an NCCL all-gather).

The shard rule is the reference's (PartStartPointer / PartDivisionSize, src/utils.hpp:26-27):
rank i takes samples [i*(S/P), (i+1)*(S/P)), the last rank also takes the remainder; the results
are concatenated in rank order as getFinalSamples does (src/nextdoor.cu:3211-3237).  Every function
also takes explicit cut points (`bounds`), which balanced_bounds computes from per-sample weights.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import api


class _DevicePtr:
    """Zero-copy view of a device buffer owned by the library."""

    def __init__(self, ptr, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<i4", "data": (int(ptr), False), "version": 3}


def shard(total: int, rank: int, world: int, bounds=None):
    """(first, count) of rank's seed range: the reference's equal ranges, or the cut points
    `bounds` (world + 1 ascending sample indices from 0 to total, e.g. from balanced_bounds)."""
    if bounds is None:
        return api.shard_range(total, rank, world)
    assert len(bounds) == world + 1 and bounds[0] == 0 and bounds[world] == total
    return int(bounds[rank]), int(bounds[rank + 1] - bounds[rank])


def balanced_bounds(weights, world: int):
    """Cut points of `world` CONTIGUOUS seed ranges of (nearly) equal total weight.

    The reference cuts a job into ranges of equal sample counts (src/utils.hpp:26-27).  When the
    cost of a sample depends on where it starts -- a walk from a vertex without neighbours ends at
    once, and graph generators and crawls put such vertices at one end of the id range -- equal
    counts leave the ranks with unequal work and the job waits for the slowest.  The draws are keyed
    by the global sample index, so any contiguous cut gives the same samples; this one balances
    `weights` (a 1-D tensor or array, one non-negative value per sample of the job).  Returns
    world + 1 Python ints; every rank computes the same cut from the same weights."""
    w = torch.as_tensor(weights)
    total = int(w.shape[0])
    if total == 0 or world == 1:
        return [0] + [total] * world
    c = torch.cumsum(w.to(torch.float64), 0)
    if float(c[-1]) <= 0:
        return [shard(total, r, world)[0] for r in range(world)] + [total]
    targets = c[-1] * torch.arange(1, world, dtype=torch.float64, device=c.device) / world
    cuts = torch.searchsorted(c, targets, right=False) + 1      # the sample that reaches the target stays on the left
    inner = [min(int(v), total) for v in cuts.tolist()]
    for i in range(1, len(inner)):
        inner[i] = max(inner[i], inner[i - 1])
    return [0] + inner + [total]


IDLE_WALK_WEIGHT = 1.0 / 20  # measured on the 2^24-vertex PPR job cut 4 and 8 ways: the value that levels the ranks' times


def walk_start_weights(graph: "api.Graph", initial, idle: float = IDLE_WALK_WEIGHT):
    """Per-sample weights for balanced_bounds of a walk job on a replicated graph: 1 for a walk
    whose start vertex has neighbours, `idle` for one that cannot start (it still costs its slot
    in the first step and its row of the result).  `initial`: the job's start vertices, a CUDA
    int tensor on the graph's device."""
    row_ptr = torch.as_tensor(_DevicePtr(graph.row_ptr_device_ptr(), (graph.V + 1,)), device=initial.device)
    v = initial.to(torch.int64).clamp(0, graph.V - 1)
    has = (row_ptr[v + 1] > row_ptr[v]) & (initial >= 0) & (initial < graph.V)
    return torch.where(has, 1.0, idle)


def device_samples(sampler: "api.Sampler") -> torch.Tensor:
    """The sampler's final-sample array as a CUDA tensor [S, finalSampleSize] without a copy."""
    if sampler.S == 0:
        return torch.empty((0, sampler.fs), dtype=torch.int32, device="cuda")
    return torch.as_tensor(_DevicePtr(sampler.final_samples_device_ptr(), (sampler.S, sampler.fs)), device="cuda")


def all_gather_samples(local: torch.Tensor, total: int, group=None, bounds=None) -> torch.Tensor:
    """Concatenates the ranks' shards [count_r, fs] into [total, fs] on every rank.  Shards may
    differ in length (the last one holds the remainder; balanced cuts differ throughout): they are
    padded to the longest for the collective and trimmed afterwards."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    fs = local.shape[1]
    counts = [shard(total, r, world, bounds)[1] for r in range(world)]
    assert local.shape[0] == counts[rank], "local shard does not have the size of its seed range"
    longest = max(counts)
    padded = local
    if local.shape[0] != longest:
        padded = torch.zeros((longest, fs), dtype=local.dtype, device=local.device)
        padded[: local.shape[0]] = local
    out = torch.empty((world * longest, fs), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, padded.contiguous(), group=group)
    if all(c == longest for c in counts):
        return out
    return torch.cat([out[r * longest: r * longest + counts[r]] for r in range(world)], dim=0)


def gather_samples_start(local: torch.Tensor, total: int, full: torch.Tensor | None, dst: int = 0, group=None, bounds=None):
    """Starts the transfer of every rank's shard [count_r, fs] to rank `dst`, which places the shards
    in rank order in `full` [total, fs] -- the concatenation getFinalSamples makes across devices
    (src/nextdoor.cu:3211-3237), but landing on ONE rank instead of all of them.  Point-to-point
    sends and receives (NCCL or gloo); `full` is only used on `dst`.  Returns the list of pending
    work handles: wait for all of them before `full` is read or `local` is overwritten."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    first, count = shard(total, rank, world, bounds)
    assert local.shape[0] == count, "local shard does not have the size of its seed range"
    if rank == dst:
        assert full is not None and full.shape[0] == total
        if count:
            full[first:first + count].copy_(local, non_blocking=True)
        ops = []
        for r in range(world):
            f, c = shard(total, r, world, bounds)
            if r != dst and c > 0:
                ops.append(dist.P2POp(dist.irecv, full[f:f + c], r, group))
    else:
        ops = [dist.P2POp(dist.isend, local, dst, group)] if count > 0 else []
    return dist.batch_isend_irecv(ops) if ops else []


def gather_samples_to(local: torch.Tensor, total: int, dst: int = 0, group=None, bounds=None):
    """Blocking form: returns [total, fs] on rank `dst`, None elsewhere."""
    rank = dist.get_rank(group)
    full = torch.empty((total, local.shape[1]), dtype=local.dtype, device=local.device) if rank == dst else None
    for w in gather_samples_start(local.contiguous(), total, full, dst, group, bounds):
        w.wait()
    return full


class PackedRowsGather:
    """The result of a sharded WALK job on rank `dst`, moved by row prefixes.

    getFinalSamples concatenates the devices' dense arrays (src/nextdoor.cu:3211-3237); for walks
    that end early almost every slot of those arrays is the invalid id.  Here every rank packs its
    rows' valid prefixes (nd_sampler_pack_rows), sends the row lengths and the packed vertices, and
    `dst` writes them into ITS dense [total, fs] array (nd_rows_unpack), which it keeps from job to
    job with a per-row length, so that a job rewrites only the slots a walk fills now or filled in
    the previous job.  `full` on `dst` ends up equal to the concatenation of the dense shards.

    Per job: h = start(sampler) right after sampler.sample(sync=False); later finish(h) -- it waits
    on the host for that sampler's packing only, so another sampler's job can be running on the
    device meanwhile -- and returns when `full` holds the job (the calling thread's current stream
    is synchronised) and the sampler may be run again."""

    def __init__(self, total: int, fs: int, invalid: int, dst: int = 0, group=None, bounds=None, device=None):
        self.group, self.dst, self.total, self.fs, self.invalid = group, dst, int(total), int(fs), int(invalid)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.ranges = [shard(self.total, r, self.world, bounds) for r in range(self.world)]
        self._comm_cpu = dist.get_backend(group) == "gloo"
        self.full = self.full_len = None
        self.values_moved = 0            # vertices of the last finished job, all ranks together
        if self.rank == dst:
            self.full = torch.full((self.total, self.fs), self.invalid, dtype=torch.int32, device=self.device)
            self.full_len = torch.zeros(self.total, dtype=torch.int32, device=self.device)
            longest = max(c for _, c in self.ranges)
            self._scratch = torch.empty(api.rows_scratch_words(longest), dtype=torch.int32, device=self.device)
            self._lens = {r: torch.empty(c, dtype=torch.int32, device=self.device)
                          for r, (_, c) in enumerate(self.ranges) if r != dst}
            self._vals = {r: torch.empty(0, dtype=torch.int32, device=self.device) for r in self._lens}

    def start(self, sampler: "api.Sampler"):
        assert sampler.S == self.ranges[self.rank][1], "the sampler does not hold this rank's seed range"
        len_ptr, vals_ptr = sampler.pack_rows()
        return sampler, len_ptr, vals_ptr

    def _view(self, ptr, n):
        return torch.as_tensor(_DevicePtr(ptr, (n,)), device=self.device) if n > 0 else torch.empty(0, dtype=torch.int32, device=self.device)

    def _unpack(self, r, len_ptr, vals_ptr):
        f, c = self.ranges[r]
        if c == 0:
            return
        api.rows_unpack(self.device.index, torch.cuda.current_stream(self.device).cuda_stream, c, self.fs, self.invalid,
                        len_ptr, vals_ptr, self.full[f:f + c].data_ptr(), self.full_len[f:f + c].data_ptr(),
                        self._scratch.data_ptr())

    def finish(self, handle):
        sampler, len_ptr, vals_ptr = handle
        n = sampler.pack_rows_total()
        mine = torch.tensor([n], dtype=torch.int64, device="cpu" if self._comm_cpu else self.device)
        totals = torch.empty(self.world, dtype=torch.int64, device=mine.device)
        dist.all_gather_into_tensor(totals, mine, group=self.group)
        totals = totals.tolist()
        self.values_moved = int(sum(totals))
        count = self.ranges[self.rank][1]
        if self.rank != self.dst:
            if count > 0:
                lens, vals = self._view(len_ptr, count), self._view(vals_ptr, n)
                if self._comm_cpu:
                    dist.send(lens.cpu(), self.dst, group=self.group)
                    if n > 0:
                        dist.send(vals.cpu(), self.dst, group=self.group)
                else:
                    ops = [dist.P2POp(dist.isend, lens, self.dst, self.group)]
                    if n > 0:
                        ops.append(dist.P2POp(dist.isend, vals, self.dst, self.group))
                    for w in dist.batch_isend_irecv(ops):
                        w.wait()
        else:
            for r in self._lens:                                   # room for the incoming vertices
                if totals[r] > self._vals[r].shape[0]:
                    self._vals[r] = torch.empty(int(totals[r]) + int(totals[r]) // 4 + 1024, dtype=torch.int32, device=self.device)
            if self._comm_cpu:
                for r, lens in self._lens.items():
                    if lens.shape[0] == 0:
                        continue
                    buf = torch.empty(lens.shape[0], dtype=torch.int32)
                    dist.recv(buf, r, group=self.group)
                    lens.copy_(buf)
                    if totals[r] > 0:
                        buf = torch.empty(int(totals[r]), dtype=torch.int32)
                        dist.recv(buf, r, group=self.group)
                        self._vals[r][:totals[r]].copy_(buf)
            else:
                ops = []
                for r, lens in self._lens.items():
                    if lens.shape[0] == 0:
                        continue
                    ops.append(dist.P2POp(dist.irecv, lens, r, self.group))
                    if totals[r] > 0:
                        ops.append(dist.P2POp(dist.irecv, self._vals[r][:totals[r]], r, self.group))
                works = dist.batch_isend_irecv(ops) if ops else []
                self._unpack(self.dst, len_ptr, vals_ptr)          # this rank's own rows meanwhile
                for w in works:
                    w.wait()
            if self._comm_cpu:
                self._unpack(self.dst, len_ptr, vals_ptr)
            for r, lens in self._lens.items():
                self._unpack(r, lens.data_ptr(), self._vals[r].data_ptr())
        torch.cuda.current_stream(self.device).synchronize()
