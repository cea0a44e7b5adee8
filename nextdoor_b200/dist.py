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


IDLE_WALK_WEIGHT = 1.0 / 7   # measured on the 2^24-vertex PPR job cut 4 and 8 ways: the value that levels the ranks' times


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
