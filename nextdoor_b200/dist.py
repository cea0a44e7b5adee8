"""Multi-GPU plumbing of the sampling path: one process per GPU, graph replicated, samples
sharded by seed range, and only the final sample gather crossing NVLink (an NCCL all-gather).

The shard rule is the reference's (PartStartPointer / PartDivisionSize, src/utils.hpp:26-27):
rank i takes samples [i*(S/P), (i+1)*(S/P)), the last rank also takes the remainder; the results
are concatenated in rank order as getFinalSamples does (src/nextdoor.cu:3211-3237).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import api


class _DevicePtr:
    """Zero-copy view of a device buffer owned by the library."""

    def __init__(self, ptr, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<i4", "data": (int(ptr), False), "version": 3}


def shard(total: int, rank: int, world: int):
    return api.shard_range(total, rank, world)


def device_samples(sampler: "api.Sampler") -> torch.Tensor:
    """The sampler's final-sample array as a CUDA tensor [S, finalSampleSize] without a copy."""
    if sampler.S == 0:
        return torch.empty((0, sampler.fs), dtype=torch.int32, device="cuda")
    return torch.as_tensor(_DevicePtr(sampler.final_samples_device_ptr(), (sampler.S, sampler.fs)), device="cuda")


def all_gather_samples(local: torch.Tensor, total: int, group=None) -> torch.Tensor:
    """Concatenates the ranks' shards [count_r, fs] into [total, fs] on every rank.  Shards may
    differ in length (the last one holds the remainder): they are padded to the longest for the
    collective and trimmed afterwards."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    fs = local.shape[1]
    counts = [shard(total, r, world)[1] for r in range(world)]
    assert local.shape[0] == counts[rank], "local shard does not have the reference's shard size"
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


def gather_samples_start(local: torch.Tensor, total: int, full: torch.Tensor | None, dst: int = 0, group=None):
    """Starts the transfer of every rank's shard [count_r, fs] to rank `dst`, which places the shards
    in rank order in `full` [total, fs] -- the concatenation getFinalSamples makes across devices
    (src/nextdoor.cu:3211-3237), but landing on ONE rank instead of all of them.  Point-to-point
    sends and receives (NCCL or gloo); `full` is only used on `dst`.  Returns the list of pending
    work handles: wait for all of them before `full` is read or `local` is overwritten."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    first, count = shard(total, rank, world)
    assert local.shape[0] == count, "local shard does not have the reference's shard size"
    if rank == dst:
        assert full is not None and full.shape[0] == total
        if count:
            full[first:first + count].copy_(local, non_blocking=True)
        ops = []
        for r in range(world):
            f, c = shard(total, r, world)
            if r != dst and c > 0:
                ops.append(dist.P2POp(dist.irecv, full[f:f + c], r, group))
    else:
        ops = [dist.P2POp(dist.isend, local, dst, group)] if count > 0 else []
    return dist.batch_isend_irecv(ops) if ops else []


def gather_samples_to(local: torch.Tensor, total: int, dst: int = 0, group=None):
    """Blocking form: returns [total, fs] on rank `dst`, None elsewhere."""
    rank = dist.get_rank(group)
    full = torch.empty((total, local.shape[1]), dtype=local.dtype, device=local.device) if rank == dst else None
    for w in gather_samples_start(local.contiguous(), total, full, dst, group):
        w.wait()
    return full
