"""Random walks over a graph that is PARTITIONED across the GPUs of a process group instead of
replicated: rank r holds the CSR rows of one contiguous vertex range, every step runs next() on
the walkers that currently stand on the rank's vertices (`nd_walk_step_packed`), and the survivors are
routed to the owners of their new vertices with one all-to-all.  At the end every (sample, step,
vertex) record travels to the sample's home rank (the reference's seed shards, src/utils.hpp:26-27)
with one more all-to-all.

This is the path the reference's CSR partitioner was written for (src/graph_partitioner.cuh:1-173)
but never got: its multi-GPU code replicates the graph (src/nextdoor.cu:1893-1911) and the
partitioned variant is a stub (ENABLE_GRAPH_PARTITION_FOR_GLOBAL_MEM, src/csr.hpp:371-374).  Because
every draw is keyed by (global sample, step), the result is bit-identical to the replicated
sampler's, whatever the number of ranks.

Supported applications: uniform walk, DeepWalk, PPR (a step needs only the transit's own row).
node2vec reads the adjacency of the PREVIOUS vertex, which lives on another rank, and is refused.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch
import torch.distributed as dist

from . import api
from ._lib import APP_DEEPWALK, APP_PPR, APP_UNIFORM_WALK, check, lib


def split_bounds(row_ptr, parts: int) -> np.ndarray:
    """Vertex boundaries b[0..parts] of `parts` contiguous ranges holding about E/parts CSR entries
    each (the reference's partitioner also cuts by size, src/graph_partitioner.cuh:40-110)."""
    row_ptr = np.asarray(row_ptr, np.int64)
    V, E = row_ptr.shape[0] - 1, int(row_ptr[-1])
    b = np.zeros(parts + 1, np.int64)
    for k in range(1, parts):
        b[k] = min(max(int(np.searchsorted(row_ptr, (E * k) // parts, side="left")), int(b[k - 1])), V)
    b[parts] = V
    return b


def local_rows(row_ptr, col, w, lo: int, hi: int):
    """The CSR of the vertex range [lo, hi) with GLOBAL vertex ids: a row-offset array of full
    length whose rows outside the range are empty, and only the range's entries of col / w."""
    row_ptr = np.asarray(row_ptr, np.int64)
    V = row_ptr.shape[0] - 1
    e0, e1 = int(row_ptr[lo]), int(row_ptr[hi])
    rp = np.zeros(V + 1, np.int32)
    rp[lo:hi + 1] = (row_ptr[lo:hi + 1] - e0).astype(np.int32)
    rp[hi + 1:] = e1 - e0
    return rp, np.ascontiguousarray(col[e0:e1], np.int32), np.ascontiguousarray(w[e0:e1], np.float32)


class _LibraryOps:
    """The four device operations of a partitioned step, as the library's kernels (C ABI)."""

    def __init__(self, graph, params, device, parts):
        self.graph, self.params, self.device, self.parts = graph, params, device, parts
        self._cursor = torch.zeros(parts, dtype=torch.int64, device=device)

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def step_packed(self, step, wk):
        nxt = torch.empty_like(wk)
        check(lib.nd_walk_step_packed(self.graph._h, C.byref(self.params), step, int(wk.shape[0]),
                                      C.c_void_p(wk.data_ptr()), C.c_void_p(nxt.data_ptr()), self._stream()))
        return nxt

    def finish(self):
        """Reads and clears the device status word of the step kernels (a rejection loop that hit
        its cap); waits for the stream."""
        status = C.c_int(0)
        check(lib.nd_walk_step_status(self.device.index, self._stream(), C.byref(status)))
        if status.value:
            raise RuntimeError(f"partitioned walk: device status word 0x{status.value:x} (a rejection loop hit its iteration cap)")

    def route_count(self, wk, by_sample, bounds, counts):
        check(lib.nd_route_count(self.device.index, int(wk.shape[0]), C.c_void_p(wk.data_ptr()), by_sample,
                                 C.c_void_p(bounds.data_ptr()), self.parts, C.c_void_p(counts.data_ptr()), self._stream()))

    def route_scatter(self, wk, by_sample, bounds, counts, n_out):
        out = torch.empty(n_out, dtype=torch.int64, device=self.device)
        check(lib.nd_route_scatter(self.device.index, int(wk.shape[0]), C.c_void_p(wk.data_ptr()), by_sample,
                                   C.c_void_p(bounds.data_ptr()), self.parts, C.c_void_p(counts.data_ptr()),
                                   C.c_void_p(self._cursor.data_ptr()), C.c_void_p(out.data_ptr()), self._stream()))
        return out

    def records_store(self, mine, step, first, count, steps, out):
        check(lib.nd_records_store(self.device.index, int(mine.shape[0]), C.c_void_p(mine.data_ptr()), step, first, count, steps,
                                   C.c_void_p(out.data_ptr()), self._stream()))


class PartitionedWalker:
    """One rank of a partitioned walk job.

    row_ptr_local / col_local / w_local: this rank's rows as returned by local_rows().
    bounds: the vertex boundaries of ALL ranks (split_bounds), identical on every rank.
    ops: an object with the four device operations (step_packed, route_count, route_scatter,
    records_store; see _LibraryOps for their contracts).  Default: the library's kernels on
    `device`.  The CPU tests of the multi-rank host logic pass their own restatement, so that they
    drive the same routing code the GPUs run.
    """

    def __init__(self, row_ptr_local, col_local, w_local, bounds, params, group=None, device=None, ops=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.params = params
        if params.app not in (APP_UNIFORM_WALK, APP_DEEPWALK, APP_PPR):
            raise ValueError("partitioned sampling supports the uniform walk, DeepWalk and PPR (a step of node2vec "
                             "needs the previous vertex's adjacency, which lives on another rank)")
        self.V = int(np.asarray(row_ptr_local).shape[0] - 1)
        self.bounds = np.asarray(bounds, np.int64)
        assert self.bounds.shape[0] == self.world + 1 and self.bounds[-1] == self.V
        if ops is None:
            dev_index = torch.cuda.current_device() if device is None else torch.device(device).index
            self.device = torch.device("cuda", dev_index)
            self.graph = api.Graph.from_csr(row_ptr_local, col_local, w_local, device=dev_index)
            self.ops = _LibraryOps(self.graph, params, self.device, self.world)
        else:
            self.device = torch.device(device or "cpu")
            self.graph = None
            self.ops = ops
        # collectives run on the tensors' own device unless the backend cannot (gloo with CUDA tensors)
        self._comm_cpu = dist.is_initialized() and dist.get_backend(group) == "gloo" and self.device.type == "cuda"
        self.bytes_sent = 0

    def _gather_counts(self, counts):
        """Every rank's count rows (k rows of P destinations) -> [P ranks, k, P] on the host: the
        one host synchronisation of a step."""
        P = self.world
        k = int(counts.numel()) // P
        if P == 1:
            return counts.cpu().view(1, k, 1)
        if self._comm_cpu:
            allc = torch.empty(P * k * P, dtype=torch.int64)
            dist.all_gather_into_tensor(allc, counts.cpu().reshape(-1), group=self.group)
        else:
            allc = torch.empty(P * k * P, dtype=torch.int64, device=self.device)
            dist.all_gather_into_tensor(allc, counts.reshape(-1), group=self.group)
        return allc.cpu().view(P, k, P)

    def _all_to_all(self, src, send, recv):
        if self.world == 1:
            return src
        if self._comm_cpu:
            dst = torch.empty(int(sum(recv)), dtype=torch.int64)
            dist.all_to_all_single(dst, src.cpu(), output_split_sizes=recv, input_split_sizes=send, group=self.group)
            dst = dst.to(self.device)
        else:
            dst = torch.empty(int(sum(recv)), dtype=torch.int64, device=self.device)
            dist.all_to_all_single(dst, src, output_split_sizes=recv, input_split_sizes=send, group=self.group)
        self.bytes_sent += 8 * (int(sum(send)) - send[self.rank])
        return dst

    def run(self, total_samples: int, initial=None):
        """Walks samples [0, total_samples); returns this rank's home shard [count, steps] (int32 on
        `device`, invalid = V) and the shard's first sample.  `initial`: the initial vertex of every
        sample (array of total_samples), default sample s starts at vertex s mod V.
        A walker is one 64-bit word, (global sample id << 32) | vertex; all ones = ended."""
        steps, P, r, ops = int(self.params.steps), self.world, self.rank, self.ops
        first, count = api.shard_range(total_samples, r, P)
        dev = self.device
        if not hasattr(self, "_counts"):
            self._counts = torch.zeros(P, dtype=torch.int64, device=dev)
            self._vbounds = torch.as_tensor(self.bounds, dtype=torch.int64, device=dev)
        sid = torch.arange(first, first + count, dtype=torch.int64, device=dev)
        if initial is None:
            cur = sid % self.V
        else:
            cur = torch.as_tensor(np.ascontiguousarray(initial[first:first + count], np.int32), device=dev).to(torch.int64)
        nxt = torch.where((cur >= 0) & (cur < self.V), (sid << 32) | cur, torch.full_like(sid, -1))
        records = []   # per step: this rank's (sample, new vertex) words, grouped by the owner of the vertex
        for step in range(-1, steps):
            # route the live walkers to the owners of their vertices (step -1: the initial vertices)
            if step >= 0:
                nxt = ops.step_packed(step, wk)
            ops.route_count(nxt, 0, self._vbounds, self._counts)
            mat = self._gather_counts(self._counts)[:, 0, :]            # [sender, destination]
            send, recv = mat[r].tolist(), mat[:, r].tolist()
            live = ops.route_scatter(nxt, 0, self._vbounds, self._counts, int(sum(send)))
            if step >= 0:
                records.append(live)
            if int(mat.sum()) == 0 or step + 1 == steps:
                break
            wk = self._all_to_all(live, send, recv)
        # every step's records go to the samples' home ranks: all counts first (one synchronisation),
        # then scatter / all-to-all / store per step without touching the host
        out = torch.full((count, steps), self.V, dtype=torch.int32, device=dev)
        if records:
            starts = [api.shard_range(total_samples, k, P)[0] for k in range(P)] + [(1 << 40)]
            hbounds = torch.as_tensor(starts, dtype=torch.int64, device=dev)
            hcounts = torch.zeros((len(records), P), dtype=torch.int64, device=dev)
            for k, rec in enumerate(records):
                ops.route_count(rec, 1, hbounds, hcounts[k])
            hmat = self._gather_counts(hcounts)                          # [sender, step, destination]
            for k, rec in enumerate(records):
                send, recv = hmat[r, k].tolist(), hmat[:, k, r].tolist()
                mine = self._all_to_all(ops.route_scatter(rec, 1, hbounds, hcounts[k], int(sum(send))), send, recv)
                ops.records_store(mine, k, first, count, steps, out)
        if hasattr(ops, "finish"):
            ops.finish()
        return out, first
