"""Host-side mirror of the reference's interface for the sampling path, over the C ABI.

* `Graph` / `Sampler` follow the C++ surface of src/libNextDoor.hpp (loadGraph, transferCSRToGPUs,
  allocNextDoorDataOnGPU, doTransitParallelSampling / doSampleParallelSampling, getFinalSamples,
  freeDeviceData), one object per device.
* `SamplingModule` has the five functions of the reference's per-app Python extension modules
  (src/nextDoorPythonModule.cu:40-102): initSampling, sample, finalSamples, finalSampleLength,
  freeDeviceMemory -- plus finalSamplesArray, which the reference exports as a C symbol for ctypes
  (:89-93) and which returns a numpy view here.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import (APP_DEEPWALK, APP_FASTGCN_IS, APP_FASTGCN_REF, APP_KHOP, APP_KHOP_DISTINCT,  # noqa: F401
                   APP_LADIES_IS, APP_LADIES_REF, APP_NODE2VEC, APP_PPR, APP_UNIFORM_WALK,
                   MODE_SAMPLE_PARALLEL, MODE_TRANSIT_PARALLEL, MODE_TRANSIT_PARALLEL_LB, AppParams,
                   NdError, check, lib)

KERNEL_TYPES = {"TransitParallel": MODE_TRANSIT_PARALLEL, "SampleParallel": MODE_SAMPLE_PARALLEL}


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def app_params(app, steps=None, fanout=None, batch=64, p=2.0, q=0.5, stop_prob=0.01, seed=0,
               n2v_ref_compat=1) -> AppParams:
    """Defaults are the reference's compile-time constants: 100-step walks (randomWalks.cu:4),
    fan-out 25 then 10 (khop.cu:3-8), 5 layers x 64 with batches of 64 (fastgcnSampling.cu:1-4),
    p=2, q=0.5 (randomWalks.cu:149-150), walkEndProb 0.01 (randomWalks.cu:105)."""
    pr = AppParams()
    pr.app = app
    if app <= APP_NODE2VEC:
        pr.steps = 100 if steps is None else steps
        pr.fanout[0] = 1
    elif app in (APP_KHOP, APP_KHOP_DISTINCT):
        fan = list(fanout) if fanout is not None else [25, 10]
        pr.steps = len(fan) if steps is None else steps
        for i, f in enumerate(fan[:_lib.MAX_FANOUT]):
            pr.fanout[i] = f
    else:
        pr.steps = 5 if steps is None else steps
        pr.fanout[0] = 64 if fanout is None else (fanout if isinstance(fanout, int) else fanout[0])
    pr.batch = batch
    pr.p, pr.q, pr.stop_prob = p, q, stop_prob
    pr.seed = seed
    pr.n2v_ref_compat = n2v_ref_compat
    return pr


def final_sample_size(params: AppParams) -> int:
    return int(lib.nd_final_sample_size(C.byref(params)))


def initial_sample_size(params: AppParams) -> int:
    return int(lib.nd_initial_sample_size(C.byref(params)))


def launch_count() -> int:
    """Kernels this process has launched through the library so far."""
    return int(lib.nd_launch_count())


def shard_range(total: int, idx: int, parts: int):
    """PartStartPointer / PartDivisionSize of the reference (src/utils.hpp:26-27)."""
    f, c = C.c_int64(0), C.c_int64(0)
    check(lib.nd_shard_range(total, idx, parts, C.byref(f), C.byref(c)))
    return f.value, c.value


class Graph:
    """A CSR replica in one GPU's HBM."""

    def __init__(self, handle, device):
        self._h = handle
        self.device = device
        V, E, md, dev = C.c_int32(0), C.c_int64(0), C.c_int32(0), C.c_int(0)
        check(lib.nd_graph_info(self._h, C.byref(V), C.byref(E), C.byref(md), C.byref(dev)))
        self.V, self.E, self.max_degree = V.value, E.value, md.value

    @classmethod
    def from_csr(cls, row_ptr, col, w, max_w=None, device=0):
        row_ptr = np.ascontiguousarray(row_ptr, np.int32)
        col = np.ascontiguousarray(col, np.int32)
        w = np.ascontiguousarray(w, np.float32)
        if max_w is not None:
            max_w = np.ascontiguousarray(max_w, np.float32)
        h = C.c_void_p()
        check(lib.nd_graph_from_csr(device, row_ptr.shape[0] - 1, col.shape[0], _ptr(row_ptr), _ptr(col),
                                    _ptr(w), _ptr(max_w), C.byref(h)))
        return cls(h, device)

    @classmethod
    def from_edge_records(cls, src, dst, w, device=0):
        rec = np.empty(len(src), dtype=[("s", "<i4"), ("d", "<i4"), ("w", "<f4")])
        rec["s"], rec["d"], rec["w"] = src, dst, w
        h = C.c_void_p()
        check(lib.nd_graph_from_edge_records(device, rec.shape[0], _ptr(rec), C.byref(h)))
        return cls(h, device)

    @classmethod
    def load(cls, path, graph_type="edge-list", graph_format="binary", device=0):
        """loadGraph(file, type, format) of the reference (src/nextdoor.cu:1845-1891): binary edge
        list (12-byte records), text edge list, text adjacency list."""
        h = C.c_void_p()
        check(lib.nd_graph_load(device, str(path).encode(), graph_type.encode(), graph_format.encode(), C.byref(h)))
        return cls(h, device)

    @classmethod
    def rmat(cls, V, M, seed=0, device=0):
        h = C.c_void_p()
        check(lib.nd_graph_rmat(device, V, M, seed, C.byref(h)))
        return cls(h, device)

    def to_host(self):
        row_ptr = np.empty(self.V + 1, np.int32)
        col = np.empty(self.E, np.int32)
        w = np.empty(self.E, np.float32)
        mw = np.empty(self.V, np.float32)
        check(lib.nd_graph_to_host(self._h, _ptr(row_ptr), _ptr(col), _ptr(w), _ptr(mw)))
        return row_ptr, col, w, mw

    def row_ptr_device_ptr(self) -> int:
        """Address of the replica's row-offset array [V + 1] int32 in device memory (read-only for callers)."""
        rp = C.c_void_p()
        check(lib.nd_graph_device_ptrs(self._h, C.byref(rp), None, None, None))
        return int(rp.value)

    def partition(self, budget_bytes, max_parts=4096):
        fv = np.zeros(max_parts, np.int32)
        lv = np.zeros(max_parts, np.int32)
        fe = np.zeros(max_parts, np.int64)
        le = np.zeros(max_parts, np.int64)
        n = C.c_int32(0)
        check(lib.nd_graph_partition(self._h, budget_bytes, max_parts, _ptr(fv), _ptr(lv), _ptr(fe), _ptr(le), C.byref(n)))
        k = n.value
        return fv[:k], lv[:k], fe[:k], le[:k]

    def free(self):
        if self._h:
            lib.nd_graph_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Sampler:
    """NextDoorData of one device: the shard [first_sample, first_sample + num_samples) of the job."""

    def __init__(self, graph: Graph, params: AppParams, num_samples=None, first_sample=0, initial=None):
        self.graph = graph
        self.params = params
        self.fs = final_sample_size(params)
        self.isz = initial_sample_size(params)
        if num_samples is None:
            num_samples = graph.V
        self.S = int(num_samples)
        self.first = int(first_sample)
        if initial is not None:
            initial = np.ascontiguousarray(initial, np.int32)
            assert initial.size == self.S * self.isz, "initialSampleSize mismatch"
        h = C.c_void_p()
        check(lib.nd_sampler_create(graph._h, C.byref(params), self.S, self.first, _ptr(initial), C.byref(h)))
        self._h = h

    def set_initial(self, initial):
        initial = np.ascontiguousarray(initial, np.int32)
        assert initial.size == self.S * self.isz
        check(lib.nd_sampler_set_initial(self._h, _ptr(initial)))

    def set_stream(self, stream_ptr):
        check(lib.nd_sampler_set_stream(self._h, C.c_void_p(stream_ptr)))

    def sample(self, mode=MODE_TRANSIT_PARALLEL_LB, sync=True):
        check(lib.nd_sampler_sample(self._h, mode))
        if sync:
            check(lib.nd_sampler_sync(self._h))

    def sync(self):
        check(lib.nd_sampler_sync(self._h))

    def final_samples(self, out=None):
        if out is None:
            out = np.empty(self.S * self.fs, np.int32)
        check(lib.nd_sampler_final_samples(self._h, _ptr(out)))
        return out.reshape(self.S, self.fs)

    def final_samples_async(self, out, copy_stream=None):
        """Enqueue the device-to-host copy (on `copy_stream`, a raw cudaStream_t, ordered after the
        sampling issued so far; or on the sampler's own stream).  Synchronise that stream before
        reading `out`."""
        check(lib.nd_sampler_final_samples_async(self._h, _ptr(out), C.c_void_p(copy_stream) if copy_stream else None))

    def host_update_begin(self, out, row_len, copy_stream=None):
        """Walk apps: start bringing the dense host array `out` (with its per-row lengths `row_len`,
        see new_host_result) up to date while copying only the rows' valid prefixes."""
        check(lib.nd_sampler_host_update_begin(self._h, _ptr(out), _ptr(row_len), C.c_void_p(copy_stream) if copy_stream else None))

    def host_update_fetch(self):
        check(lib.nd_sampler_host_update_fetch(self._h))

    def host_update_finish(self) -> int:
        """Blocks until `out` holds this job's result; returns the vertex slots that crossed PCIe."""
        n = C.c_int64(0)
        check(lib.nd_sampler_host_update_finish(self._h, C.byref(n)))
        return int(n.value)

    def pack_rows(self):
        """Walk apps: enqueue the packing of the rows' valid prefixes; returns the device addresses
        (row lengths [S] int32, packed vertices int32), valid until this sampler's next sample()."""
        a, b = C.c_void_p(), C.c_void_p()
        check(lib.nd_sampler_pack_rows(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def pack_rows_total(self) -> int:
        """Waits for pack_rows(); the number of packed vertices."""
        n = C.c_int64(0)
        check(lib.nd_sampler_pack_rows_total(self._h, C.byref(n)))
        return int(n.value)

    def final_samples_device_ptr(self):
        p = C.c_void_p()
        check(lib.nd_sampler_final_samples_device(self._h, C.byref(p)))
        return p.value

    def aux(self):
        L, B = self.params.fanout[0], self.params.batch
        collective = self.params.app >= APP_FASTGCN_REF
        adj_row = adj_col = prob = hop = None
        if collective:
            n = self.S * self.params.steps * max(L, B) * L
            adj_row = np.empty(n, np.int32)
            adj_col = np.empty(n, np.int32)
            prob = np.zeros(self.S * self.fs, np.float32)
        if self.params.app == APP_KHOP_DISTINCT:
            hop = np.zeros(self.S * self.params.steps, np.int32)
        check(lib.nd_sampler_aux(self._h, _ptr(adj_row), _ptr(adj_col), _ptr(prob), _ptr(hop)))
        return dict(adj_row=adj_row, adj_col=adj_col, prob=prob, hop_counts=hop)

    def stats(self):
        st = np.zeros(8, np.int64)
        check(lib.nd_sampler_stats(self._h, _ptr(st), 8))
        return dict(sampled_edges=int(st[0]), live_pairs=int(st[1]), weight_tries=int(st[2]),
                    n2v_tries=int(st[3]), n2v_probes=int(st[4]), union_ids=int(st[5]), union_unique=int(st[6]),
                    pairs_not_entered=int(st[7]))

    def live_pairs(self):
        """Walks, transit-parallel modes: pairs in the map of each step of the last sample() (PPR in
        the load-balanced mode leaves out pairs whose walk is known to stop at that step)."""
        live = np.zeros(self.params.steps, np.int32)
        check(lib.nd_sampler_live_pairs(self._h, _ptr(live), live.shape[0]))
        return live

    def set_profiling(self, on=True):
        check(lib.nd_sampler_set_profiling(self._h, int(on)))

    def phase_ms(self):
        ms = np.zeros(len(_lib.PHASES), np.float32)
        ln = np.zeros(len(_lib.PHASES), np.int32)
        check(lib.nd_sampler_phase_ms(self._h, _ptr(ms), _ptr(ln), len(_lib.PHASES)))
        return {p: (float(ms[i]), int(ln[i])) for i, p in enumerate(_lib.PHASES)}

    def free(self):
        if self._h:
            lib.nd_sampler_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def rows_scratch_words(n_rows: int) -> int:
    return int(lib.nd_rows_scratch_words(n_rows))


def rows_unpack(device, stream, n_rows, steps, invalid, len_ptr, vals_ptr, out_ptr, row_len_ptr, scratch_ptr):
    """nd_rows_unpack on raw device addresses (ints); `stream` a raw cudaStream_t or None."""
    check(lib.nd_rows_unpack(device, C.c_void_p(stream) if stream else None, n_rows, steps, invalid, C.c_void_p(len_ptr),
                             C.c_void_p(vals_ptr), C.c_void_p(out_ptr), C.c_void_p(row_len_ptr), C.c_void_p(scratch_ptr)))


def host_fill(arr, value):
    """arr[:] = value with the library's host threads (the first fill of a large result array)."""
    flat = arr.reshape(-1)
    check(lib.nd_host_fill_int32(_ptr(flat), flat.shape[0], int(value)))


class PipelinedSampler:
    """The job cut into `chunks` seed ranges that are sampled one after the other on one stream
    while the result of each finished chunk is copied to the host on a second stream, so the
    device-to-host copy overlaps the sampling of the following chunks.  Output is identical to one
    Sampler over the whole range: the draws are keyed by the global sample index.
    `stream` / `copy_stream` are raw cudaStream_t values (a non-default `stream` lets every chunk
    replay its CUDA graph)."""

    def __init__(self, graph: Graph, params: AppParams, num_samples, first_sample=0, initial=None, chunks=4,
                 stream=None, copy_stream=None, depth=1, sparse_rows=False):
        """depth > 1 keeps that many independent sets of samplers (own result buffers) and rotates
        through them job by job, so with run_async() a whole job's copy overlaps the next job's
        sampling even with chunks=1 (no small-launch penalty from cutting the job).
        sparse_rows=True (walk apps; otherwise ignored): a host array handed to run()/run_async() is
        filled with the invalid id once and remembered by its address; later jobs into the same array
        copy only the rows' valid prefixes and rewrite only the slots that changed since the array's
        previous job.  The array ends up exactly as with the dense copy, provided the caller does not
        write to it in between (forget(out) drops the memory of an array).  The default copies the
        dense array every time."""
        self.S, self.fs, self.isz = int(num_samples), final_sample_size(params), initial_sample_size(params)
        self.device, self.copy_stream = graph.device, copy_stream
        self.sets, self._job = [], 0
        # Walk jobs move only the rows' valid prefixes to the host (nd_sampler_host_update_*): the
        # per-row lengths of every host array this object has filled, by the array's address, and
        # the jobs whose rows are still to be written (at most one per sampler set).
        self.sparse_rows = sparse_rows and params.app <= APP_NODE2VEC
        self.invalid = graph.V
        self._row_len, self._pending = {}, {}
        self.values_copied = 0          # vertex slots the last finished job moved over PCIe
        for _ in range(max(1, depth)):
            parts = []
            for c in range(chunks):
                f, n = shard_range(self.S, c, chunks)
                init = None if initial is None else np.ascontiguousarray(initial[f * self.isz:(f + n) * self.isz], np.int32)
                smp = Sampler(graph, params, num_samples=n, first_sample=first_sample + f, initial=init)
                if stream is not None:
                    smp.set_stream(stream)
                parts.append((f, n, smp))
            self.sets.append(parts)
        self.parts = self.sets[0]

    def run(self, initial_host, out_host, mode=MODE_TRANSIT_PARALLEL_LB):
        """initial_host / out_host: (pinned) numpy int32 arrays of the whole job; returns after everything landed."""
        self.run_async(initial_host, out_host, mode)
        self.wait()

    def run_async(self, initial_host, out_host, mode=MODE_TRANSIT_PARALLEL_LB):
        """Enqueue one job and return.  Jobs enqueued back to back overlap: a chunk of the next
        job is sampled while the last chunk of this one is still on its way to the host (the
        library orders a chunk's next sampling after its own pending copy).  Give consecutive
        jobs different `out_host` buffers and call wait() before reading them."""
        k = self._job % len(self.sets)
        self.parts = self.sets[k]
        self._job += 1
        if not self.sparse_rows:
            for f, n, smp in self.parts:
                if initial_host is not None:
                    smp.set_initial(initial_host[f * self.isz:(f + n) * self.isz])
                smp.sample(mode, sync=False)
                smp.final_samples_async(out_host[f * self.fs:(f + n) * self.fs], self.copy_stream)
            return
        self._finish(k)                                   # this set's previous job still owns its staging buffers
        others = [j for j in self._pending if j != k]
        for j in others:                                  # the lengths of the job before have landed: its vertices
            for _, _, smp in self.sets[j]:                # cross while this job is sampled
                smp.host_update_fetch()
        row_len = self._rows_of(out_host)
        for f, n, smp in self.parts:
            if initial_host is not None:
                smp.set_initial(initial_host[f * self.isz:(f + n) * self.isz])
            smp.sample(mode, sync=False)
            smp.host_update_begin(out_host[f * self.fs:(f + n) * self.fs], row_len[f:f + n], self.copy_stream)
        self._pending[k] = True
        for j in others:                                  # ... and its rows are written while the device works on this one
            self._finish(j)

    def _rows_of(self, out_host):
        key = (out_host.__array_interface__["data"][0], out_host.size)
        if key not in self._row_len:
            host_fill(out_host, self.invalid)
            self._row_len[key] = np.zeros(self.S, np.int32)
        return self._row_len[key]

    def forget(self, out_host):
        """The caller is going to write to `out_host` itself: the next job into it starts from a fresh fill."""
        self._row_len.pop((out_host.__array_interface__["data"][0], out_host.size), None)

    def _finish(self, k):
        if self._pending.pop(k, None):
            self.values_copied = sum(smp.host_update_finish() for _, _, smp in self.sets[k])

    def wait(self):
        for k in list(self._pending):
            self._finish(k)
        for parts in self.sets:
            for _, _, smp in parts:
                smp.sync()
        if self.copy_stream:
            check(lib.nd_stream_sync(self.device, C.c_void_p(self.copy_stream)))

    def stats(self):
        tot = {}
        for _, _, smp in self.parts:
            for k, v in smp.stats().items():
                tot[k] = tot.get(k, 0) + v
        return tot

    def free(self):
        for parts in self.sets:
            for _, _, smp in parts:
                smp.free()


class SamplingModule:
    """Stand-in for one of the reference's per-app Python modules (e.g. UniformRandomWalkPy3)."""

    def __init__(self, params: AppParams, device=0, mode=MODE_SAMPLE_PARALLEL):
        self._params = params
        self._device = device
        self._mode = mode  # the reference's sample() runs the sample-parallel path (:54-58)
        self._graph = None
        self._sampler = None
        self._final = None

    def initSampling(self, graph_path):
        self._graph = Graph.load(graph_path, device=self._device)
        n = self._graph.V
        if self._params.app <= APP_NODE2VEC and n < 256 * 1024:
            n = 100 * n  # RandomWalkApp::numSamples, randomWalks.cu:23-26
        if self._params.app == APP_UNIFORM_WALK:
            n = self._graph.V  # example/uniformRandWalk.cu:55-58
        if self._params.app >= APP_FASTGCN_REF:
            n = 10000  # NUM_SAMPLES, fastgcnSampling.cu:4
        self._sampler = Sampler(self._graph, self._params, num_samples=n)

    def sample(self):
        self._final = None
        self._sampler.sample(self._mode)

    def finalSamplesArray(self):
        if self._final is None:
            self._final = self._sampler.final_samples().reshape(-1)
        return self._final

    def finalSamples(self):
        return self.finalSamplesArray().tolist()

    def finalSamplesTensor(self):
        """The final samples as a CUDA tensor [numSamples, finalSampleSize] that aliases the
        library's device buffer: no device-to-host copy and no Python list (the reference builds the
        list element by element, src/nextDoorPythonModule.cu:60-72).  Valid until the next sample()
        or freeDeviceMemory(); hand it to a loader as is or through DLPack (torch.utils.dlpack).
        Treat it as read-only: the library keeps this array between calls and rewrites only what changes."""
        from . import dist as _dist
        return _dist.device_samples(self._sampler)

    def finalSampleLength(self):
        return int(self.finalSamplesArray().size)

    def freeDeviceMemory(self):
        if self._sampler:
            self._sampler.free()
        if self._graph:
            self._graph.free()
        self._sampler = self._graph = None
