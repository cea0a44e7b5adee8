"""The allocation-free map inversion (nd_invert_map_static) against the ordinary one.

The static variant exists for a sampler that lives in the same process as a training job:
cudaMalloc/cudaFree synchronise the device (stalling the training streams) and may fail outright
once the framework's allocator owns nearly all of HBM, so this entry point keeps its histograms in
a fixed array inside the library.  The array survives from call to call, which is what the second
round below is about: a stale counter left by the first call would corrupt the second.
Collected last on purpose (file name), runs both alone and after the rest of the suite.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _invert(nd, fn, keys, vals, invalid):
    import torch
    dk, dv = torch.from_numpy(keys).cuda(), torch.from_numpy(vals).cuda()
    ok, ov = torch.empty_like(dk), torch.empty_like(dv)
    live = C.c_int64(-1)
    nd.check(fn(0, keys.shape[0], dk.data_ptr(), dv.data_ptr(), invalid, ok.data_ptr(), ov.data_ptr(), C.byref(live)))
    n = live.value
    return ok.cpu().numpy()[:n], ov.cpu().numpy()[:n]


def test_static_inversion_matches_allocating_one_twice_in_a_row(nd):
    rng = np.random.default_rng(5)
    limit = int(nd.lib.nd_static_max_pairs())
    assert limit == 1 << 20
    # two different shapes back to back: the second must not see anything of the first
    for n, vmax in ((limit, 1 << 20), (300_001, 56944), (1, 2)):
        keys = rng.integers(0, vmax, n).astype(np.int32)
        keys[rng.random(n) < 0.25] = vmax // 2       # a hub
        keys[rng.random(n) < 0.1] = vmax             # dead pairs, dropped
        vals = rng.permutation(n).astype(np.int32)
        ek, ev = _invert(nd, nd.lib.nd_invert_map, keys, vals, vmax)
        for _ in range(2):
            gk, gv = _invert(nd, nd.lib.nd_invert_map_static, keys, vals, vmax)
            assert np.array_equal(gk, ek) and np.array_equal(gv, ev)   # integer work: bit-exact


def test_static_inversion_allocates_nothing_and_runs_on_a_caller_stream(nd):
    """What the entry point is for: the device's free memory is the same before and after a call
    (once the array's address has been looked up by a first call), and the stream variant gives the
    same result while working only on the caller's stream."""
    import torch
    rng = np.random.default_rng(7)
    n, vmax = 200_000, 1 << 18
    keys = rng.integers(0, vmax + 1, n).astype(np.int32)
    vals = rng.permutation(n).astype(np.int32)
    ek, ev = _invert(nd, nd.lib.nd_invert_map, keys, vals, vmax)
    _invert(nd, nd.lib.nd_invert_map_static, keys, vals, vmax)            # first call on the device: address look-up
    st = torch.cuda.Stream()
    dk, dv = torch.from_numpy(keys).cuda(), torch.from_numpy(vals).cuda()
    ok, ov = torch.empty_like(dk), torch.empty_like(dv)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    live = C.c_int64(-1)
    nd.check(nd.lib.nd_invert_map_static_on(0, st.cuda_stream, n, dk.data_ptr(), dv.data_ptr(), vmax, ok.data_ptr(), ov.data_ptr(),
                                            C.byref(live)))
    free_mid = torch.cuda.mem_get_info()[0]
    dk.copy_(torch.from_numpy(keys)); dv.copy_(torch.from_numpy(vals))
    torch.cuda.synchronize()
    live2 = C.c_int64(-1)
    nd.check(nd.lib.nd_invert_map_static(0, n, dk.data_ptr(), dv.data_ptr(), vmax, ok.data_ptr(), ov.data_ptr(), C.byref(live2)))
    free_after = torch.cuda.mem_get_info()[0]
    assert free_before == free_mid == free_after, "the allocation-free entry point changed the device's free memory"
    assert live.value == live2.value == ek.shape[0]
    assert np.array_equal(ok.cpu().numpy()[:live.value], ek) and np.array_equal(ov.cpu().numpy()[:live.value], ev)


def test_static_inversion_rejects_oversize(nd):
    live = C.c_int64(0)
    rc = nd.lib.nd_invert_map_static(0, int(nd.lib.nd_static_max_pairs()) + 1, 1, 1, 10, 1, 1, C.byref(live))
    assert rc == 4
    assert b"exceed the fixed scratch" in nd.lib.nd_last_error()
    nd.check(nd.lib.nd_invert_map_static(0, 0, None, None, 10, None, None, C.byref(live)))
    assert live.value == 0
