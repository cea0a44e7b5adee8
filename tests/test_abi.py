"""CPU tests of the boundary: the shared library loads, exports every symbol the public header
declares, computes the host-only helpers, and refuses to compute without a CUDA device."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from nextdoor_b200 import build
    build.build()
    from nextdoor_b200 import _lib
    return _lib


def test_header_symbols_are_exported(lib):
    hdr = open(os.path.join(ROOT, "include", "nextdoor_b200.h")).read()
    declared = set(re.findall(r"^(?:int|int64_t|const char \*)\s*(nd_[a-z0-9_]+)\(", hdr, flags=re.M))
    assert len(declared) >= 25
    raw = C.CDLL(lib.LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), f"{name} declared in the header but not exported"
    assert declared <= set(lib.EXPORTED), declared - set(lib.EXPORTED)


def test_host_only_helpers(lib):
    from nextdoor_b200 import api
    assert api.final_sample_size(api.app_params(api.APP_KHOP)) == 275
    assert api.final_sample_size(api.app_params(api.APP_DEEPWALK)) == 100
    assert api.final_sample_size(api.app_params(api.APP_FASTGCN_REF)) == 5 * 64
    assert api.initial_sample_size(api.app_params(api.APP_LADIES_IS, batch=32)) == 32
    # PartStartPointer / PartDivisionSize: the last part takes the remainder (utils.hpp:26-27)
    assert api.shard_range(10, 0, 3) == (0, 3)
    assert api.shard_range(10, 2, 3) == (6, 4)
    total = sum(api.shard_range(56944, i, 8)[1] for i in range(8))
    assert total == 56944


@pytest.mark.parametrize("threads", ["1", "3", "16"])
def test_host_fill_and_row_helpers(lib, monkeypatch, threads):
    """The host-side helpers of the row-prefix result path run without a device: the threaded fill
    (thread counts that do not divide the length, lengths below the thread count) and the scratch
    size of nd_rows_unpack; the update calls refuse a null sampler."""
    from nextdoor_b200 import api
    monkeypatch.setenv("ND_HOST_THREADS", threads)
    for n in (0, 1, 2, 7, 1000, 100003):
        a = np.full(n + 2, -5, np.int32)
        api.host_fill(a[1:n + 1], 42)
        assert (a[1:n + 1] == 42).all() and a[0] == -5 and a[n + 1] == -5
    assert lib.lib.nd_host_fill_int32(None, 4, 1) == 1
    assert api.rows_scratch_words(0) == 1 and api.rows_scratch_words(1) == 2
    assert api.rows_scratch_words(4096) == 2 and api.rows_scratch_words(4097) == 3
    assert lib.lib.nd_sampler_host_update_begin(None, None, None, None) == 1
    assert lib.lib.nd_sampler_pack_rows(None, None, None) == 1


def test_struct_layout_matches_oracle(lib, ndo):
    a, b = lib.AppParams, ndo.Params
    assert C.sizeof(a) == C.sizeof(b)
    assert [f[0] for f in a._fields_] == [f[0] for f in b._fields_]


def test_no_device_fails_loudly(lib):
    if lib.lib.nd_device_count() > 0:
        pytest.skip("a CUDA device is present")
    from nextdoor_b200 import api
    with pytest.raises(api.NdError) as e:
        api.Graph.from_csr(np.array([0, 1, 2], np.int32), np.array([1, 0], np.int32), np.ones(2, np.float32))
    assert e.value.code == 2 and "CUDA" in str(e.value)


def test_bad_arguments_are_rejected(lib):
    from nextdoor_b200 import api
    f, c = C.c_int64(), C.c_int64()
    assert lib.lib.nd_shard_range(10, 3, 3, C.byref(f), C.byref(c)) == 1
    assert b"bad argument" in lib.lib.nd_last_error()
    assert lib.lib.nd_sampler_sample(None, 0) == 1


def test_header_is_plain_c_and_cxx():
    """The boundary is a C ABI: the header must compile as C11 and as C++17 without any CUDA or
    torch include."""
    import shutil
    import subprocess
    hdr = os.path.join(ROOT, "include", "nextdoor_b200.h")
    for cc, lang, std in (("gcc", "c", "-std=c11"), ("g++", "c++", "-std=c++17")):
        exe = shutil.which(cc) or os.path.join("/usr/bin", cc)
        r = subprocess.run([exe, std, "-fsyntax-only", "-Wall", "-x", lang, hdr], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
