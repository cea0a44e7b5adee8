"""GPU test of the Python surface that mirrors the reference's per-app modules
(src/nextDoorPythonModule.cu:40-132): initSampling / sample / finalSamples / finalSampleLength /
finalSamplesArray / freeDeviceMemory, plus the zero-copy device tensor for GNN loaders."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
APPS = os.path.join(os.path.dirname(os.path.abspath(__file__)), "apps")


@pytest.mark.parametrize("app,kw", [(0, {}), (3, {"p": 2.0, "q": 0.5})])
def test_module_functions(nd, ndo, tmp_path, app, kw):
    import torch
    src, dst, w = ndo.rmat_records(900, 6000, seed=3)
    path = str(tmp_path / "graph.bin")
    ndo.write_edge_list_binary(path, src, dst, w)
    hg = ndo.csr_from_records(src, dst, w)
    pr = nd.app_params(app, steps=30, seed=5, **kw)
    mod = nd.SamplingModule(pr)
    mod.initSampling(path)
    mod.sample()
    S = hg.V if app == 0 else 100 * hg.V            # the reference's numSamples for the two apps
    exp = ndo.sample(hg, ndo.make_params(app, steps=30, seed=5, **kw), S)["out"]
    arr = mod.finalSamplesArray()
    assert arr.dtype == np.int32 and arr.shape == (S * 30,)
    assert np.array_equal(arr.reshape(S, 30), exp)
    lst = mod.finalSamples()
    assert isinstance(lst, list) and len(lst) == S * 30 == mod.finalSampleLength() and lst[:60] == exp.reshape(-1)[:60].tolist()
    t = mod.finalSamplesTensor()
    assert t.is_cuda and t.dtype == torch.int32 and tuple(t.shape) == (S, 30)
    assert np.array_equal(t.cpu().numpy(), exp)
    again = torch.utils.dlpack.from_dlpack(torch.utils.dlpack.to_dlpack(t))
    assert again.data_ptr() == t.data_ptr()          # still the library's buffer, no copy
    mod.sample()                                       # a second run gives the same samples (keyed draws)
    assert np.array_equal(mod.finalSamplesArray().reshape(S, 30), exp)
    mod.freeDeviceMemory()


def _import_module(name, folder):
    import importlib.util
    path = os.path.join(folder, name + ".so")
    if not os.path.exists(path):
        return None
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("name,steps", [("NdOwnWalkPy3", 12), ("UniformRandomWalkPy3", 100)])
def test_compiled_cpython_module(ndo, tmp_path, name, steps):
    """The real extension modules: an application file that ends with
    #include "nextDoorPythonModule.cu", compiled with -DPYTHON_3 the way the reference's
    example/Makefile:9-11 does (this project's own app, and -- where the reference tree was present
    at build time -- the reference's example/uniformRandWalk.cu unchanged), imported and driven as
    README.md:73-95 shows: initSampling, sample, finalSamples, finalSampleLength, freeDeviceMemory
    and the C symbol finalSamplesArray read through ctypes (src/nextDoorPythonModule.cu:40-132)."""
    import ctypes as C
    folder = os.path.join(APPS, "_ref") if name == "UniformRandomWalkPy3" else APPS
    mod = _import_module(name, folder)
    if mod is None:
        pytest.skip("built without the reference tree")
    src, dst, w = ndo.rmat_records(700, 5000, seed=4)
    path = str(tmp_path / "graph.bin")
    ndo.write_edge_list_binary(path, src, dst, w)
    hg = ndo.csr_from_records(src, dst, w)
    S = hg.V                                           # numSamples of both apps: one walk per vertex
    exp = ndo.sample(hg, ndo.make_params(ndo.APP_UNIFORM_WALK, steps=steps, seed=0), S)["out"]
    mod.initSampling(path)
    mod.sample()
    lst = mod.finalSamples()
    assert isinstance(lst, list) and len(lst) == S * steps == mod.finalSampleLength()
    assert np.array_equal(np.array(lst, np.int32).reshape(S, steps), exp)
    fn = C.CDLL(mod.__file__).finalSamplesArray
    fn.restype = C.POINTER(C.c_int)
    arr = np.ctypeslib.as_array(fn(), shape=(S * steps,))
    assert np.array_equal(arr.reshape(S, steps), exp)
    mod.sample()                                       # keyed draws: a second run gives the same samples
    assert np.array_equal(np.ctypeslib.as_array(fn(), shape=(S * steps,)).reshape(S, steps), exp)
    mod.freeDeviceMemory()
