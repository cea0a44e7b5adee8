"""GPU test of the Python surface that mirrors the reference's per-app modules
(src/nextDoorPythonModule.cu:40-132): initSampling / sample / finalSamples / finalSampleLength /
finalSamplesArray / freeDeviceMemory, plus the zero-copy device tensor for GNN loaders."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


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
