import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def ndo():
    from oracle import ndo as m
    m.build()
    m.lib()
    return m


@pytest.fixture(scope="session")
def small_graph(ndo):
    """R-MAT, 2000 vertices, 12000 undirected edges: isolated vertices, hubs and duplicate edges."""
    return ndo.rmat_graph(2000, 12000, seed=1)


@pytest.fixture(scope="session")
def tiny_graph(ndo):
    """Hand-checkable graph: a path 0-1-2, a triangle 3-4-5, a duplicate edge 6=7, isolated 8, 9."""
    src = np.array([0, 1, 1, 2, 3, 4, 3, 5, 4, 5, 6, 7, 6, 7], np.int32)
    dst = np.array([1, 0, 2, 1, 4, 3, 5, 3, 5, 4, 7, 6, 7, 6], np.int32)
    w = np.array([1, 1, 2, 2, 1.5, 1.5, 3, 3, 4.5, 4.5, 2, 2, 1, 1], np.float32)
    return ndo.csr_from_records(src, dst, w, V=10)


@pytest.fixture(scope="session")
def nd():
    """The product library; GPU tests only."""
    from nextdoor_b200 import api
    return api
