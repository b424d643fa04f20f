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
def oracle():
    from oracle import build as obuild
    obuild.build()
    from oracle import oracle as o
    return o


def make_graph(n, m, seed=0, symmetric=False, max_degree=None):
    """Small seeded R-MAT CSC on the CPU as numpy int64 arrays."""
    from graph_sampling_b200.synthetic import rmat_csc
    indptr, indices = rmat_csc(n, m, seed=seed, symmetric=symmetric, max_degree=max_degree, device="cpu")
    return indptr.numpy().astype(np.int64), indices.numpy().astype(np.int64)


@pytest.fixture(scope="session")
def small_graph():
    return make_graph(2000, 40000, seed=11)


@pytest.fixture(scope="session")
def cfg1_graph():
    """Small GraphSAGE configuration: 100,000 nodes, 2,000,000 directed edges."""
    return make_graph(100_000, 2_000_000, seed=0x5EED + 1)


@pytest.fixture(scope="session")
def hub_graph():
    """A graph with isolated nodes, degree-1 nodes and hubs (degree in the thousands)."""
    rng = np.random.default_rng(5)
    n = 5000
    deg = np.zeros(n, dtype=np.int64)
    deg[:50] = rng.integers(2000, 4500, 50)       # hubs
    deg[50:1000] = rng.integers(0, 40, 950)
    deg[1000:1100] = 1
    deg[1100:1200] = 0
    deg[1200:] = rng.integers(0, 12, n - 1200)
    perm = rng.permutation(n)
    deg = deg[perm]
    indptr = np.zeros(n + 1, dtype=np.int64)
    indptr[1:] = np.cumsum(deg)
    cols = []
    for c in range(n):
        cols.append(np.sort(rng.choice(n, size=deg[c], replace=False)))
    indices = np.concatenate(cols).astype(np.int64)
    return indptr, indices
