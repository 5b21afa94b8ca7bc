import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "fastgl-ae_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def make_graph(n_nodes, avg_degree, seed=12345, hub=None):
    """Small seeded power-law CSR (numpy): int64 indptr, int32 indices.  ``hub`` adds a node adjacent to
    that many distinct others so that deg > fanout paths are exercised."""
    rng = np.random.default_rng(seed)
    m = int(n_nodes * avg_degree / 2)
    w = 1.0 / np.arange(1, n_nodes + 1) ** 0.8
    w /= w.sum()
    src = rng.choice(n_nodes, size=m, p=w)
    dst = rng.integers(0, n_nodes, size=m)
    keep = src != dst
    src, dst = src[keep], dst[keep]
    if hub:
        others = rng.choice(np.arange(1, n_nodes), size=min(hub, n_nodes - 1), replace=False)
        src = np.concatenate([src, others])
        dst = np.concatenate([dst, np.zeros_like(others)])
    s2 = np.concatenate([src, dst])
    d2 = np.concatenate([dst, src])
    order = np.argsort(d2, kind="stable")
    indices = s2[order].astype(np.int32)
    indptr = np.zeros(n_nodes + 1, dtype=np.int64)
    np.cumsum(np.bincount(d2, minlength=n_nodes), out=indptr[1:])
    return indptr, indices


@pytest.fixture(scope="session")
def small_graph():
    return make_graph(2000, 12, seed=7, hub=300)
