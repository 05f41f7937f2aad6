import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle_py
    oracle_py.build()
    return oracle_py


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "e8_golden.npz"))


def small_params(**kw):
    from octex_b200 import build_index
    base = dict(copies=8, blocks=2, pca_dims=32, list_len=16, min_cell=1, log_buckets=12,
                sketch_width=32, table_len=16)
    base.update(kw)
    return build_index.IndexParams(**base)


@pytest.fixture(scope="session")
def small_index():
    """20 000 x 48 clustered rows, 8 copies of 2 blocks (the shape of the reference's own
    equivalence test, cpp/tests/test_search.cu:509-597): (arrays, meta, base, queries)."""
    from octex_b200 import build_index, synth
    base = synth.plumbing(20000, 48, seed=0)
    queries = synth.plumbing(300, 48, seed=1)
    arrays, meta = build_index.build_arrays(base, small_params(), device="cpu")
    return arrays, meta, base, queries


@pytest.fixture(scope="session")
def wide_index():
    """6 000 x 128 rows, 6 copies of 4 blocks, sketch 64, five spacings with a min_cell filter."""
    from octex_b200 import build_index, synth
    base = synth.descriptor_like(6000, 128, seed=0)
    queries = synth.descriptor_like(200, 128, seed=1)
    arrays, meta = build_index.build_arrays(
        base, small_params(copies=6, blocks=4, pca_dims=64, list_len=32, min_cell=4,
                           sketch_width=64, table_len=32), device="cpu")
    return arrays, meta, base, queries


def recall(ids, truth):
    k = truth.shape[1]
    return float(np.mean([len(set(ids[i, :k]) & set(truth[i])) / k for i in range(len(truth))]))
