"""The adapters are drop-in replacements: the calls of cuvs.neighbors.cagra and of a Faiss GPU
index run on this package and give the results of its native interface (modelled on the
reference's tests/test_dropin.py; seeded synthetic data instead of its SIFT1M index)."""
import numpy as np
import pytest

import octex_b200
from octex_b200 import cuvs as cagra
from octex_b200 import faiss, index_dir, synth
from conftest import recall

pytestmark = pytest.mark.gpu
K = 10
BUILD = dict(copies=8, blocks=2, pca_dims=32, list_len=16, min_cell=1, log_buckets=12,
             sketch_width=32, table_len=16)
SEARCH = dict(read=16, starts=32, waves=2)


def data(seed=0, n=20000, m=200, d=48):
    base = synth.plumbing(n, d, seed=seed)
    queries = synth.plumbing(m, d, seed=seed + 100)
    d2 = ((queries ** 2).sum(1)[:, None] - 2.0 * queries @ base.T + (base ** 2).sum(1)[None, :])
    truth = np.argsort(d2, axis=1)[:, :K]
    return base, queries, truth


@pytest.fixture(scope="module")
def native_dir(small_index, tmp_path_factory):
    arrays, meta, _, queries = small_index
    path = str(tmp_path_factory.mktemp("dropin") / "idx")
    index_dir.write_index(path, arrays, meta)
    return path, queries


def test_cuvs_search_matches_native(native_dir):
    import torch
    path, queries = native_dir
    native = octex_b200.load(path, placement="replicate")
    D_ref, I_ref = native.search(queries, K, **SEARCH)
    index = cagra.Index(native)
    assert index.trained and index.dim == 48 and len(index) == native.size
    sp = cagra.SearchParams(itopk_size=64, **SEARCH)  # CAGRA knobs are accepted and do nothing
    D, I = cagra.search(sp, index, queries, K)
    assert np.array_equal(I, I_ref) and np.array_equal(D, D_ref)
    # device arrays in, the caller's own output arrays filled and returned
    q = torch.as_tensor(queries, device="cuda")
    nb = torch.empty((len(queries), K), dtype=torch.int64, device="cuda")
    ds = torch.empty((len(queries), K), dtype=torch.float32, device="cuda")
    D2, I2 = cagra.search(sp, index, q, K, neighbors=nb, distances=ds)
    assert I2 is nb and D2 is ds
    assert np.array_equal(nb.cpu().numpy(), I_ref) and np.array_equal(ds.cpu().numpy(), D_ref)
    native.close()


def test_cuvs_load_forms_and_save(native_dir, tmp_path):
    path, queries = native_dir
    a = cagra.load(path, placement="replicate", copies_limit=4)
    b = cagra.load(cagra.Index(), path, placement="replicate", copies_limit=4)  # the cuVS 26.10 form
    assert a.size == b.size == 20000 and a.octex.copies == 4
    Da, Ia = cagra.search(cagra.SearchParams(**SEARCH), a, queries[:50], K)
    Db, Ib = cagra.search(cagra.SearchParams(**SEARCH), b, queries[:50], K)
    assert np.array_equal(Ia, Ib) and np.array_equal(Da, Db)
    copy = str(tmp_path / "copy")
    cagra.save(copy, a)
    c = cagra.load(copy, placement="replicate", copies_limit=4)
    Dc, Ic = cagra.search(cagra.SearchParams(**SEARCH), c, queries[:50], K)
    assert np.array_equal(Ia, Ic)
    with pytest.raises(FileExistsError):
        cagra.save(copy, a)


def test_cuvs_build_same_calls_as_cagra():
    import torch
    X, Q, gt = data()
    Xd, Qd = torch.as_tensor(X, device="cuda"), torch.as_tensor(Q, device="cuda")
    index = cagra.build(cagra.IndexParams(metric="sqeuclidean", graph_degree=32, placement="replicate",
                                          **BUILD), Xd)
    distances, neighbors = cagra.search(cagra.SearchParams(**SEARCH), index, Qd, K)
    assert neighbors.shape == (200, K) and distances.shape == (200, K) and neighbors.is_cuda
    assert recall(neighbors.cpu().numpy(), gt) >= 0.9


def test_faiss_add_then_search_and_round_trip(tmp_path):
    X, Q, gt = data(seed=1)
    index = faiss.IndexOctex(X.shape[1], placement="replicate", **BUILD, **SEARCH)
    index.train(X)  # nothing to train, as for flat indexes
    index.add(X[:12000])
    index.add(X[12000:])  # ids continue in the order of the adds
    assert index.ntotal == len(X)
    D, I = index.search(Q, K)
    assert D.dtype == np.float32 and I.dtype == np.int64 and I.shape == (len(Q), K)
    assert recall(I, gt) >= 0.9
    # per-call parameters override the defaults
    D1, I1 = index.search(Q, K, params=faiss.SearchParametersOctex(read=4, starts=10, waves=1))
    assert recall(I1, gt) < recall(I, gt) + 1e-9
    # directory round trip gives the native results
    path = str(tmp_path / "faiss_idx")
    faiss.write_index(index, path)
    again = faiss.read_index(path, placement="replicate", **SEARCH)
    assert again.ntotal == len(X) and again.d == X.shape[1] and again.is_trained
    D2, I2 = again.search(Q, K)
    assert np.array_equal(I2, I) and np.array_equal(D2, D)
    native = octex_b200.load(path, placement="replicate")
    D3, I3 = native.search(Q, K, **SEARCH)
    assert np.array_equal(I3, I)
    # GpuIndexCagra builds in train, as in Faiss
    cagra_like = faiss.GpuIndexCagra(faiss.StandardGpuResources(), X.shape[1], faiss.METRIC_L2,
                                     placement="replicate", **BUILD, **SEARCH)
    cagra_like.train(X)
    assert cagra_like.is_trained and cagra_like.ntotal == len(X)
    D4, I4 = cagra_like.search(Q, K)
    assert recall(I4, gt) >= 0.9
