"""The GPU index builder (cuvsOctexBuild / octexB200Build) against independent checks of what it
writes, in the manner of the reference's own build tests (cpp/tests/test_build.cu:180-513 of
hpdic/octex): shapes and dtypes of the directory, consistency of the cell arrays, lists made of a
cell's own rows nearest first, the sketch against its definition, the neighbor table against brute
force with the reverse-edge rule, and the recall of a search over the result."""
import json
import os

import numpy as np
import pytest

import octex_b200
from conftest import recall

pytestmark = pytest.mark.gpu

PARAMS = dict(copies=6, blocks=4, pca_dims=64, list_len=16, min_cell=3, log_buckets=12,
              sketch_width=64, table_len=24, seed=5)


@pytest.fixture(scope="module")
def built(tmp_path_factory):
    from octex_b200 import synth
    base = synth.plumbing(30000, 96, seed=0)
    queries = synth.plumbing(400, 96, seed=1)
    path = str(tmp_path_factory.mktemp("native") / "idx")
    octex_b200.build_native(base, path, **PARAMS)
    arrays = {name[:-4]: np.load(os.path.join(path, name)) for name in os.listdir(path) if name.endswith(".npy")}
    meta = json.load(open(os.path.join(path, "meta.json")))
    return path, arrays, meta, base, queries


def test_directory_shapes(built):
    _, a, meta, base, _ = built
    n, D = base.shape
    C, L, w, l, T1 = 6, 5, 32, 16, (1 << 12) + 1
    assert meta["format"] == 1 and meta["n"] == n and meta["dim"] == D and meta["copies"] == C
    assert meta["blocks"] == 4 and meta["list_len"] == l and meta["log_buckets"] == 12
    assert meta["sketch_width"] == 64 and meta["table_len"] == 24 and meta["metric"] == "sqeuclidean"
    assert np.allclose(meta["spacings"], [2, 2.5, 3.2, 4, 5])
    assert a["mean"].shape == (D,) and a["mean"].dtype == np.float32
    assert a["proj"].shape == (C, D, w) and a["shift"].shape == (C, w)
    assert a["lists"].dtype == np.int32 and a["lists"].shape[0] == C and a["lists"].shape[1] % l == 0
    assert a["keys"].dtype == np.int64 and a["keys"].shape[:2] == (C, L)
    assert a["offsets"].shape == (C, L, T1) and a["offsets"].dtype == np.int32
    assert a["base"].shape == (C, L) and a["cells"].shape == (C, L)
    assert a["sketch"].shape == (n, 64) and a["sketch"].dtype == np.int8
    assert a["vectors"].shape == (n, D) and a["vectors"].dtype == np.float16
    assert a["table"].shape == (n, 24) and a["table"].dtype == np.int32
    assert np.array_equal(a["vectors"], base.astype(np.float16))
    assert (a["shift"] >= 0).all() and (a["shift"] < 2).all()


def test_cells_are_consistent(built, oracle):
    """Bucket bounds, codes and lists of every (copy, spacing): the cells are in (bucket, code)
    order, a cell's list holds rows whose own code is the cell's, nearest to the cell centre first,
    and every row of a kept cell's population is accounted for by the cell counts."""
    _, a, meta, base, _ = built
    n, D = base.shape
    C, L, l, T = 6, 5, 16, 1 << 12
    x16 = a["vectors"].astype(np.float32)
    for c in range(C):
        y = (x16 - a["mean"]) @ a["proj"][c] + a["shift"][c]
        row = 0
        for j in range(L):
            f = meta["spacings"][j]
            M = int(a["cells"][c, j])
            assert a["base"][c, j] == row
            off = a["offsets"][c, j]
            keys = a["keys"][c, j, :M]
            assert off[0] == 0 and off[-1] == M and (np.diff(off) >= 0).all()
            bucket = keys & (T - 1)
            assert (np.diff(bucket) >= 0).all()
            assert np.array_equal(np.searchsorted(bucket, np.arange(T + 1)), off)
            same = np.diff(bucket) == 0
            assert (np.diff(keys)[same] > 0).all(), "codes ascend inside a bucket"
            assert len(np.unique(keys)) == M
            codes = oracle.cell_code(y, 4, float(np.float32(1.0 / f)))
            uniq, pop = np.unique(codes, return_counts=True)
            want = uniq if j == L - 1 else uniq[pop >= 3]
            # the projection here sums in another order than the builder's kernel: a row next to a
            # cell wall may fall on the other side, so the sets agree up to a few cells
            assert len(np.setxor1d(want, keys)) <= max(4, 0.01 * len(want)), (c, j)
            lists = a["lists"][c, row * l:(row + M) * l].reshape(M, l)
            assert lists.min() >= 0 and lists.max() < n
            agree = codes[lists] == keys[:, None]
            assert agree.mean() > 0.995, (c, j, float(agree.mean()))
            # members nearest to the centre first; short cells repeat their nearest row
            centre = f * oracle.e8_point((y[lists[:, 0]] / f).reshape(-1, 8)).reshape(M, 32)
            d = ((y[lists] - centre[:, None, :]) ** 2).sum(-1)
            own = np.ones((M, l), bool)  # entries before the padding (repeats of the nearest row)
            own[:, 1:] = np.cumprod(lists[:, 1:] != lists[:, :1], axis=1).astype(bool)
            steps = np.diff(d, axis=1)[own[:, 1:]]
            assert (steps >= -1e-3).mean() > 0.999
            short = ~own[:, -1]
            assert (lists[short, -1] == lists[short, 0]).all()
            row += M
        assert a["lists"].shape[1] >= row * l


def test_sketch_follows_its_definition(built):
    _, a, _, base, _ = built
    x16 = a["vectors"].astype(np.float32)
    v = (x16 - a["mean"]) @ a["sketch_basis"]
    amax = np.abs(v).max(0)
    assert np.allclose(a["sketch_scale"], amax / 127.0, rtol=1e-4)
    want = np.clip(np.rint(v / a["sketch_scale"]), -127, 127)
    assert (np.abs(a["sketch"].astype(np.float32) - want) <= 1).all()
    assert (a["sketch"].astype(np.float32) == want).mean() > 0.99
    # the basis is orthonormal (the leading principal directions of the sample)
    g = a["sketch_basis"].T @ a["sketch_basis"]
    assert np.allclose(g, np.eye(64), atol=1e-3)


def test_table_is_exact_with_reverse_edges(built, oracle):
    _, a, _, base, _ = built
    n = len(base)
    k, h = 24, 12
    x16 = a["vectors"].astype(np.float32)
    rows = np.arange(0, n, 97)
    # brute force among all rows for a sample of rows (self excluded)
    ids, dist = oracle.brute_force(x16, x16[rows], k + 1)
    table = a["table"]
    for t, v in enumerate(rows):
        fwd = [i for i in ids[t] if i != v][:k]
        got = table[v]
        got = got[got >= 0]
        assert len(set(got.tolist())) == len(got) and v not in got
        # the first half of the exact neighbors always stay
        assert set(fwd[:h]) <= set(got.tolist()), v
        # whatever else is there is an exact neighbor or a row that lists v among its first half
        for u in set(got.tolist()) - set(fwd):
            first_half_of_u = [i for i in oracle.brute_force(x16, x16[u:u + 1], h + 1)[0][0] if i != u][:h]
            assert v in first_half_of_u, (v, u)
        # nearest first
        d = ((x16[got] - x16[v]) ** 2).sum(1)
        assert (np.diff(d) >= -1e-2 * (1 + d[:-1])).all()


def test_search_over_the_built_index(built, oracle):
    path, a, meta, base, queries = built
    idx = octex_b200.load(path, devices=[0], placement="replicate")
    dist, ids = idx.search(queries, 10, read=16, starts=64, waves=2, rerank=128, wave_rerank=128)
    truth, _ = oracle.brute_force(a["vectors"].astype(np.float32), queries, 10)
    r = recall(ids, truth)
    print(f"recall@10 over the GPU-built index: {r:.4f}")
    assert r >= 0.95
    # and the checker reads the same directory to the same answer
    idx.set_projection(ordered=True)
    dist, ids = idx.search(queries, 10, read=8, starts=32, waves=1)
    want_i, want_d, _ = oracle.Index(a, meta).search(queries, 10, read=8, starts=32, waves=1)
    assert np.array_equal(ids, want_i) and np.array_equal(dist.view(np.uint32), want_d.view(np.uint32))
    idx.close()


def test_build_through_the_reference_call(tmp_path):
    """cuvsOctexBuild on a DLPack tensor, float16 data on the device, then octex_b200.build."""
    import ctypes as C
    import torch
    from octex_b200 import _lib, synth
    base = synth.plumbing(5000, 32, seed=3)
    x = torch.as_tensor(base, device="cuda").half()
    p, keep = octex_b200.index_params(copies=3, blocks=2, pca_dims=16, list_len=8, log_buckets=10, table_len=8)
    t = _lib.DLManagedTensor()
    shape = (C.c_int64 * 2)(*x.shape)
    t.dl_tensor.data = x.data_ptr()
    t.dl_tensor.device = _lib.DLDevice(2, 0)
    t.dl_tensor.ndim = 2
    t.dl_tensor.dtype = _lib.DLDataType(2, 16, 1)
    t.dl_tensor.shape = shape
    path = str(tmp_path / "a")
    os.makedirs(path)
    rc = _lib.lib().cuvsOctexBuild(C.c_size_t(0), C.byref(p), C.byref(t), path.encode())
    assert rc == _lib.CUVS_SUCCESS, _lib.lib().cuvsGetLastErrorText()
    meta = json.load(open(os.path.join(path, "meta.json")))
    assert meta["n"] == 5000 and meta["sketch_width"] == 32 and meta["blocks"] == 2
    # a float64 dataset is refused with the reference's text
    t.dl_tensor.dtype = _lib.DLDataType(2, 64, 1)
    assert _lib.lib().cuvsOctexBuild(C.c_size_t(0), C.byref(p), C.byref(t), path.encode()) == _lib.CUVS_ERROR
    assert b"float32 or float16" in _lib.lib().cuvsGetLastErrorText()
    # the package call builds and loads
    idx = octex_b200.build(base, str(tmp_path / "b"), copies=4, blocks=2, pca_dims=16, list_len=8,
                           log_buckets=10, table_len=8, placement="replicate", devices=[0])
    d, i = idx.search(base[:50], 5, read=8, starts=16, waves=1)
    assert (i[:, 0] == np.arange(50)).mean() > 0.9  # a row's nearest neighbor is itself
    idx.close()


@pytest.mark.parametrize("n,dim,k", [(3000, 96, 24), (1000, 128, 64), (777, 32, 120), (2500, 960, 16), (130, 8, 7)])
def test_tensor_core_neighbor_scan(n, dim, k):
    """octexB200ExactNeighbors: the tcgen05 scan against the plain scan and against float64 brute
    force over the same fp16 rows (ragged last tiles, one to fifteen 64-wide steps of the dimension,
    short and long lists, more rows asked for than some tiles hold)."""
    import torch
    from octex_b200 import synth
    x = torch.as_tensor(synth.plumbing(n, dim, seed=11), device="cuda").half()
    ids_t, d_t = octex_b200.exact_neighbors(x, k, method="tensor")
    ids_p, d_p = octex_b200.exact_neighbors(x, k, method="plain")
    ids_t, d_t, ids_p, d_p = (a.cpu().numpy() for a in (ids_t, d_t, ids_p, d_p))
    xf = x.double().cpu().numpy()
    g = xf @ xf.T
    sq = np.diag(g)
    full = sq[:, None] + sq[None, :] - 2 * g
    np.fill_diagonal(full, np.inf)
    order = np.argsort(full, axis=1, kind="stable")[:, :k]
    want_d = np.take_along_axis(full, order, axis=1)
    for ids, d in ((ids_t, d_t), (ids_p, d_p)):
        assert (ids >= 0).all() and (ids != np.arange(n)[:, None]).all()
        assert all(len(set(r.tolist())) == k for r in ids)
        assert (np.diff(d, axis=1) >= 0).all()                       # nearest first
        # the distances are those of the named rows, and as small as the exact ones, up to fp32
        # rounding of |a|^2 + |b|^2 - 2 a.b
        scale = 1e-3 * (1 + sq.max())
        assert np.abs(np.take_along_axis(full, ids.astype(np.int64), axis=1) - d).max() < scale
        assert np.abs(d - want_d).max() < scale
    # both scans find the same rows but for near-ties
    same = np.mean([len(set(a.tolist()) & set(b.tolist())) / k for a, b in zip(ids_t, ids_p)])
    assert same > 0.999, same


def test_searched_table(built, oracle, tmp_path):
    """The table by the index's own search (octexB200SearchedTable; cuvsOctexBuild above
    exact_table_max), the way the reference checks its own (cpp/tests/test_build.cu, table quality):
    rows hold no repeats and not themselves, most of a row's true nearest neighbors are in it, a
    search over it reaches the recall of the exact table, set_table(None) drops it."""
    path, a, meta, base, queries = built
    n, k = len(base), 24
    idx = octex_b200.load(path, devices=[0], placement="replicate")
    kw = dict(read=16, starts=64, waves=2, rerank=128, wave_rerank=128)
    truth, _ = oracle.brute_force(a["vectors"].astype(np.float32), queries, 10)
    _, ids_exact = idx.search(queries, 10, **kw)
    table = idx.searched_table(table_len=k, passes=3)
    assert table.shape == (n, k) and table.dtype == np.int32
    rows = np.arange(0, n, 131)
    x16 = a["vectors"].astype(np.float32)
    near, _ = oracle.brute_force(x16, x16[rows], k // 2 + 1)
    hit = first = 0
    for t, v in enumerate(rows):
        got = table[v][table[v] >= 0]
        assert len(set(got.tolist())) == len(got) and v not in got
        want = [i for i in near[t] if i != v][:k // 2]
        hit += len(set(want) & set(got.tolist()))
        first += len(set(want[:k // 4]) & set(got.tolist()))
    # a row keeps its k / 4 nearest found neighbors first, reverse edges may displace later ones
    # (the search of this six-copy index is approximate itself)
    print(f"true nearest {k // 4} in the row: {first / (len(rows) * (k // 4)):.3f}, nearest {k // 2}: "
          f"{hit / (len(rows) * (k // 2)):.3f}")
    assert first / (len(rows) * (k // 4)) > 0.85
    assert hit / (len(rows) * (k // 2)) > 0.7
    _, ids_searched = idx.search(queries, 10, **kw)
    r_exact, r_searched = recall(ids_exact, truth), recall(ids_searched, truth)
    print(f"recall@10 exact table {r_exact:.4f}, searched table {r_searched:.4f}")
    assert r_searched > r_exact - 0.02
    # in sketch order (no exact rerank of the table's own searches): still a usable table
    idx.searched_table(table_len=k, passes=2, sketch_order=True)
    _, ids_sketch = idx.search(queries, 10, **kw)
    assert recall(ids_sketch, truth) > r_exact - 0.05
    idx.set_table(None)
    _, ids_none = idx.search(queries, 10, read=16, starts=64, waves=0, rerank=128)
    assert ids_none.shape == ids_exact.shape
    idx.set_table(a["table"])
    _, ids_back = idx.search(queries, 10, **kw)
    assert np.array_equal(ids_back, ids_exact)
    idx.close()
    # the builder takes this way by itself above exact_table_max
    small = base[:6000]
    p2 = str(tmp_path / "searched")
    octex_b200.build_native(small, p2, exact_table_max=1000, table_passes=2, **dict(PARAMS, copies=4))
    m2 = json.load(open(os.path.join(p2, "meta.json")))
    t2 = np.load(os.path.join(p2, "table.npy"))
    assert m2["table_len"] == 24 and t2.shape == (6000, 24) and (t2[:, 0] >= 0).all()
    assert "table_searched" in m2["build_seconds"]
