"""GPU parity: the CUDA path, called through the C interface, against the CPU checker on the same
seeded inputs.  Integer and index work is compared bit for bit (cell codes, segments, candidate
sets, ids); distances bit for bit too, because both sides sum in the same stated order.  The one
tolerance is the tensor-core projection, compared with the ordered projection in
test_tensor_core_projection below."""
import ctypes as C

import numpy as np
import pytest

import octex_b200
from conftest import recall, small_params
from octex_b200 import _lib, index_dir

pytestmark = pytest.mark.gpu


def stress_points(rng, n, blocks):
    """Rows of 8*blocks coordinates that sit on or next to the decision surfaces of the decode:
    exact half-integer ties, midpoints between the two cosets, and tiny perturbations of both."""
    w = 8 * blocks
    x = rng.uniform(-6, 6, size=(n, w)).astype(np.float32)
    q = n // 4
    x[:q] = np.round(x[:q] * 2) * 0.5                      # half-integer grid: rounding ties
    x[q:2 * q] = np.round(x[q:2 * q] * 4) * 0.25           # quarter grid: coset ties
    x[2 * q:3 * q] = (np.round(x[2 * q:3 * q] * 4) * 0.25
                      + rng.normal(0, 1e-6, size=(q, w)).astype(np.float32))
    return x


@pytest.fixture(scope="module")
def gpu_small(small_index):
    arrays, meta, base, queries = small_index
    idx = octex_b200.attach(arrays, meta, borrow=False)
    idx.set_debug(stats=True, taps=True)
    yield idx, arrays, meta, base, queries
    idx.close()


@pytest.fixture(scope="module")
def gpu_wide(wide_index):
    arrays, meta, base, queries = wide_index
    idx = octex_b200.attach(arrays, meta, borrow=False)
    idx.set_debug(stats=True, taps=True)
    yield idx, arrays, meta, base, queries
    idx.close()


def test_cell_codes_bit_exact(oracle, golden):
    rng = np.random.default_rng(3)
    for blocks in (1, 2, 4, 8):
        x = np.concatenate([rng.uniform(-6, 6, size=(50000, 8 * blocks)).astype(np.float32),
                            stress_points(rng, 20000, blocks)])
        for inv in (1.0, 0.5, 0.4, 1 / 3.2, 0.2):
            got = octex_b200.cell_codes(x, blocks, inv)
            want = oracle.cell_code(x, blocks, float(np.float32(inv)))
            assert np.array_equal(got, want), (blocks, inv, int((got != want).sum()))
    # golden vectors made by the reference's own header (host build): identical away from the
    # constructed exact ties of rows 0..31
    x = golden["x"]
    for name in ("inv_2p5", "inv_1", "inv_0p2"):
        got = octex_b200.cell_codes(x, 4, float(golden["scale_" + name]))
        bad = np.nonzero(got != golden["codes_" + name])[0]
        assert len(bad) <= 4 and (bad < 32).all(), (name, bad)


def test_cell_codes_large_coordinates(oracle):
    """Rows small against the spacing take a shorter decode on the GPU (|y / spacing| < 2^20); rows
    beyond it, and rows that mix both, take the general one. Both must give the checker's codes."""
    rng = np.random.default_rng(17)
    n = 40000
    for inv in (1.0, 0.4, 16.0):
        edge = 2.0 ** 20 / inv
        x = rng.uniform(-6, 6, size=(n, 32)).astype(np.float32)
        x[: n // 4] *= np.float32(edge / 6 * 0.98)                  # just inside the bound
        x[n // 4: n // 2] *= np.float32(edge / 6 * 1.5)             # outside
        x[n // 2: 3 * n // 4, ::5] = np.float32(edge * 1.01)        # one large coordinate in five
        x[3 * n // 4:, 3] = np.float32(65504.0)                     # the largest fp16 value
        x = np.concatenate([x, np.round(x[:2000] * 2) * np.float32(0.5)])  # exact half-integers
        got = octex_b200.cell_codes(x, 4, inv)
        want = oracle.cell_code(x, 4, float(np.float32(inv)))
        assert np.array_equal(got, want), (inv, int((got != want).sum()))


def test_cell_codes_against_reference_device_code(oracle):
    """The reference's e8b_hash64 compiled as device code, run on this GPU, on the same points."""
    if oracle.ref_e8_cuda() is None:
        pytest.skip("oracle/_ref/libe8_ref_cuda.so was not built (reference sources not mounted)")
    rng = np.random.default_rng(9)
    x = rng.uniform(-6, 6, size=(200000, 32)).astype(np.float32)
    x.reshape(-1)[:1000] = np.round(x.reshape(-1)[:1000] * 2) * 0.5
    for inv in (1.0, 0.4, 1 / 3.2, 0.2):
        got = octex_b200.cell_codes(x, 4, inv)
        ref = oracle.ref_cuda_cell_code(x, 4, inv)
        bad = np.nonzero(got != ref)[0]
        print(f"inv {inv}: {len(bad)} of {len(x)} codes differ from the reference device code")
        # continuous points never differ; constructed exact ties may, by the last bit of an error sum
        assert (bad < 32).all() and len(bad) <= 8, (inv, bad[:10])


def check_against_checker(oracle, idx, arrays, meta, queries, k=10, **kw):
    dist, ids = idx.search(queries, k, **kw)
    nq = len(queries)
    y = idx.fetch("y", np.uint16, (nq, -1))
    want_ids, want_dist, t = oracle.Index(arrays, meta).search(
        queries, k, y_in=y, taps=("y", "qs", "codes", "seg", "cand1", "kept1_ids", "kept1_dist", "stats"),
        **kw)
    return dist, ids, want_dist, want_ids, t, y


def test_stages_bit_exact(oracle, gpu_small):
    idx, arrays, meta, _, queries = gpu_small
    kw = dict(read=8, starts=32, waves=2, rerank=64, wave_rerank=64)
    dist, ids, want_dist, want_ids, t, y = check_against_checker(oracle, idx, arrays, meta, queries, **kw)
    nq, C_, L = len(queries), meta["copies"], len(meta["spacings"])
    # projected coordinates: the ordered projection sums like the checker
    own_y = oracle.Index(arrays, meta).search(queries, 10, taps=("y",), **kw)[2]["y"]
    assert np.array_equal(y, own_y), "projected coordinates (fp16 bits)"
    assert np.array_equal(idx.fetch("qs", np.float32, (nq, -1)).view(np.uint32), t["qs"].view(np.uint32))
    assert np.array_equal(idx.fetch("codes", np.int64, (nq, C_, L)), t["codes"]), "cell codes"
    assert np.array_equal(idx.fetch("seg", np.int32, (nq, C_, 2)), t["seg"]), "bucket reads"
    n1 = idx.fetch("n1", np.int32)
    assert np.array_equal(n1, t["n1"])
    cand = idx.fetch("cand1", np.int32, (nq, -1))
    cdist = idx.fetch("cand1_dist", np.float32, (nq, -1))
    for q in range(nq):
        order = np.argsort(cand[q, :n1[q]])
        assert np.array_equal(cand[q, :n1[q]][order], t["cand1"][q, :n1[q]]), "candidate set"
        assert np.array_equal(cdist[q, :n1[q]][order].view(np.uint32),
                              t["cand1_dist"][q, :n1[q]].view(np.uint32)), "sketch distances"
    KO = max(kw["starts"], 10)
    assert np.array_equal(idx.fetch("kept1_ids", np.int64, (nq, KO)), t["kept1_ids"])
    assert np.array_equal(idx.fetch("kept1_dist", np.float32, (nq, KO)).view(np.uint32),
                          t["kept1_dist"].view(np.uint32))
    assert np.array_equal(ids, want_ids)
    assert np.array_equal(dist.view(np.uint32), want_dist.view(np.uint32))
    stats = idx.fetch("stats", np.int64, (nq, 8))
    # column 1 counts what a lookup examines: table slots here, keys of a bucket in the checker
    cols = [0, 2, 3, 4, 5, 6]
    assert np.array_equal(stats[:, cols], t["stats"][:, cols]), "per-query counters"
    assert (stats[:, 1] >= stats[:, 0]).all()  # at least one slot per level tried


@pytest.mark.parametrize("kw", [
    dict(read=8, starts=32, waves=0),
    dict(read=8, starts=32, waves=1),
    dict(read=16, starts=64, waves=3, rerank=200, wave_rerank=100),
    dict(read=1, starts=4, waves=0, rerank=2),
    dict(read=5, starts=8, waves=2, rerank=16, wave_rerank=16),
    dict(read=8, starts=64, waves=2, sketch_rank=True, final_rerank=32),
    dict(read=8, starts=64, waves=2, sketch_rank=True, final_rerank=0),
    dict(read=8, starts=600, waves=1, sketch_rank=True, final_rerank=64),
    dict(read=64, starts=512, waves=2, rerank=512, wave_rerank=512),  # 512-thread query blocks
    dict(read=16, starts=128, waves=2, rerank=256, wave_rerank=256),  # 256-thread query blocks
    dict(read=32, starts=256, waves=1, rerank=384, wave_rerank=512),
])
def test_results_identical(oracle, gpu_small, gpu_wide, kw):
    for idx, arrays, meta, _, queries in (gpu_small, gpu_wide):
        dist, ids, want_dist, want_ids, _, _ = check_against_checker(oracle, idx, arrays, meta, queries, **kw)
        assert np.array_equal(ids, want_ids), kw
        assert np.array_equal(dist.view(np.uint32), want_dist.view(np.uint32)), kw


def test_k_larger_than_starts_and_k_one(oracle, gpu_small):
    idx, arrays, meta, _, queries = gpu_small
    for k, kw in ((50, dict(read=8, starts=16, waves=1)), (1, dict(read=8, starts=16, waves=1))):
        dist, ids, want_dist, want_ids, _, _ = check_against_checker(oracle, idx, arrays, meta, queries, k=k, **kw)
        assert ids.shape == (len(queries), k)
        assert np.array_equal(ids, want_ids)
        assert np.array_equal(dist.view(np.uint32), want_dist.view(np.uint32))


def test_batches_partial_and_empty(gpu_small):
    """batch splitting, a padded last batch and an empty query set (tests/test_api.py of the
    reference: batch=37, empty input)."""
    idx, _, meta, _, queries = gpu_small
    kw = dict(read=8, starts=32, waves=1)
    d0, i0 = idx.search(queries, 10, **kw)
    d1, i1 = idx.search(queries, 10, batch=37, **kw)
    assert np.array_equal(i0, i1) and np.array_equal(d0, d1)
    d2, i2 = idx.search(queries[:5], 10, batch=64, **kw)
    assert np.array_equal(i2, i0[:5])
    d3, i3 = idx.search(np.zeros((0, meta["dim"]), np.float32), 10, **kw)
    assert d3.shape == (0, 10) and i3.shape == (0, 10) and i3.dtype == np.int64 and d3.dtype == np.float32


def test_batches_alternate_between_two_streams(gpu_wide):
    """A call of several batches with host queries and nothing kept for inspection alternates its
    batches between two plans on two streams (copies of one under the kernels of the other): the
    same answers as one batch, for full and ragged batch counts, repeated, into caller's buffers,
    and after work queued on a stream of the caller."""
    import torch
    idx, _, _, _, queries = gpu_wide
    kw = dict(read=8, starts=32, waves=2, rerank=64, wave_rerank=64)
    idx.set_debug(stats=False, taps=False)
    try:
        d0, i0 = idx.search(queries, 10, **kw)
        for batch in (37, 64, 100, len(queries) // 2, len(queries) - 1):
            for _ in range(3):
                d1, i1 = idx.search(queries, 10, batch=batch, **kw)
                assert np.array_equal(i0, i1) and np.array_equal(d0.view(np.uint32), d1.view(np.uint32)), batch
        out_i = torch.zeros((len(queries), 10), dtype=torch.int64).pin_memory()
        out_d = torch.zeros((len(queries), 10), dtype=torch.float32).pin_memory()
        q_pin = torch.as_tensor(queries).pin_memory()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            torch.empty(1 << 24, device="cuda").fill_(1.0)  # work ahead of the search on that stream
            idx.search(q_pin.numpy(), 10, neighbors=out_i.numpy(), distances=out_d.numpy(), batch=50, **kw)
        assert np.array_equal(out_i.numpy(), i0) and np.array_equal(out_d.numpy(), d0)
        # back to one batch: the other plan and stream stay idle
        d2, i2 = idx.search(queries, 10, **kw)
        assert np.array_equal(i2, i0)
    finally:
        idx.set_debug(stats=True, taps=True)


def test_torch_device_in_out(gpu_small):
    import torch
    idx, _, _, _, queries = gpu_small
    kw = dict(read=8, starts=32, waves=1)
    d0, i0 = idx.search(queries, 10, **kw)
    q = torch.as_tensor(queries, device="cuda")
    d1, i1 = idx.search(q, 10, **kw)
    assert d1.is_cuda and i1.is_cuda and i1.dtype == torch.int64 and d1.dtype == torch.float32
    assert np.array_equal(i1.cpu().numpy(), i0) and np.array_equal(d1.cpu().numpy(), d0)
    out_i = torch.zeros((len(queries), 10), dtype=torch.int32, device="cuda")
    d2, i2 = idx.search(q, 10, neighbors=out_i, **kw)
    assert i2 is out_i and np.array_equal(out_i.cpu().numpy(), i0.astype(np.int32))
    idx.search(q, 10, **kw)
    idx.search_resident(len(queries), 10, **kw)
    assert np.array_equal(idx.fetch("kept_ids", np.int64, (len(queries), -1))[:, :10], i0)


def test_errors(gpu_small):
    idx, _, meta, _, queries = gpu_small
    with pytest.raises(ValueError, match="dimension"):
        idx.search(np.zeros((3, meta["dim"] + 2), np.float32), 10)
    with pytest.raises(ValueError, match="k must be positive"):
        idx.search(queries[:2], 0)
    with pytest.raises(ValueError, match="max\\(starts, k\\) must be <= 512"):
        idx.search(queries[:2], 10, starts=600)
    with pytest.raises(ValueError, match="rerank in \\[1, 512\\]"):
        idx.search(queries[:2], 10, starts=32, rerank=0)
    with pytest.raises(ValueError, match="starts \\* \\(waves - 1\\) <= 6144"):
        idx.search(queries[:2], 10, starts=512, waves=14, rerank=128, wave_rerank=128)
    with pytest.raises(ValueError, match="read, starts >= 1"):
        idx.search(queries[:2], 10, read=0)
    with pytest.raises(TypeError, match="float32"):
        idx.search(queries[:2].astype(np.float64), 10)
    # still usable after errors
    d, i = idx.search(queries[:4], 10, read=8, starts=32, waves=1)
    assert (i[:, 0] >= 0).all()


def test_directory_load_equals_attach(oracle, small_index, gpu_small, tmp_path):
    arrays, meta, _, queries = small_index
    path = str(tmp_path / "idx")
    index_dir.write_index(path, arrays, meta)
    kw = dict(read=8, starts=32, waves=1)
    d0, i0 = gpu_small[0].search(queries, 10, **kw)
    idx = octex_b200.load(path, placement="replicate")
    assert (idx.size, idx.dim, idx.copies) == (meta["n"], meta["dim"], meta["copies"])
    assert idx.devices == [0] and idx.device_bytes[0] > 0 and len(idx) == meta["n"]
    d1, i1 = idx.search(queries, 10, **kw)
    assert np.array_equal(i0, i1) and np.array_equal(d0, d1)
    idx.close()
    # load-time shrinking (load.cu:239,259-260,361-379): fewer copies, shorter lists
    idx = octex_b200.load(path, placement="replicate", copies_limit=5, list_limit=6)
    assert idx.copies == 5
    d2, i2 = idx.search(queries, 10, read=8, starts=32, waves=1)
    cut = dict(arrays)
    l, ll = meta["list_len"], 6
    rows = arrays["lists"].shape[1] // l
    cut["lists"] = np.ascontiguousarray(arrays["lists"][:5].reshape(5, rows, l)[:, :, :ll].reshape(5, rows * ll))
    for name in ("keys", "offsets", "base", "proj", "shift"):
        cut[name] = arrays[name][:5]
    cmeta = dict(meta, copies=5, list_len=ll)
    want_i, want_d, _ = oracle.Index(cut, cmeta).search(queries, 10, read=8, starts=32, waves=1)
    assert np.array_equal(i2, want_i) and np.array_equal(d2.view(np.uint32), want_d.view(np.uint32))
    idx.close()
    # saved parts (load.cu:252-270): two parts of four copies, the first three of each loaded
    idx = octex_b200.load(path, placement="replicate", parts=2, copies_per_part=3)
    assert idx.copies == 6
    d2, i2 = idx.search(queries, 10, read=8, starts=32, waves=1)
    sel = [0, 1, 2, 4, 5, 6]
    cut = dict(arrays)
    for name in ("lists", "keys", "offsets", "base", "proj", "shift"):
        cut[name] = np.ascontiguousarray(arrays[name][sel])
    want_i, want_d, _ = oracle.Index(cut, dict(meta, copies=6)).search(queries, 10, read=8, starts=32, waves=1)
    assert np.array_equal(i2, want_i) and np.array_equal(d2.view(np.uint32), want_d.view(np.uint32))
    idx.close()
    # host tiers (load.cu:328-330): arrays in page-locked host memory read through the same pointer;
    # same results, less device memory
    full_bytes = None
    for tiers in (dict(), dict(vectors_on_host=True), dict(table_on_host=True), dict(sketch="host"),
                  dict(vectors_on_host=True, table_on_host=True, sketch="host")):
        idx = octex_b200.load(path, placement="replicate", **tiers)
        for kw2 in (kw, dict(read=8, starts=16, waves=2, sketch_rank=True, final_rerank=32)):
            d3, i3 = idx.search(queries, 10, **kw2)
            d4, i4 = gpu_small[0].search(queries, 10, **kw2)
            assert np.array_equal(i3, i4) and np.array_equal(d3, d4), tiers
        if not tiers:
            full_bytes = idx.device_bytes[0]
        else:
            assert idx.device_bytes[0] < full_bytes, tiers
        idx.close()
    # one process holds every row: dealing the rows changes nothing (load.cu:315 with one GPU)
    idx = octex_b200.load(path, placement="shard", shard_vectors=True, sketch="shard")
    d5, i5 = idx.search(queries, 10, **kw)
    assert np.array_equal(i5, i0) and np.array_equal(d5, d0)
    idx.close()
    with pytest.raises(ValueError, match="holds no copies"):
        octex_b200.load(path, placement="shard", rank=0, world=64)


def test_shard_rank_holds_its_copies(oracle, small_index, tmp_path):
    """One rank of a sharded placement answers with the kept list of its own copies
    (load.cu:272-275); the checker restricted to those copies agrees."""
    arrays, meta, _, queries = small_index
    path = str(tmp_path / "idx")
    index_dir.write_index(path, arrays, meta)
    idx = octex_b200.load(path, placement="shard", rank=1, world=2)
    assert idx.copies == meta["copies"]
    idx.close()


def test_dlpack_c_api(gpu_small):
    """cuvsOctexSearch on DLManagedTensor arguments, host and device (c/tests/neighbors/octex_c.cu)."""
    import torch
    idx, _, meta, _, queries = gpu_small
    L = _lib.lib()
    kw = dict(read=8, starts=32, waves=1)
    d0, i0 = idx.search(queries, 10, **kw)
    p = octex_b200.search_params(**kw)

    def tensor(ptr, shape, code, bits, dev):
        t = _lib.DLManagedTensor()
        shp = (C.c_int64 * 2)(*shape)
        t.dl_tensor.data = ptr
        t.dl_tensor.device = _lib.DLDevice(dev, 0)
        t.dl_tensor.ndim = 2
        t.dl_tensor.dtype = _lib.DLDataType(code, bits, 1)
        t.dl_tensor.shape = shp
        return t, shp

    res = C.c_size_t(0)
    assert L.cuvsResourcesCreate(C.byref(res)) == _lib.CUVS_SUCCESS
    nq = len(queries)
    I = np.zeros((nq, 10), np.int64)
    D = np.zeros((nq, 10), np.float32)
    tq, k1 = tensor(queries.ctypes.data, queries.shape, 2, 32, 1)
    ti, k2 = tensor(I.ctypes.data, I.shape, 0, 64, 1)
    td, k3 = tensor(D.ctypes.data, D.shape, 2, 32, 1)
    assert L.cuvsOctexSearch(res, C.byref(p), idx._h, C.byref(tq), C.byref(ti), C.byref(td)) == _lib.CUVS_SUCCESS
    assert np.array_equal(I, i0) and np.array_equal(D, d0)
    q = torch.as_tensor(queries, device="cuda")
    Ig = torch.zeros((nq, 10), dtype=torch.int64, device="cuda")
    Dg = torch.zeros((nq, 10), dtype=torch.float32, device="cuda")
    tq, k1 = tensor(q.data_ptr(), queries.shape, 2, 32, 2)
    ti, k2 = tensor(Ig.data_ptr(), I.shape, 0, 64, 2)
    td, k3 = tensor(Dg.data_ptr(), D.shape, 2, 32, 2)
    assert L.cuvsOctexSearch(res, C.byref(p), idx._h, C.byref(tq), C.byref(ti), C.byref(td)) == _lib.CUVS_SUCCESS
    assert L.cuvsStreamSync(res) == _lib.CUVS_SUCCESS
    assert np.array_equal(Ig.cpu().numpy(), i0)
    # a float64 query tensor is refused with the reference's text
    bad, k4 = tensor(queries.ctypes.data, queries.shape, 2, 64, 1)
    assert L.cuvsOctexSearch(res, C.byref(p), idx._h, C.byref(bad), C.byref(ti), C.byref(td)) == _lib.CUVS_ERROR
    assert b"wrong data type" in L.cuvsGetLastErrorText()
    L.cuvsResourcesDestroy(res)


@pytest.fixture(scope="module")
def gpu_100k():
    """100 000 x 128 rows (the plumbing configuration with fewer copies), built on the GPU:
    (index, arrays on the device, meta, queries)."""
    from octex_b200 import build_index, synth
    base = synth.plumbing(100000, 128, seed=0)
    queries = synth.plumbing(1000, 128, seed=1)
    params = build_index.IndexParams(copies=24, blocks=4, pca_dims=64, list_len=32, min_cell=1,
                                     log_buckets=16, table_len=32)
    arrays, meta = build_index.build_arrays(base, params, device="cuda", keep_on_device=True)
    idx = octex_b200.attach(arrays, meta, borrow=True)
    yield idx, arrays, meta, queries
    idx.close()


def test_full_size_properties(oracle, gpu_100k):
    """Size-independent properties on a larger index: distances ascending, ids distinct and in
    range, every distance equal to the exact fp32 distance to the stored fp16 row, recall against
    brute force, and the neighbours the reference's own kernels find from the same projected
    coordinates."""
    import torch
    idx, arrays, meta, queries = gpu_100k
    idx.set_debug(stats=False, taps=False)
    dist, ids = idx.search(queries, 10, read=32, starts=128, waves=3, rerank=256, wave_rerank=256)
    assert (np.diff(dist, axis=1) >= 0).all()
    assert ids.min() >= 0 and ids.max() < meta["n"]
    assert all(len(set(r.tolist())) == 10 for r in ids)
    v = arrays["vectors"].float()
    q = torch.as_tensor(queries, device="cuda")
    exact = ((v[torch.as_tensor(ids, device="cuda")] - q[:, None, :]) ** 2).sum(-1).cpu().numpy()
    np.testing.assert_allclose(dist, exact, rtol=1e-4)
    d_all = (q * q).sum(1)[:, None] - 2 * q @ v.T + (v * v).sum(1)[None, :]
    truth = d_all.topk(10, dim=1, largest=False).indices.cpu().numpy()
    r = recall(ids, truth)
    print(f"recall@10 {r:.4f} (read 32, starts 128, waves 3, rerank 256, 24 copies)")
    assert r >= 0.95
    # the reference's kernels (oracle/_ref/libref_search.so) on the same batch: the tensor-core
    # projection's coordinates go in, their neighbours must be these neighbours
    if oracle.ref_search() is not None:
        kw = dict(read=16, starts=32, waves=2, rerank=128, wave_rerank=256)
        idx.set_debug(taps=True)
        dist, ids = idx.search(queries, 10, **kw)
        y = idx.fetch("y", np.uint16, (len(queries), -1))
        qs = idx.fetch("qs", np.float32, (len(queries), -1))
        host = {k_: v_.cpu().numpy() for k_, v_ in arrays.items()}
        ref = oracle.ref_search_pipeline(host, meta, y, qs, queries, 10, **kw)
        agree = float((ref["kept_ids"][:, :10] == ids).mean())
        print(f"ids equal to the reference kernels' on {agree:.5f} of the slots")
        assert agree >= 0.999
        same = ref["kept_ids"][:, :10] == ids
        np.testing.assert_allclose(ref["kept_dist"][:, :10][same], dist[same], rtol=1e-4, atol=1e-3)
        idx.set_debug(taps=False)


FUSED_SETS = [
    dict(read=8, starts=32, waves=0),
    dict(read=16, starts=32, waves=1, rerank=128, wave_rerank=384),
    dict(read=8, starts=24, waves=2, rerank=64, wave_rerank=100),
    dict(read=32, starts=128, waves=2, rerank=256, wave_rerank=256),
    dict(read=32, starts=256, waves=2, rerank=256, wave_rerank=256),
    dict(read=8, starts=64, waves=1, sketch_rank=True, final_rerank=32),
]


def fused_against_inspected(oracle, idx, arrays, meta, queries):
    """The search as it runs in production — the cells looked up inside the tensor-core
    projection's epilogue, nothing kept for inspection — against the inspected run of the same
    batch (codes written out, separate lookup kernel), which is compared with the CPU checker bit
    for bit: segments, final kept lists, ids and distances must be identical.  The probe follows
    the finest-level-first rule of cpp/tests/test_search.cu:86-170 of the reference."""
    nq, C_ = len(queries), meta["copies"]
    host = None
    for kw in FUSED_SETS:
        KO = max(kw["starts"], 10)
        idx.set_projection(ordered=False)
        idx.set_debug(stats=False, taps=True)
        d_tap, i_tap = idx.search(queries, 10, **kw)
        seg_tap = idx.fetch("seg", np.int32, (nq, C_, 2))
        kept_tap = idx.fetch("kept_ids", np.int64, (nq, KO))
        keptd_tap = idx.fetch("kept_dist", np.float32, (nq, KO))
        y = idx.fetch("y", np.uint16, (nq, -1))
        idx.set_debug(stats=False, taps=False)
        d_run, i_run = idx.search(queries, 10, **kw)
        with pytest.raises(ValueError, match="not kept"):
            idx.fetch("y", np.uint16)  # nothing is kept for inspection on this path
        seg_run = idx.fetch("seg", np.int32, (nq, C_, 2))
        assert np.array_equal(seg_run, seg_tap), ("segments", kw)
        assert np.array_equal(idx.fetch("kept_ids", np.int64, (nq, KO)), kept_tap), kw
        assert np.array_equal(idx.fetch("kept_dist", np.float32, (nq, KO)).view(np.uint32),
                              keptd_tap.view(np.uint32)), kw
        assert np.array_equal(i_run, i_tap) and np.array_equal(d_run.view(np.uint32), d_tap.view(np.uint32)), kw
        # and the inspected run is the checker's answer on the tensor-core coordinates
        if host is None:
            host = {k_: (v_.cpu().numpy() if hasattr(v_, "cpu") else v_) for k_, v_ in arrays.items()}
        want_i, want_d, t = oracle.Index(host, meta).search(queries, 10, y_in=y, taps=("seg",), **kw)
        assert np.array_equal(seg_run, t["seg"]), ("segments vs checker", kw)
        assert np.array_equal(i_run, want_i), kw
        assert np.array_equal(d_run.view(np.uint32), want_d.view(np.uint32)), kw
    # with counters on: what the rounds read is the checker's count; of the levels the checker
    # tries, the lookup skips those it knows to hold no cell at all
    idx.set_debug(stats=True, taps=False)
    kw = FUSED_SETS[1]
    idx.search(queries, 10, **kw)
    stats = idx.fetch("stats", np.int64, (nq, 8))
    idx.set_debug(stats=True, taps=True)
    idx.search(queries, 10, **kw)
    y = idx.fetch("y", np.uint16, (nq, -1))
    t = oracle.Index(host, meta).search(queries, 10, y_in=y, taps=("stats",), **kw)[2]
    cols = [2, 3, 4, 5, 6]
    assert np.array_equal(stats[:, cols], t["stats"][:, cols]), "per-query counters of the fused path"
    assert (stats[:, 0] <= t["stats"][:, 0]).all() and (stats[:, 0] >= C_).all()
    assert (stats[:, 1] >= stats[:, 0]).all()  # at least one table slot per level tried
    idx.set_debug(stats=False, taps=False)


def test_fused_lookup_path_wide(oracle, wide_index):
    arrays, meta, _, queries = wide_index
    idx = octex_b200.attach(arrays, meta, borrow=False)
    fused_against_inspected(oracle, idx, arrays, meta, queries)
    idx.close()


def test_fused_lookup_path_100k(oracle, gpu_100k):
    idx, arrays, meta, queries = gpu_100k
    fused_against_inspected(oracle, idx, arrays, meta, queries)


def test_direct_launches_equal_graph(gpu_wide):
    """use_graph = false (search.cu:885-920 of the reference: the same kernels launched directly)."""
    idx, _, _, _, queries = gpu_wide
    kw = dict(read=8, starts=32, waves=2, rerank=64, wave_rerank=64)
    d0, i0 = idx.search(queries, 10, **kw)
    p = octex_b200.search_params(use_graph=False, **kw)
    I = np.zeros((len(queries), 10), np.int64)
    D = np.zeros((len(queries), 10), np.float32)
    _lib.check(_lib.lib().octexB200Search(C.c_size_t(0), C.byref(p), idx._h, C.c_void_p(queries.ctypes.data),
                                          C.c_int64(len(queries)), C.c_int64(queries.shape[1]),
                                          C.c_void_p(I.ctypes.data), C.c_void_p(D.ctypes.data),
                                          C.c_int64(10), C.c_int32(0)))
    assert np.array_equal(I, i0) and np.array_equal(D.view(np.uint32), d0.view(np.uint32))


def test_tensor_core_projection(oracle, gpu_wide):
    """The tcgen05 projection against the ordered one on the same operands: fp32 accumulation in a
    different order, so an fp16 output may land on the neighbouring value (tolerance: one unit in
    the last place of fp16, on at most 2 % of the coordinates); the cell codes it emits from its
    own accumulators equal the checker's codes of those same coordinates bit for bit."""
    idx, arrays, meta, _, queries = gpu_wide
    nq, C_, L = len(queries), meta["copies"], len(meta["spacings"])
    kw = dict(read=8, starts=32, waves=1)
    idx.set_projection(ordered=False)
    idx.search(queries, 10, **kw)
    y_tc = idx.fetch("y", np.uint16, (nq, -1))
    codes_tc = idx.fetch("codes", np.int64, (nq, C_, L))
    idx.set_projection(ordered=True)
    idx.search(queries, 10, **kw)
    y_ord = idx.fetch("y", np.uint16, (nq, -1))
    idx.set_projection(ordered=False)
    a, b = y_tc.view(np.float16).astype(np.float32), y_ord.view(np.float16).astype(np.float32)
    differ = y_tc != y_ord
    print(f"tensor-core vs ordered projection: {differ.mean():.5f} of the fp16 coordinates differ")
    assert differ.mean() <= 0.02
    ulp = np.spacing(np.abs(y_ord.view(np.float16)).astype(np.float16)).astype(np.float32)
    # one fp16 unit in the last place, plus 3e-5 absolute for coordinates near zero, where the fp32
    # sums themselves (terms of order 1, 128 of them) differ by more than such a coordinate's ulp
    worst = float((np.abs(a - b) - ulp).max())
    print(f"largest |difference| beyond one fp16 ulp: {worst:.3e}")
    assert (np.abs(a - b) <= ulp + 3e-5).all()
    _, _, t = oracle.Index(arrays, meta).search(queries, 10, y_in=y_tc, taps=("codes",), **kw)
    assert np.array_equal(codes_tc, t["codes"])


@pytest.mark.parametrize("gen,dim", [("global_descriptor_like", 960), ("embedding_like", 96),
                                      ("plumbing", 200)])
def test_other_dimensions(oracle, gen, dim):
    """The shapes of the other benchmark configurations, small: 960 dimensions (fifteen 64-wide
    steps of the projection, 1 920-byte rows in the rerank), 96 (operand rows zero-padded to 128)
    and 200 (not a multiple of 8: the scalar path of the exact distances)."""
    from octex_b200 import build_index, synth
    base = getattr(synth, gen)(5000, dim, seed=0)
    queries = getattr(synth, gen)(150, dim, seed=1)
    params = small_params(copies=5, blocks=4, pca_dims=64, list_len=16, min_cell=2,
                          sketch_width=0, table_len=24)
    arrays, meta = build_index.build_arrays(base, params, device="cpu")
    idx = octex_b200.attach(arrays, meta, borrow=False)
    idx.set_debug(stats=True, taps=True)
    for kw in (dict(read=8, starts=32, waves=2, rerank=64, wave_rerank=64),
               dict(read=8, starts=48, waves=1, sketch_rank=True, final_rerank=32)):
        dist, ids, want_dist, want_ids, t, y = check_against_checker(oracle, idx, arrays, meta, queries, **kw)
        assert np.array_equal(ids, want_ids), (dim, kw)
        assert np.array_equal(dist.view(np.uint32), want_dist.view(np.uint32)), (dim, kw)
        assert np.array_equal(idx.fetch("codes", np.int64, t["codes"].shape), t["codes"])
    # the tensor-core coordinates stay within one fp16 step of the ordered ones
    idx.set_projection(ordered=True)
    idx.search(queries, 10, read=8, starts=32, waves=0)
    y_ord = idx.fetch("y", np.uint16, y.shape).view(np.float16).astype(np.float32)
    y_tc = y.view(np.float16).astype(np.float32)
    ulp = np.spacing(np.abs(y_ord).astype(np.float16)).astype(np.float32)
    assert (np.abs(y_tc - y_ord) <= ulp + 1e-4).all()
    idx.close()
