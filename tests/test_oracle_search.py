"""The CPU checker's search: the behaviours the reference's kernel tests pin
(cpp/tests/test_search.cu:86-504 of hpdic/octex) restated on small seeded indexes, and recall
against exact brute force (tests/test_recall.py:31-47)."""
import numpy as np
import pytest

from conftest import recall


@pytest.fixture(scope="module")
def ox(oracle, small_index):
    arrays, meta, base, queries = small_index
    return oracle.Index(arrays, meta), arrays, meta, base, queries


def test_recall_and_order(ox, oracle):
    ix, arrays, meta, base, queries = ox
    truth, _ = oracle.brute_force(arrays["vectors"].astype(np.float32), queries, 10)
    ids, dist, _ = ix.search(queries, 10, read=8, starts=32, waves=1)
    assert recall(ids, truth) >= 0.95
    assert (np.diff(dist, axis=1) >= 0).all(), "nearest first"
    # distances are exact fp32 squared L2 to the fp16 rows
    v = arrays["vectors"].astype(np.float32)
    want = ((v[ids[:, 0]] - queries) ** 2).sum(1)
    np.testing.assert_allclose(dist[:, 0], want, rtol=1e-4)
    ids2, _, _ = ix.search(queries, 10, read=16, starts=64, waves=2)
    assert recall(ids2, truth) >= recall(ids, truth) - 1e-9


def test_probe_matches_csr(ox):
    """seg = ((base + p) * list_len, read) for the finest level that holds the query's cell, (0, 0)
    when none does (test_search.cu:86-170)."""
    ix, arrays, meta, _, queries = ox
    _, _, t = ix.search(queries[:50], 10, read=5, starts=16, waves=0, taps=("codes", "seg"))
    C, L, l = meta["copies"], len(meta["spacings"]), meta["list_len"]
    T = 1 << meta["log_buckets"]
    for q in range(50):
        for c in range(C):
            want = (0, 0)
            for j in range(L):
                h = int(t["codes"][q, c, j])
                o = arrays["offsets"][c, j]
                b = h & (T - 1)
                hit = [p for p in range(o[b], o[b + 1]) if int(arrays["keys"][c, j, p]) == h]
                if hit:
                    want = ((int(arrays["base"][c, j]) + hit[0]) * l, 5)
                    break
            assert tuple(t["seg"][q, c]) == want


def test_candidates_are_the_union(ox):
    """Distinct ids of all segments, each once (test_search.cu:185-288)."""
    ix, arrays, meta, _, queries = ox
    _, _, t = ix.search(queries[:40], 10, read=8, starts=16, waves=0, taps=("seg", "cand1"))
    for q in range(40):
        want = set()
        for c in range(meta["copies"]):
            s, n = t["seg"][q, c]
            want |= set(arrays["lists"][c, s:s + n].tolist())
        got = t["cand1"][q, :t["n1"][q]]
        assert len(set(got.tolist())) == len(got) and set(got.tolist()) == want


def test_waves_zero_and_padding(ox):
    ix, _, _, _, queries = ox
    ids, dist, _ = ix.search(queries[:20], 10, read=1, starts=4, waves=0, rerank=2)
    assert ids.shape == (20, 10)
    short = ids < 0
    assert short.any(), "rerank depth 2 leaves fewer than k results"
    assert np.isinf(dist[short]).all() and (ids[short] == -1).all()
    assert (~short[:, 0]).all()


def test_sketch_rank_modes(ox, oracle):
    ix, arrays, _, _, queries = ox
    truth, _ = oracle.brute_force(arrays["vectors"].astype(np.float32), queries, 10)
    ids, dist, _ = ix.search(queries, 10, read=8, starts=64, waves=2, sketch_rank=True, final_rerank=32)
    assert recall(ids, truth) >= 0.75  # a 32-coordinate sketch ranks 48-dimensional rows roughly
    assert (np.diff(dist, axis=1) >= 0).all()
    ids0, dist0, _ = ix.search(queries, 10, read=8, starts=64, waves=2, sketch_rank=True, final_rerank=0)
    assert (np.diff(dist0, axis=1) >= 0).all(), "sketch order when final_rerank is 0"


def test_parts_merge(ox, oracle):
    """A sharded first round (copies split in 3) still finds the neighbors; the merged kept list
    holds each id once (test_search.cu:416-472)."""
    ix, arrays, _, _, queries = ox
    truth, _ = oracle.brute_force(arrays["vectors"].astype(np.float32), queries, 10)
    ids, _, t = ix.search(queries, 10, read=8, starts=32, waves=1, parts=3, taps=("kept1_ids",))
    assert recall(ids, truth) >= 0.95
    for row in t["kept1_ids"]:
        real = row[row >= 0]
        assert len(set(real.tolist())) == len(real)


def test_errors(ox):
    ix, _, _, _, queries = ox
    with pytest.raises(RuntimeError, match="read, starts"):
        ix.search(queries[:2], 10, read=0)
    with pytest.raises(RuntimeError, match="k >= 1"):
        ix.search(queries[:2], 0)


def test_sketch_distance_forms_agree(oracle, small_index, wide_index):
    """The sketch distance in the reference's fp32 terms, sum (c s - q)^2
    (cpp/src/neighbors/octex/detail/search_kernels.cuh:228-251), and in the integer form the CUDA
    path evaluates (row constant - 2 alpha * int8 x int16 dot product + query constant): values
    within 1e-3 relative (the 16-bit weights; the sketch distance only ranks candidates for the
    exact rerank), and the same neighbours from the same candidates."""
    for arrays, meta, _, queries in (small_index, wide_index):
        ix = oracle.Index(arrays, meta)
        for kw in (dict(read=8, starts=32, waves=2, rerank=64, wave_rerank=64),
                   dict(read=16, starts=16, waves=0, rerank=32)):
            i0, d0, t0 = ix.search(queries, 10, taps=("cand1",), sketch_form="reference", **kw)
            i1, d1, t1 = ix.search(queries, 10, taps=("cand1",), sketch_form="product", **kw)
            assert np.array_equal(t0["cand1"], t1["cand1"])
            held = t0["cand1"] >= 0
            a, b = t0["cand1_dist"][held], t1["cand1_dist"][held]
            assert (b >= 0).all()
            assert np.max(np.abs(a - b) / (1.0 + np.abs(a))) < 1e-3
            assert (i0 == i1).mean() >= 0.999
            same = i0 == i1
            assert np.allclose(d0[same], d1[same], rtol=1e-3)
        # a search that ranks by sketch distance takes the fp32 sum in both forms: identical answers
        kw = dict(read=8, starts=48, waves=1, sketch_rank=True, final_rerank=32)
        i0, d0, _ = ix.search(queries, 10, sketch_form="reference", **kw)
        i1, d1, _ = ix.search(queries, 10, sketch_form="product", **kw)
        assert np.array_equal(i0, i1) and np.array_equal(d0, d1)
