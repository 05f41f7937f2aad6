"""The CPU checker against the reference's own search kernels run on this GPU.

oracle/_ref/libref_search.so holds probe_kernel, gather_kernel, rerank_keep_kernel and
pick_starts_kernel, sketch_keep_kernel, final_rerank_kernel and take_k_kernel of the reference (cpp/src/neighbors/octex/detail/search_kernels.cuh), compiled
unmodified and launched with the shapes of its search.cu.  Fed the same projected coordinates,
sketch-space queries and queries, the reference's kernels and the checker must agree: segments and
candidate sets exactly, sketch and exact distances to the last bits the different summation orders
leave (the tolerance of the reference's own tests, cpp/tests/test_search.cu:185-288: 1e-3 (1 + d)),
kept lists up to near-ties.  This is what pins the checker to the reference beyond the E8 decode;
the product's kernels are in turn compared with the checker bit for bit (test_gpu_parity.py)."""
import numpy as np
import pytest

import octex_b200

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("which", ["small", "wide"])
@pytest.mark.parametrize("kw", [
    dict(read=8, starts=32, waves=2, rerank=64, wave_rerank=64),
    dict(read=16, starts=24, waves=1, rerank=128, wave_rerank=200),
    dict(read=4, starts=16, waves=0, rerank=32),
    dict(read=8, starts=64, waves=2, sketch_rank=True, final_rerank=32),
    dict(read=8, starts=48, waves=1, sketch_rank=True, final_rerank=0),
])
def test_checker_matches_reference_kernels(oracle, small_index, wide_index, which, kw):
    if oracle.ref_search() is None:
        pytest.skip("oracle/_ref/libref_search.so was not built (reference sources not mounted)")
    arrays, meta, _, queries = small_index if which == "small" else wide_index
    queries = queries[:150]
    nq = len(queries)
    # projected coordinates and sketch-space queries of the batch: the product's own (fp16 / fp32)
    idx = octex_b200.attach(arrays, meta, borrow=False)
    idx.set_debug(stats=True, taps=True)
    idx.search(queries, 10, **kw)
    y = idx.fetch("y", np.uint16, (nq, -1))
    qs = idx.fetch("qs", np.float32, (nq, -1))
    idx.close()
    full = dict(rerank=128, wave_rerank=128)
    full.update(kw)
    ref = oracle.ref_search_pipeline(arrays, meta, y, qs, queries, 10, **full)
    # the checker evaluates the sketch distance in the reference's own fp32 terms here
    best_ids, best_dist, t = oracle.Index(arrays, meta).search(
        queries, 10, y_in=y, taps=("seg", "cand1", "kept1_ids", "kept1_dist"),
        sketch_form="reference", **kw)
    stages = [(ref["kept1_ids"], ref["kept1_dist"], t["kept1_ids"], t["kept1_dist"]),
              (ref["best_ids"], ref["best_dist"], best_ids, best_dist)]
    if not kw.get("sketch_rank"):
        # with k = KO the checker's result is its whole final kept list
        KO = max(kw["starts"], 10)
        want_ids, want_dist, _ = oracle.Index(arrays, meta).search(queries, KO, y_in=y,
                                                                   sketch_form="reference", **kw)
        stages.append((ref["kept_ids"], ref["kept_dist"], want_ids, want_dist))

    # cell lookup: identical segments
    assert np.array_equal(ref["seg"], t["seg"]), "segments"
    # first-round candidates: the same set per query, sketch distances within the reference's tolerance
    assert np.array_equal(ref["n1"], t["n1"])
    worst = 0.0
    for q in range(nq):
        n = ref["n1"][q]
        order = np.argsort(ref["cand1"][q, :n])
        assert np.array_equal(ref["cand1"][q, :n][order], t["cand1"][q, :n]), "candidate set"
        a, b = ref["dist1"][q, :n][order], t["cand1_dist"][q, :n]
        worst = max(worst, float(np.max(np.abs(a - b) / (1.0 + np.abs(b)), initial=0.0)))
    assert worst < 1e-5, worst
    # kept lists after the first round and after the waves: the same ids up to near-ties of the
    # distances (summation orders differ), distances within 1e-5 relative
    for got_i, got_d, want_i, want_d in stages:
        # rows with the same ids in the same order: distances to the last bits of the summation
        rows = (got_i == want_i).all(axis=1)
        assert rows.mean() > 0.9, float(rows.mean())
        finite = np.isfinite(want_d[rows])
        assert np.array_equal(finite, np.isfinite(got_d[rows]))
        assert np.allclose(got_d[rows][finite], want_d[rows][finite], rtol=1e-5, atol=1e-4)
        # the other rows differ by near-ties (of exact distances, or of sketch distances at the
        # rerank cut): almost all ids are shared
        shared = sum(len((set(got_i[q]) & set(want_i[q])) - {-1}) for q in range(nq))
        assert shared > 0.999 * max(int((want_i >= 0).sum()), 1), shared
