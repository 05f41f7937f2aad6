"""The cuVS-style and Faiss-style adapters: parameter handling and error behaviour that need no GPU
(the reference's tests/test_dropin.py and tests/test_api.py are the model)."""
import numpy as np
import pytest

from octex_b200 import cuvs as cagra
from octex_b200 import faiss
from octex_b200 import index as native


def test_cuvs_params_sort_fields():
    ip = cagra.IndexParams(metric="sqeuclidean", copies=8, list_len=16, graph_degree=32,
                           placement="replicate", build_algo="nn_descent")
    assert ip.params == {"copies": 8, "list_len": 16} and ip.load_args == {"placement": "replicate"}
    sp = cagra.SearchParams(max_queries=512, read=8, starts=16, itopk_size=64, team_size=4)
    assert sp.params == {"read": 8, "starts": 16, "batch": 512}
    assert cagra.SearchParams(max_queries=512, batch=64).params == {"batch": 64}
    with pytest.raises(TypeError, match="unknown index parameter 'bogus'"):
        cagra.IndexParams(bogus=1)
    with pytest.raises(TypeError, match="unknown search parameter"):
        cagra.SearchParams(bogus=1)
    with pytest.raises(ValueError, match="sqeuclidean"):
        cagra.IndexParams(metric="inner_product")


def test_cuvs_empty_index_and_load_forms():
    empty = cagra.Index()
    assert not empty.trained and empty.dim == 0 and empty.size == 0 and len(empty) == 0
    with pytest.raises(ValueError, match="empty"):
        cagra.search(cagra.SearchParams(), empty, np.zeros((1, 8), np.float32), 1)
    with pytest.raises(ValueError, match="empty"):
        cagra.save("nowhere", empty)
    with pytest.raises(ValueError, match="filtered"):
        cagra.search(None, empty, np.zeros((1, 8), np.float32), 1, filter=object())
    with pytest.raises(TypeError, match="load"):
        cagra.load()
    with pytest.raises(TypeError, match="load"):
        cagra.load("a", "b", "c")
    with pytest.raises(FileNotFoundError):
        cagra.load("/nonexistent/index/dir")


def test_faiss_index_bookkeeping():
    with pytest.raises(ValueError, match="METRIC_L2"):
        faiss.IndexOctex(16, faiss.METRIC_INNER_PRODUCT)
    with pytest.raises(TypeError, match="unknown parameters"):
        faiss.IndexOctex(16, bogus=3)
    ix = faiss.IndexOctex(16, copies=4, read=8, placement="replicate")
    assert ix.index_params == {"copies": 4} and ix.search_params == {"read": 8}
    assert ix.load_args == {"placement": "replicate"}
    assert ix.d == 16 and ix.ntotal == 0 and ix.is_trained and ix.metric_type == faiss.METRIC_L2
    ix.train(np.zeros((3, 16), np.float32))
    ix.add(np.zeros((3, 16), np.float32))
    ix.add(np.zeros((5, 16), np.float16))
    assert ix.ntotal == 8
    with pytest.raises(ValueError, match="dimension 8"):
        ix.add(np.zeros((2, 8), np.float32))
    ix.reset()
    assert ix.ntotal == 0
    with pytest.raises(RuntimeError, match="empty"):
        ix.build()
    g = faiss.GpuIndexCagra(faiss.StandardGpuResources(), 16, faiss.METRIC_L2)
    assert not g.is_trained
    cfg = faiss.GpuIndexCagraConfig()
    cfg.device = 0
    g2 = faiss.GpuIndexCagra(None, 16, config=cfg)
    assert g2.index_params["devices"] == [0]
    assert faiss.GpuIndexCagra(16).d == 16
    assert faiss.SearchParametersCagra(read=4, itopk_size=9).params == {"read": 4}


def test_native_build_rejects_bad_input():
    with pytest.raises(TypeError, match="unknown index parameters"):
        native.build(np.zeros((4, 8), np.float32), bogus=1)
    with pytest.raises(TypeError, match="float32 or float16"):
        native.build(np.zeros((4, 8), np.int32))
    with pytest.raises(ValueError, match="matrix"):
        native.build(np.zeros(8, np.float32))
    with pytest.raises(ValueError, match="sqeuclidean"):
        native.build(np.zeros((4, 8), np.float32), metric="cosine")
