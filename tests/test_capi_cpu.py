"""The C boundary without a GPU: the library loads, exports every symbol the header declares,
parameter defaults are the reference's, and the argument errors that need no GPU carry the texts the
reference's C test greps for (c/tests/neighbors/octex_c.cu:203-248 of hpdic/octex, run there with
OCTEX_C_API_ONLY=1)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import octex_b200
from octex_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    import __graft_entry__
    __graft_entry__.build()
    return _lib.lib()


def test_exports_every_declared_symbol(L):
    header = open(os.path.join(ROOT, "include", "octex_b200.h")).read()
    declared = set(re.findall(r"OCTEX_B200_EXPORT\s+[\w\s\*]+?\b(\w+)\s*\(", header))
    assert len(declared) >= 31
    assert declared == set(_lib.SYMBOLS)
    for name in declared:
        assert hasattr(L, name), name


def _err(L):
    t = L.cuvsGetLastErrorText()
    return t.decode() if t else ""


def test_param_defaults(L):
    ip = C.POINTER(_lib.IndexParams)()
    assert L.cuvsOctexIndexParamsCreate(C.byref(ip)) == _lib.CUVS_SUCCESS
    p = ip.contents
    assert (p.copies, p.blocks, p.pca_dims, p.list_len, p.min_cell, p.log_buckets) == (200, 4, 64, 64, 1, 20)
    assert (p.sketch_width, p.table_len, p.list_probes, p.table_passes) == (0, 64, 16, 3)
    assert p.reverse_edges and not p.exact_lists and not p.member_lists and not p.write_behind
    assert p.exact_table_max == 20000000 and p.seed == 0
    assert not p.spacings and not p.devices
    lp = C.POINTER(_lib.LoadParams)()
    assert L.cuvsOctexLoadParamsCreate(C.byref(lp)) == _lib.CUVS_SUCCESS
    q = lp.contents
    assert q.placement == 1 and q.sketch == 0 and not q.vectors_on_host and not q.table_on_host
    assert (q.parts, q.copies_per_part, q.copies_limit, q.list_limit) == (0, 0, 0, 0)
    sp = C.POINTER(_lib.SearchParams)()
    assert L.cuvsOctexSearchParamsCreate(C.byref(sp)) == _lib.CUVS_SUCCESS
    s = sp.contents
    assert (s.read, s.starts, s.waves, s.rerank, s.wave_rerank, s.batch) == (32, 128, 2, 128, 128, 10000)
    assert not s.sketch_rank and s.final_rerank == 32
    assert s.balanced_gather and s.fused_merge and s.use_graph
    assert L.cuvsOctexSearchParamsDestroy(sp) == _lib.CUVS_SUCCESS
    assert L.cuvsOctexLoadParamsDestroy(lp) == _lib.CUVS_SUCCESS
    assert L.cuvsOctexIndexParamsDestroy(ip) == _lib.CUVS_SUCCESS


def test_errors_without_a_gpu(L):
    h = C.POINTER(_lib.IndexHandle)()
    assert L.cuvsOctexIndexCreate(C.byref(h)) == _lib.CUVS_SUCCESS
    size = C.c_int64(0)
    assert L.cuvsOctexIndexGetSize(h, C.byref(size)) == _lib.CUVS_ERROR
    assert "empty" in _err(L)

    ip = C.POINTER(_lib.IndexParams)()
    L.cuvsOctexIndexParamsCreate(C.byref(ip))
    x64 = np.zeros((2, 2), np.float64)
    shape = (C.c_int64 * 2)(2, 2)
    t = _lib.DLManagedTensor()
    t.dl_tensor.data = x64.ctypes.data
    t.dl_tensor.device = _lib.DLDevice(1, 0)
    t.dl_tensor.ndim = 2
    t.dl_tensor.dtype = _lib.DLDataType(2, 64, 1)
    t.dl_tensor.shape = shape
    assert L.cuvsOctexBuild(C.c_size_t(0), ip, C.byref(t), b"unused") == _lib.CUVS_ERROR
    assert "float32 or float16" in _err(L)
    assert L.cuvsOctexBuild(C.c_size_t(0), ip, C.byref(t), None) == _lib.CUVS_ERROR
    assert "NULL" in _err(L)

    lp = C.POINTER(_lib.LoadParams)()
    L.cuvsOctexLoadParamsCreate(C.byref(lp))
    lp.contents.placement = 7
    assert L.cuvsOctexLoad(C.c_size_t(0), b"unused", lp, h) == _lib.CUVS_ERROR
    assert "placement" in _err(L)
    lp.contents.placement = 1
    lp.contents.sketch = 9
    assert L.cuvsOctexLoad(C.c_size_t(0), b"unused", lp, h) == _lib.CUVS_ERROR
    assert "sketch placement" in _err(L)
    # a success clears the text
    assert L.cuvsOctexLoadParamsDestroy(lp) == _lib.CUVS_SUCCESS
    assert _err(L) == ""
    assert L.cuvsOctexIndexDestroy(h) == _lib.CUVS_SUCCESS
    assert L.cuvsOctexIndexParamsDestroy(ip) == _lib.CUVS_SUCCESS


def test_python_argument_checks(tmp_path):
    """Error types of the reference's Python layer (tests/test_cpu.py:24-77)."""
    with pytest.raises(TypeError, match="unknown search parameter"):
        octex_b200.search_params(reed=3)
    with pytest.raises(ValueError, match="placement must be one of"):
        octex_b200.load_params(placement="everywhere")
    with pytest.raises(ValueError, match="sketch must be one of"):
        octex_b200.load_params(sketch="disk")
    with pytest.raises(TypeError, match="unknown load parameter"):
        octex_b200.load_params(gpus=[0])
    with pytest.raises(FileNotFoundError, match="not an index directory"):
        octex_b200.load(tmp_path)
    (tmp_path / "meta.json").write_text('{"format": 1, "metric": "cosine"}')
    with pytest.raises(ValueError, match="not supported"):
        octex_b200.load(tmp_path)
    p = octex_b200.search_params(read=8, sketch_rank=True)
    assert p.read == 8 and p.sketch_rank and p.starts == 128
