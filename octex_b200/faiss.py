"""GPU indexes with the interface of ``faiss.Index`` answered by this package (the reference's
``octex.faiss``, octex/faiss.py:44-166 of hpdic/octex).  Faiss itself is not imported.

    from octex_b200 import faiss                  # was: import faiss
    index = faiss.IndexOctex(d)                   # or faiss.GpuIndexCagra(faiss.StandardGpuResources(), d)
    index.add(xb)                                 # batches add up; ids are positions in the order of the adds
    D, I = index.search(xq, k)                    # float32 squared distances, int64 ids, nearest first
    faiss.write_index(index, "index_dir"); index = faiss.read_index("index_dir")

The index is built by the first search after an ``add`` (or by ``build()``); ``GpuIndexCagra``
builds in ``train`` as Faiss does.  Only ``METRIC_L2`` is supported.
"""
from __future__ import annotations

import os

import numpy as np

from . import index as _native

METRIC_INNER_PRODUCT = 0  # faiss.METRIC_INNER_PRODUCT
METRIC_L2 = 1             # faiss.METRIC_L2
_PLACEMENT = ("placement", "vectors_on_host", "shard_vectors", "table_on_host", "sketch")


def _host_rows(x, d):
    """A batch of vectors as a host float32 / float16 matrix of ``d`` columns."""
    a, _ = _native.adopt(x)
    if _native._is_torch(a):
        a = a.detach().cpu().numpy()
    a = np.asarray(a)
    if a.dtype not in (np.float32, np.float16):
        a = a.astype(np.float32)
    if a.ndim != 2 or a.shape[1] != d:
        got = a.shape[1] if a.ndim == 2 else a.shape
        raise ValueError(f"octex.faiss: vectors have dimension {got}, the index {d}")
    return a


class SearchParametersOctex:
    """Search parameters of one call (fields of ``search_params``); CAGRA's fields are dropped."""

    def __init__(self, **fields):
        self.params = {n: v for n, v in fields.items() if n in _native.SEARCH_PARAMS}


SearchParametersCagra = SearchParametersOctex


class IndexOctex:
    """``d``, ``ntotal``, ``is_trained``, ``metric_type``, ``train``, ``add``, ``search``, ``reset``
    as on a ``faiss.Index``.  Keyword arguments: index parameters (copies, list_len, ...), placement
    (placement, vectors_on_host, ...) and default search parameters (read, starts, waves, ...)."""

    def __init__(self, d, metric=METRIC_L2, **options):
        if metric != METRIC_L2:
            raise ValueError("octex.faiss: only METRIC_L2 is supported (the search is by squared "
                             "Euclidean distance)")
        self.d = int(d)
        self.metric_type = metric
        self.is_trained = True
        self.index_params, self.load_args, self.search_params = {}, {}, {}
        stray = []
        for name, value in options.items():
            if name in _PLACEMENT:
                self.load_args[name] = value
            elif name in _native.INDEX_PARAMS:
                self.index_params[name] = value
            elif name in _native.SEARCH_PARAMS:
                self.search_params[name] = value
            else:
                stray.append(name)
        if stray:
            raise TypeError(f"octex.faiss: unknown parameters {sorted(stray)}")
        self.reset()

    def reset(self):
        self._rows = []     # host batches already in the built index, in order
        self._waiting = []  # batches added since the last build
        self._native_index = None

    @property
    def ntotal(self):
        have = self._native_index.size if self._native_index is not None else 0
        return have + sum(len(b) for b in self._waiting)

    def train(self, x):
        """Nothing to train (as for a flat index)."""

    def add(self, x):
        self._waiting.append(_host_rows(x, self.d))

    def build(self):
        """Index everything added so far (the first search after an ``add`` does it too)."""
        if self._native_index is not None and not self._waiting:
            return self
        if self._native_index is not None and not self._rows:
            # came from a directory: its stored vectors are the rows so far
            self._rows = [np.asarray(_native.stored_vectors(self._native_index.path))]
        batches = self._rows + self._waiting
        if not batches:
            raise RuntimeError("octex.faiss: the index is empty")
        if len(batches) == 1:
            rows = batches[0]
        else:
            rows = np.concatenate([b.astype(np.float32, copy=False) for b in batches])
        if self._native_index is not None:
            self._native_index.close()
        self._native_index = _native.build(rows, **self.load_args, **self.index_params)
        self._rows, self._waiting = batches, []
        return self

    def search(self, x, k, *, params=None, D=None, I=None):
        if self._native_index is None or self._waiting:
            self.build()
        chosen = dict(self.search_params)
        chosen.update(getattr(params, "params", None) or {})
        return self._native_index.search(x, k, distances=D, neighbors=I, **chosen)

    @property
    def octex(self):
        """The ``octex_b200.Index`` behind this index (built on access)."""
        return self.build()._native_index


class StandardGpuResources:
    """Stands in for ``faiss.StandardGpuResources``: this package manages its own CUDA resources."""

    def noTempMemory(self):
        pass

    def setTempMemory(self, size):
        pass


class GpuIndexCagraConfig:
    """Stands in for ``faiss.GpuIndexCagraConfig``: ``device`` picks the GPU, the rest is unused."""

    def __init__(self):
        self.device = None
        self.graph_degree = 64
        self.intermediate_graph_degree = 128


class GpuIndexCagra(IndexOctex):
    """``faiss.GpuIndexCagra(res, d, metric, config)``: ``train(x)`` builds the index of ``x``."""

    def __init__(self, res=None, d=None, metric=METRIC_L2, config=None, **options):
        if d is None and isinstance(res, int):  # GpuIndexCagra(d)
            res, d = None, res
        device = getattr(config, "device", None)
        if device is not None and "devices" not in options:
            options["devices"] = [int(device)]
        super().__init__(d, metric, **options)
        self.is_trained = False

    def train(self, x):
        self.reset()
        IndexOctex.add(self, x)
        self.build()
        self.is_trained = True

    def add(self, x):
        IndexOctex.add(self, x)
        self.is_trained = True


def write_index(index, path):
    """Write the directory of an ``IndexOctex`` (built first if needed) to ``path``."""
    index.octex.save(os.fspath(path))


def read_index(path, **options):
    """An ``IndexOctex`` over an index directory; placement and default search parameters as
    keyword arguments."""
    defaults = {n: v for n, v in options.items() if n in _native.SEARCH_PARAMS}
    where = {n: v for n, v in options.items() if n not in _native.SEARCH_PARAMS}
    native = _native.load(os.fspath(path), **where)
    index = IndexOctex(native.dim, **defaults)
    index._native_index = native
    return index
