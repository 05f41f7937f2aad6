"""The calls of ``cuvs.neighbors.cagra`` answered by this package (the reference's ``octex.cuvs``,
octex/cuvs.py:70-167 of hpdic/octex, over the C interface of ``liboctex_b200.so``).

    from octex_b200 import cuvs as cagra                 # was: from cuvs.neighbors import cagra
    index = cagra.build(cagra.IndexParams(), dataset)
    distances, neighbors = cagra.search(cagra.SearchParams(), index, queries, k)
    cagra.save("index_dir", index); index = cagra.load("index_dir")

``IndexParams`` and ``SearchParams`` take the octex parameters (copies, list_len, ... and read,
starts, waves, ...).  The CAGRA parameters are accepted and do nothing; ``max_queries`` sets the
batch size.  Only ``metric="sqeuclidean"`` is supported (ValueError otherwise).  Results come back
in the framework of the queries; an index is a directory: ``save`` copies it, ``load`` reads it.
"""
from __future__ import annotations

import os

from . import index as _native

# names cuvs.neighbors.cagra knows and this search has no use for
CAGRA_INDEX_FIELDS = frozenset((
    "intermediate_graph_degree", "graph_degree", "build_algo", "nn_descent_niter",
    "ivf_pq_build_params", "ivf_pq_search_params", "ace_params", "refinement_rate", "compression",
    "guarantee_connectivity", "add_data_on_build"))
CAGRA_SEARCH_FIELDS = frozenset((
    "itopk_size", "max_iterations", "algo", "team_size", "search_width", "min_iterations",
    "thread_block_size", "hashmap_mode", "hashmap_min_bitlen", "hashmap_max_fill_rate",
    "num_random_samplings", "rand_xor_mask", "persistent", "persistent_lifetime",
    "persistent_device_usage"))
PLACEMENT_FIELDS = ("placement", "vectors_on_host", "shard_vectors", "table_on_host", "sketch")


def _sort_out(given: dict, wanted, tolerated, kind: str) -> dict:
    """The entries of ``given`` this package uses; entries CAGRA would take are dropped, anything
    else is a TypeError."""
    kept = {}
    for name in given:
        if name in wanted:
            kept[name] = given[name]
        elif name not in tolerated:
            raise TypeError(f"octex.cuvs: unknown {kind} parameter {name!r}")
    return kept


class IndexParams:
    """Build parameters: the metric, the fields of ``index_params`` and where the index is placed."""

    def __init__(self, metric="sqeuclidean", **fields):
        _native.check_metric(metric)
        self.metric = metric
        kept = _sort_out(fields, _native.INDEX_PARAMS + PLACEMENT_FIELDS, CAGRA_INDEX_FIELDS, "index")
        self.load_args = {n: kept[n] for n in kept if n in PLACEMENT_FIELDS}
        self.params = {n: kept[n] for n in kept if n not in PLACEMENT_FIELDS}

    def __repr__(self):
        return f"octex.cuvs.IndexParams(metric={self.metric!r}, {self.params}, {self.load_args})"


class SearchParams:
    """Search parameters: the fields of ``search_params``; ``max_queries`` is the batch size."""

    def __init__(self, max_queries=0, **fields):
        self.params = _sort_out(fields, _native.SEARCH_PARAMS, CAGRA_SEARCH_FIELDS, "search")
        if max_queries and "batch" not in self.params:
            self.params["batch"] = int(max_queries)

    def __repr__(self):
        return f"octex.cuvs.SearchParams({self.params})"


class Index:
    """The index handle of the cuVS calls: empty until ``build`` or ``load`` fills it."""

    def __init__(self, native=None):
        self._native = native

    def _need(self):
        if self._native is None:
            raise ValueError("octex.cuvs: the index is empty (build or load it first)")
        return self._native

    @property
    def octex(self):
        """The ``octex_b200.Index`` behind the handle."""
        return self._need()

    @property
    def trained(self):
        return self._native is not None

    @property
    def dim(self):
        return 0 if self._native is None else self._native.dim

    @property
    def size(self):
        return 0 if self._native is None else self._native.size

    def __len__(self):
        return self.size

    def __repr__(self):
        return f"octex.cuvs.Index({self._native!r})"


def build(index_params, dataset, resources=None):
    """An index of ``dataset`` [n, dim] (float32 or float16)."""
    ip = index_params if index_params is not None else IndexParams()
    return Index(_native.build(dataset, metric=ip.metric, **ip.load_args, **ip.params))


def search(search_params, index, queries, k, neighbors=None, distances=None, resources=None,
           filter=None):
    """``(distances, neighbors)`` of the k nearest neighbors, written into the given arrays if any."""
    if filter is not None:
        raise ValueError("octex.cuvs: filtered search is not supported")
    sp = search_params if search_params is not None else SearchParams()
    return index._need().search(queries, k, neighbors=neighbors, distances=distances, **sp.params)


def save(filename, index, include_dataset=True, resources=None):
    """Copy the index directory to ``filename`` (the vectors always go along)."""
    index._need().save(filename)


def load(*where, resources=None, **load_args):
    """``load(path)``, or ``load(index, path)`` as cuVS 26.10 spells it (fills the given empty
    handle); returns the handle.  Keyword arguments are those of ``octex_b200.load``."""
    if len(where) == 1:
        handle, path = Index(), where[0]
    elif len(where) == 2 and isinstance(where[0], Index):
        handle, path = where
    elif len(where) == 2 and isinstance(where[1], Index):
        path, handle = where
    else:
        raise TypeError("octex.cuvs.load(path) or load(index, path)")
    handle._native = _native.load(os.fspath(path), **load_args)
    return handle
