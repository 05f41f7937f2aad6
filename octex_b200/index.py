"""Python side of the search path: ``load`` / ``attach`` / ``Index.search``.

Mirrors the reference's ``octex.Index.search`` and ``octex.load`` (octex/index.py:188-235,295-340 of
hpdic/octex): same argument names, defaults, error types and the ``(distances, neighbors)`` return
order, with results in the framework (numpy or torch) and on the device of the queries.  The
reference goes through a nanobind extension; this module calls the C interface of
``liboctex_b200.so`` through ctypes.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import shutil
import tempfile

import numpy as np

from . import _lib

METRICS = ("sqeuclidean", "l2")
SEARCH_PARAMS = ("read", "starts", "waves", "rerank", "wave_rerank", "batch", "sketch_rank",
                 "final_rerank")
_SWITCHES = ("use_graph",)  # fields of the C struct the reference's Python layer does not expose
LOAD_PARAMS = ("devices", "placement", "vectors_on_host", "shard_vectors", "table_on_host",
               "sketch", "parts", "copies_per_part", "copies_limit", "list_limit")
# fields of cuvs::neighbors::octex::index_params (cpp/include/cuvs/neighbors/octex.hpp:32-92); the
# builder of this package (tooling, octex_b200/build_index.py) uses the first group and accepts the
# second without effect (they choose between build strategies of the reference's builder)
INDEX_PARAMS = ("copies", "blocks", "pca_dims", "spacings", "list_len", "min_cell", "log_buckets",
                "sketch_width", "table_len", "reverse_edges", "seed", "devices",
                "exact_lists", "list_probes", "member_lists", "exact_table_max", "table_passes",
                "table_sketch_order", "write_behind")
_BUILDER_FIELDS = INDEX_PARAMS[:11]
PLACEMENTS = ("shard", "replicate")
SKETCH_PLACEMENTS = ("replicate", "shard", "host")


def check_metric(metric):
    if str(metric).lower() not in METRICS:
        raise ValueError(
            f"octex: metric {metric!r} is not supported; octex searches by squared Euclidean "
            "distance (metric='sqeuclidean')")


def _torch():
    try:
        import torch
        return torch
    except ImportError:  # pragma: no cover
        return None


def _is_torch(a):
    t = _torch()
    return t is not None and isinstance(a, t.Tensor)


def adopt(a):
    """``(array, back)``: numpy arrays and torch tensors pass through with ``back`` None. An array
    of another framework (CuPy, anything with ``__dlpack__`` or ``__cuda_array_interface__``)
    becomes a torch view of the same memory, and ``back`` turns a torch result into that
    framework's array when its module offers ``from_dlpack`` (else the torch tensor is returned) —
    results come back in the framework of the queries (octex/_arrays.py:32-150 of the reference)."""
    if isinstance(a, np.ndarray) or _is_torch(a):
        return a, None
    torch = _torch()
    if torch is not None and hasattr(a, "__dlpack__"):
        t = torch.from_dlpack(a)
    elif torch is not None and hasattr(a, "__cuda_array_interface__"):
        t = torch.as_tensor(a, device="cuda")
    else:
        return np.asarray(a), None
    import sys
    home = sys.modules.get(type(a).__module__.split(".")[0])
    give = getattr(home, "from_dlpack", None)
    return t, (lambda r: give(r) if give is not None else r)


def stored_vectors(path):
    """The fp16 vectors of an index directory, memory-mapped [n, dim]."""
    with open(os.path.join(os.fspath(path), "meta.json")) as f:
        meta = json.load(f)
    name = meta.get("files", {}).get("vectors", "vectors.npy")
    return np.load(name if os.path.isabs(name) else os.path.join(os.fspath(path), name), mmap_mode="r")


class _Resources:
    """cuvsResources_t bound to a CUDA stream."""

    def __init__(self, stream=0):
        self.h = C.c_size_t(0)
        _lib.check(_lib.lib().cuvsResourcesCreate(C.byref(self.h)))
        _lib.check(_lib.lib().cuvsStreamSet(self.h, C.c_void_p(stream)))

    def sync(self):
        _lib.check(_lib.lib().cuvsStreamSync(self.h))

    def __del__(self):
        try:
            _lib.lib().cuvsResourcesDestroy(self.h)
        except Exception:
            pass


def search_params(**kw) -> _lib.SearchParams:
    """struct cuvsOctexSearchParams with the defaults of the C++ API, then ``kw``."""
    for name in kw:
        if name not in SEARCH_PARAMS and name not in _SWITCHES:
            raise TypeError(f"octex: unknown search parameter {name!r}; valid: {', '.join(SEARCH_PARAMS)}")
    pp = C.POINTER(_lib.SearchParams)()
    _lib.check(_lib.lib().cuvsOctexSearchParamsCreate(C.byref(pp)))
    p = _lib.SearchParams()
    C.memmove(C.byref(p), pp, C.sizeof(p))
    _lib.check(_lib.lib().cuvsOctexSearchParamsDestroy(pp))
    for name, value in kw.items():
        if value is not None:
            setattr(p, name, bool(value) if name in ("sketch_rank",) + _SWITCHES else int(value))
    return p


def load_params(placement="shard", sketch="replicate", **kw):
    """(struct cuvsOctexLoadParams, keep-alive) from the reference's keyword arguments."""
    if placement not in PLACEMENTS:
        raise ValueError(f"octex: placement must be one of {PLACEMENTS}, not {placement!r}")
    if sketch not in SKETCH_PLACEMENTS:
        raise ValueError(f"octex: sketch must be one of {SKETCH_PLACEMENTS}, not {sketch!r}")
    for name in kw:
        if name not in LOAD_PARAMS:
            raise TypeError(f"octex: unknown load parameter {name!r}; valid: {', '.join(LOAD_PARAMS)}")
    p = _lib.LoadParams()
    p.placement = 1 if placement == "shard" else 0
    p.sketch = SKETCH_PLACEMENTS.index(sketch)
    keep = None
    devices = kw.get("devices")
    if devices is not None:
        devices = [int(v) for v in ([devices] if isinstance(devices, int) else devices)]
        keep = (C.c_int32 * len(devices))(*devices)
        p.devices = C.cast(keep, C.POINTER(C.c_int32))
        p.n_devices = len(devices)
    for name in ("vectors_on_host", "shard_vectors", "table_on_host"):
        if kw.get(name) is not None:
            setattr(p, name, bool(kw[name]))
    for name in ("parts", "copies_per_part", "copies_limit", "list_limit"):
        if kw.get(name) is not None:
            setattr(p, name, int(kw[name]))
    return p, keep


class Index:
    """An index placed on the GPU of this process.  Create it with ``load`` or ``attach``."""

    def __init__(self, handle, path=None, keep=None):
        self._h = handle
        self._path = None if path is None else os.fspath(path)
        self._keep = keep  # arrays borrowed by the library live as long as the index
        self._connected = False  # set by octex_b200.dist.connect
        self._res = {}  # cuvsResources per caller stream, made once

    def _get(self, fn, ctype):
        v = ctype(0)
        _lib.check(getattr(_lib.lib(), fn)(self._h, C.byref(v)))
        return int(v.value)

    @property
    def size(self):
        return self._get("cuvsOctexIndexGetSize", C.c_int64)

    @property
    def dim(self):
        return self._get("cuvsOctexIndexGetDim", C.c_int64)

    @property
    def copies(self):
        return self._get("cuvsOctexIndexGetCopies", C.c_int32)

    @property
    def devices(self):
        n = self._get("cuvsOctexIndexGetNumDevices", C.c_int32)
        out = (C.c_int32 * n)()
        _lib.check(_lib.lib().cuvsOctexIndexGetDevices(self._h, out))
        return list(out)

    @property
    def device_bytes(self):
        n = self._get("cuvsOctexIndexGetNumDevices", C.c_int32)
        out = (C.c_int64 * n)()
        _lib.check(_lib.lib().cuvsOctexIndexGetDeviceBytes(self._h, out))
        return list(out)

    @property
    def path(self):
        return self._path

    @property
    def metric(self):
        return "sqeuclidean"

    def __len__(self):
        return self.size

    def __repr__(self):
        return (f"octex_b200.Index(size={self.size}, dim={self.dim}, copies={self.copies}, "
                f"devices={self.devices})")

    def close(self):
        """Release the index.  For an index connected to other processes
        (``octex_b200.dist.connect``) this is a collective: every process calls it, and each
        returns only after all have unmapped the others' row ranges."""
        if self._h is not None:
            if self._connected:
                self._connected = False
                _lib.check(_lib.lib().octexB200CommDisconnect(self._h))
            _lib.lib().cuvsOctexIndexDestroy(self._h)
            self._h = None

    def _resources(self, stream):
        res = self._res.get(stream)
        if res is None:
            if len(self._res) > 16:
                self._res.clear()
            res = self._res[stream] = _Resources(stream)
        return res

    def memory_report(self):
        """Device memory of this process's GPU by index part, in bytes (``detail::memory_report``,
        cpp/src/neighbors/octex/search.cu:999-1016 of the reference): ``device``, ``copies``,
        ``sketch``, ``table``, ``vectors``, ``other``, and ``buffers`` of the cached search
        configuration.  Arrays kept in host memory count 0."""
        out = (C.c_int64 * 7)()
        _lib.check(_lib.lib().octexB200MemoryReport(self._h, out))
        names = ("device", "copies", "sketch", "table", "vectors", "other", "buffers")
        return dict(zip(names, (int(v) for v in out)))

    def set_table(self, table):
        """Replace the neighbor table by ``table`` int32 [n, table_len] (numpy, or a torch tensor on
        any device; copied), or drop it with ``None`` (``octexB200SetTable``).  One process only."""
        if table is None:
            _lib.check(_lib.lib().octexB200SetTable(self._h, None, C.c_int32(0)))
            return
        if _is_torch(table):
            t = table.detach().to(_torch().int32).contiguous()
            ptr, shape = t.data_ptr(), tuple(t.shape)
        else:
            t = np.ascontiguousarray(table, dtype=np.int32)
            ptr, shape = t.ctypes.data, t.shape
        if len(shape) != 2 or shape[0] != self.size:
            raise ValueError("octex: the table must be [n, table_len]")
        _lib.check(_lib.lib().octexB200SetTable(self._h, C.c_void_p(ptr), C.c_int32(shape[1])))

    def searched_table(self, table_len=64, passes=3, reverse_edges=True, sketch_order=False):
        """Make the neighbor table by this index's own search (``octexB200SearchedTable``: the
        reference's table for more rows than ``exact_table_max``), keep it, and return it as a
        numpy array int32 [n, table_len]."""
        out = np.empty((self.size, int(table_len)), np.int32)
        res = self._resources(0)
        _lib.check(_lib.lib().octexB200SearchedTable(res.h, self._h, C.c_int32(int(table_len)), C.c_int32(int(passes)),
                                                     C.c_int32(int(bool(reverse_edges))), C.c_int32(int(bool(sketch_order))),
                                                     C.c_void_p(out.ctypes.data)))
        return out

    def save(self, path):
        """Copy the index directory to ``path`` (a new or empty directory); ``load(path)`` restores
        the index (octex/index.py:259-270 of the reference)."""
        path = os.fspath(path)
        if self._path is None:
            raise ValueError("octex: this index was attached from arrays in memory and has no directory")
        if os.path.exists(path) and (not os.path.isdir(path) or os.listdir(path)):
            raise FileExistsError(f"octex: {path} exists and is not an empty directory")
        if os.path.abspath(path) != os.path.abspath(self._path):
            shutil.copytree(self._path, path, dirs_exist_ok=True)
        return path

    def __del__(self):
        try:
            self._connected = False  # no collective from a finaliser: the others may be gone
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ search
    def search(self, queries, k=10, *, read=32, starts=128, waves=2, rerank=128, wave_rerank=128,
               batch=10000, sketch_rank=False, final_rerank=32, neighbors=None, distances=None):
        """Approximate k nearest neighbors of ``queries`` [m, dim].

        Returns ``(distances, neighbors)``: float32 squared Euclidean distances and int64 ids
        [m, k], nearest first, as numpy arrays for numpy queries and as torch tensors on the
        queries' device for torch queries.  ``neighbors`` / ``distances`` receive the results in
        place when given (cast if needed) and are returned.
        """
        k = int(k)
        if k <= 0:
            raise ValueError("octex: k must be positive")
        queries, back = adopt(queries)
        if back is not None:  # another framework's arrays: work on torch views, hand back its own kind
            neighbors = None if neighbors is None else adopt(neighbors)[0]
            distances = None if distances is None else adopt(distances)[0]
            D, I = self.search(queries, k, read=read, starts=starts, waves=waves, rerank=rerank,
                               wave_rerank=wave_rerank, batch=batch, sketch_rank=sketch_rank,
                               final_rerank=final_rerank, neighbors=neighbors, distances=distances)
            return back(D), back(I)
        p = search_params(read=read, starts=starts, waves=waves, rerank=rerank,
                          wave_rerank=wave_rerank, batch=batch, sketch_rank=sketch_rank,
                          final_rerank=final_rerank)
        torch = _torch()
        if _is_torch(queries):
            q = queries.detach()
            if q.dtype != torch.float32:
                raise TypeError("octex: queries must be float32")
            q = q.contiguous()
            if q.dim() != 2:
                raise ValueError("octex: queries must be a matrix [m, dim]")
            m, d = q.shape
            on_device = q.is_cuda
            def usable(g, dt):
                return (_is_torch(g) and g.dtype == dt and g.device == q.device
                        and g.is_contiguous() and tuple(g.shape) == (m, k))
            I = neighbors if usable(neighbors, torch.int64) else \
                torch.empty((m, k), dtype=torch.int64, device=q.device)
            D = distances if usable(distances, torch.float32) else \
                torch.empty((m, k), dtype=torch.float32, device=q.device)
            ptrs = (q.data_ptr(), I.data_ptr(), D.data_ptr())
            stream = torch.cuda.current_stream(q.device).cuda_stream if on_device else 0
        else:
            q = np.ascontiguousarray(queries)
            if q.dtype != np.float32:
                raise TypeError("octex: queries must be float32")
            if q.ndim != 2:
                raise ValueError("octex: queries must be a matrix [m, dim]")
            m, d = q.shape
            on_device = False
            def usable(g, dt):
                return (isinstance(g, np.ndarray) and g.dtype == dt and g.flags.c_contiguous
                        and g.flags.writeable and g.shape == (m, k))
            I = neighbors if usable(neighbors, np.int64) else np.empty((m, k), np.int64)
            D = distances if usable(distances, np.float32) else np.empty((m, k), np.float32)
            ptrs = (q.ctypes.data, I.ctypes.data, D.ctypes.data)
            stream = 0
        if d != self.dim:
            raise ValueError(f"octex: queries have dimension {d}, the index {self.dim}")
        for given in (neighbors, distances):
            if given is not None and tuple(given.shape) != (m, k):
                raise ValueError(f"octex: output arrays must have shape {(m, k)}, not {tuple(given.shape)}")
        res = self._resources(stream)
        _lib.check(_lib.lib().octexB200Search(
            res.h, C.byref(p), self._h, C.c_void_p(ptrs[0]), C.c_int64(m), C.c_int64(d),
            C.c_void_p(ptrs[1]), C.c_void_p(ptrs[2]), C.c_int64(k), C.c_int32(1 if on_device else 0)))
        if on_device:
            res.sync()
            _lib.check(_lib.lib().octexB200CheckLast(self._h))
        if neighbors is not None and neighbors is not I:
            neighbors[...] = I if not _is_torch(neighbors) or _is_torch(I) else torch.as_tensor(I)
            I = neighbors
        if distances is not None and distances is not D:
            distances[...] = D if not _is_torch(distances) or _is_torch(D) else torch.as_tensor(D)
            D = distances
        return D, I

    # ------------------------------------------------------------------ observation
    def set_debug(self, stats=False, taps=False):
        _lib.check(_lib.lib().octexB200SetDebug(self._h, C.c_int32(int(stats)), C.c_int32(int(taps))))

    def set_projection(self, ordered=False):
        """``ordered=True``: project with the kernel that sums in dimension order (a CPU
        implementation can reproduce its coordinates bit for bit) instead of the tensor cores."""
        _lib.check(_lib.lib().octexB200SetProjection(self._h, C.c_int32(int(ordered))))

    def fetch(self, name: str, dtype, shape=None):
        """A named intermediate array of the last batch as a numpy array."""
        nbytes = C.c_int64(0)
        _lib.check(_lib.lib().octexB200Fetch(self._h, name.encode(), None, C.c_int64(0), C.byref(nbytes)))
        out = np.empty(nbytes.value // np.dtype(dtype).itemsize, dtype)
        _lib.check(_lib.lib().octexB200Fetch(self._h, name.encode(), C.c_void_p(out.ctypes.data),
                                            C.c_int64(out.nbytes), C.byref(nbytes)))
        return out if shape is None else out.reshape(shape)

    def search_resident(self, n_queries, k=10, stream=0, **kw):
        """Search again the queries the previous ``search`` left on the GPU; results stay there.
        ``stream``: the CUDA stream (handle) the work is ordered after and signals back to."""
        p = search_params(**kw)
        res = self._resources(stream)
        _lib.check(_lib.lib().octexB200SearchResident(res.h, C.byref(p), self._h,
                                                      C.c_int64(n_queries), C.c_int64(k)))

    def profile_batch(self, n_queries, k=10, **kw):
        """Milliseconds per kernel of one batch of the queries already on the GPU, as
        ``[(name, ms), ...]`` in launch order."""
        p = search_params(**kw)
        ms = (C.c_float * 64)()
        n = C.c_int32(0)
        _lib.check(_lib.lib().octexB200ProfileBatch(C.c_size_t(0), C.byref(p), self._h,
                                                    C.c_int64(n_queries), C.c_int64(k), ms,
                                                    C.c_int32(64), C.byref(n)))
        waves = int(p.waves)
        names = ["center_sketch", "project", "cell_codes", "probe", "round_lists"]
        extra = n.value - 6 - waves  # several processes: the exchanges are timed on their own
        if extra >= 3:
            names += ["exchange", "merge"]
        names += [f"round_rows[{i}]" for i in range(waves)] + ["best_k"]
        if extra in (1, 3):
            names += ["gather_results"]
        return list(zip(names, [float(ms[i]) for i in range(n.value)]))


def _new_handle():
    h = C.POINTER(_lib.IndexHandle)()
    _lib.check(_lib.lib().cuvsOctexIndexCreate(C.byref(h)))
    return h


def load(path, devices=None, placement="shard", vectors_on_host=False, *, shard_vectors=False,
         table_on_host=False, sketch="replicate", parts=0, copies_per_part=0, copies_limit=0,
         list_limit=0, rank=0, world=1):
    """Load an index directory onto the GPU of this process (``devices``: one CUDA id, default
    the current device).  ``rank`` / ``world``: this process among the processes sharing the index
    (one per GPU); with ``placement="shard"`` it holds its share of the copies."""
    path = os.fspath(path)
    if not os.path.isfile(os.path.join(path, "meta.json")):
        raise FileNotFoundError(f"octex: {path} is not an index directory (no meta.json)")
    with open(os.path.join(path, "meta.json")) as f:
        check_metric(json.load(f).get("metric", "sqeuclidean"))
    p, keep = load_params(placement=placement, sketch=sketch, devices=devices,
                          vectors_on_host=vectors_on_host, shard_vectors=shard_vectors,
                          table_on_host=table_on_host, parts=parts,
                          copies_per_part=copies_per_part, copies_limit=copies_limit,
                          list_limit=list_limit)
    h = _new_handle()
    try:
        _lib.check(_lib.lib().octexB200LoadRank(C.c_size_t(0), path.encode(), C.byref(p),
                                                C.c_int32(rank), C.c_int32(world), h))
    except Exception:
        _lib.lib().cuvsOctexIndexDestroy(h)
        raise
    del keep
    return Index(h, path)


def build(dataset, path=None, *, metric="sqeuclidean", placement="shard", vectors_on_host=False,
          table_on_host=False, shard_vectors=False, sketch="replicate", **index_params):
    """Build an index of ``dataset`` [n, dim] (float32 or float16; numpy, torch, or any array
    ``adopt`` understands) and load it — the call of the reference's ``octex.build``
    (octex/index.py:337-375).  The directory goes to ``path``, or to a temporary directory that
    lives as long as the returned index (``Index.save`` keeps it).  Keyword arguments are the
    fields of ``index_params``; ``devices`` selects the GPU the index is loaded on.

    With a GPU the library's own builder makes the directory (``octexB200Build``: member lists and
    an exact neighbor table, CUDA kernels on the current device); without one, the package's
    tooling (``octex_b200.build_index``, torch on the CPU) writes the same format for small
    data."""
    from . import build_index
    check_metric(metric)
    unknown = set(index_params) - set(INDEX_PARAMS)
    if unknown:
        raise TypeError(f"octex: unknown index parameters {sorted(unknown)}")
    torch = _torch()
    data, _ = adopt(dataset)
    dt = str(data.dtype).replace("torch.", "")
    if dt not in ("float32", "float16"):
        raise TypeError("octex: dataset must be float32 or float16")
    if len(data.shape) != 2:
        raise ValueError("octex: dataset must be a matrix [n, dim]")
    fields = {k: v for k, v in index_params.items() if k in _BUILDER_FIELDS}
    if "spacings" in fields:
        fields["spacings"] = [float(f) for f in fields["spacings"]]
    tmp = None
    if path is None:
        tmp = tempfile.TemporaryDirectory(prefix="octex-")
        path = tmp.name
    path = os.fspath(path)
    os.makedirs(path, exist_ok=True)
    if torch is not None and torch.cuda.is_available():
        build_native(data, path, **fields)
    else:
        build_index.build(data, path, build_index.IndexParams(**fields), device="cpu")
    idx = load(path, devices=index_params.get("devices"), placement=placement,
               vectors_on_host=vectors_on_host, table_on_host=table_on_host,
               shard_vectors=shard_vectors, sketch=sketch)
    idx._tmpdir = tmp
    return idx


def index_params(**kw):
    """(struct cuvsOctexIndexParams with the defaults of the C++ API, then ``kw``; keep-alive)."""
    unknown = set(kw) - set(INDEX_PARAMS)
    if unknown:
        raise TypeError(f"octex: unknown index parameters {sorted(unknown)}")
    pp = C.POINTER(_lib.IndexParams)()
    _lib.check(_lib.lib().cuvsOctexIndexParamsCreate(C.byref(pp)))
    p = _lib.IndexParams()
    C.memmove(C.byref(p), pp, C.sizeof(p))
    _lib.check(_lib.lib().cuvsOctexIndexParamsDestroy(pp))
    keep = []
    for name, value in kw.items():
        if value is None:
            continue
        if name == "spacings":
            arr = (C.c_float * len(value))(*[float(f) for f in value])
            keep.append(arr)
            p.spacings, p.n_spacings = C.cast(arr, C.POINTER(C.c_float)), len(value)
        elif name == "devices":
            devs = [int(v) for v in ([value] if isinstance(value, int) else value)]
            arr = (C.c_int32 * len(devs))(*devs)
            keep.append(arr)
            p.devices, p.n_devices = C.cast(arr, C.POINTER(C.c_int32)), len(devs)
        else:
            setattr(p, name, value)
    return p, keep


def build_native(dataset, path, verbose=False, **params):
    """Build an index directory at ``path`` with the library's own GPU builder
    (``octexB200Build``).  ``dataset`` [n, dim]: float32 or float16, numpy or torch, host or
    device memory."""
    data, _ = adopt(dataset)
    if _is_torch(data):
        data = data.detach().contiguous()
        kind, ptr = str(data.dtype).replace("torch.", ""), data.data_ptr()
    else:
        data = np.ascontiguousarray(data)
        kind, ptr = str(data.dtype), data.ctypes.data
    if kind not in ("float32", "float16"):
        raise TypeError("octex: dataset must be float32 or float16")
    if len(data.shape) != 2:
        raise ValueError("octex: dataset must be a matrix [n, dim]")
    p, keep = index_params(**params)
    os.makedirs(os.fspath(path), exist_ok=True)
    _lib.check(_lib.lib().octexB200Build(
        C.c_size_t(0), C.byref(p), C.c_void_p(ptr), C.c_int64(data.shape[0]), C.c_int64(data.shape[1]),
        C.c_int32(1 if kind == "float16" else 0), C.c_int32(int(verbose)), os.fspath(path).encode()))
    del keep
    return os.fspath(path)


def exact_neighbors(rows, k, method="auto"):
    """The ``k`` nearest other rows of every row of ``rows`` [n, dim] (a torch CUDA tensor, used as
    float16) by squared L2: ``(ids int32 [n, k], distances float32 [n, k])`` as torch tensors on the
    same GPU, nearest first (``octexB200ExactNeighbors``).  ``method``: "auto", "tensor" (the
    tcgen05 scan; dim a multiple of 8, k <= 120) or "plain"."""
    torch = _torch()
    if not (_is_torch(rows) and rows.is_cuda and rows.dim() == 2):
        raise TypeError("octex: exact_neighbors takes a torch CUDA matrix [n, dim]")
    x = rows.detach().to(torch.float16).contiguous()
    n, dim = x.shape
    ids = torch.empty((n, int(k)), dtype=torch.int32, device=x.device)
    dist = torch.empty((n, int(k)), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        torch.cuda.current_stream().synchronize()
        _lib.check(_lib.lib().octexB200ExactNeighbors(
            C.c_size_t(0), C.c_void_p(x.data_ptr()), C.c_int64(n), C.c_int32(dim), C.c_int32(int(k)),
            C.c_int32({"auto": 0, "tensor": 1, "plain": 2}[method]), C.c_void_p(ids.data_ptr()),
            C.c_void_p(dist.data_ptr())))
    return ids, dist


def _address(a):
    if a is None:
        return None
    if _is_torch(a):
        return a.data_ptr()
    return a.ctypes.data


def attach(arrays: dict, meta: dict, devices=None, placement="replicate", borrow=True, rank=0,
           world=1, **load_kw):
    """Place an index from arrays in memory (numpy arrays, or torch tensors on any device) with the
    names, dtypes and shapes of an index directory.  Device tensors that need no re-layout are used
    in place when ``borrow`` is set, and are kept alive by the returned index."""
    torch = _torch()
    want = {"mean": "float32", "proj": "float32", "shift": "float32", "lists": "int32",
            "keys": "int64", "offsets": "int32", "base": "int32", "sketch_basis": "float32",
            "sketch_scale": "float32", "sketch": "int8", "vectors": "float16", "table": "int32"}
    held = {}
    for name, dt in want.items():
        if name not in arrays:
            continue
        a = arrays[name]
        if _is_torch(a):
            a = a.detach().to(getattr(torch, dt)).contiguous()
        else:
            a = np.ascontiguousarray(a, dtype=dt)
        held[name] = a
    spac = np.asarray(meta["spacings"], np.float32)
    s = _lib.Arrays()
    s.n, s.dim, s.copies, s.blocks = meta["n"], meta["dim"], meta["copies"], meta["blocks"]
    s.list_len, s.log_buckets = meta["list_len"], meta["log_buckets"]
    s.sketch_width, s.table_len = meta["sketch_width"], meta.get("table_len", 0)
    s.spacings, s.n_spacings = spac.ctypes.data, len(spac)
    s.borrow = 1 if borrow else 0
    s.stride, s.mmax = held["lists"].shape[1], held["keys"].shape[2]
    for name in want:
        setattr(s, name, _address(held.get(name)))
    p, keep = load_params(placement=placement, devices=devices, **load_kw)
    h = _new_handle()
    try:
        _lib.check(_lib.lib().octexB200Attach(C.c_size_t(0), C.byref(s), C.byref(p),
                                              C.c_int32(rank), C.c_int32(world), h))
    except Exception:
        _lib.lib().cuvsOctexIndexDestroy(h)
        raise
    del keep
    return Index(h, None, keep=held if borrow else None)


def cell_codes(y, blocks: int, inv_f: float) -> np.ndarray:
    """Cell codes of rows of 8*blocks float32 coordinates scaled by ``inv_f``, computed on the GPU."""
    y = np.ascontiguousarray(y, np.float32).reshape(-1, 8 * blocks)
    out = np.empty(y.shape[0], np.int64)
    _lib.check(_lib.lib().octexB200CellCodes(C.c_void_p(y.ctypes.data), C.c_int64(y.shape[0]),
                                            C.c_int32(blocks), C.c_float(inv_f),
                                            C.c_void_p(out.ctypes.data)))
    return out
