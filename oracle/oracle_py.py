"""TEST INFRASTRUCTURE ONLY: ctypes bindings of the CPU checker (liboctex_oracle.so).

Imported by tests/, by the smoke check and by the CPU-baseline leg of the benchmark, never by the
package itself.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class OracleIndex(C.Structure):
    _fields_ = [("n", C.c_int64), ("dim", C.c_int64),
                ("copies", C.c_int32), ("blocks", C.c_int32), ("levels", C.c_int32),
                ("list_len", C.c_int32), ("log_buckets", C.c_int32), ("sketch_width", C.c_int32),
                ("table_len", C.c_int32), ("pad_", C.c_int32),
                ("stride", C.c_int64), ("mmax", C.c_int64),
                ("spacings", C.c_void_p), ("mean", C.c_void_p), ("proj", C.c_void_p),
                ("shift", C.c_void_p), ("lists", C.c_void_p), ("keys", C.c_void_p),
                ("offsets", C.c_void_p), ("base", C.c_void_p), ("basis", C.c_void_p),
                ("scale", C.c_void_p), ("sketch", C.c_void_p), ("vectors", C.c_void_p),
                ("table", C.c_void_p)]


class OracleParams(C.Structure):
    _fields_ = [("read", C.c_int32), ("starts", C.c_int32), ("waves", C.c_int32),
                ("rerank", C.c_int32), ("wave_rerank", C.c_int32), ("batch", C.c_int32),
                ("sketch_rank", C.c_int32), ("final_rerank", C.c_int32),
                ("parts", C.c_int32), ("threads", C.c_int32), ("sketch_form", C.c_int32)]


class OracleTaps(C.Structure):
    _fields_ = [("y_in", C.c_void_p), ("y", C.c_void_p), ("qs", C.c_void_p),
                ("codes", C.c_void_p), ("seg", C.c_void_p), ("cand1", C.c_void_p),
                ("cand1_dist", C.c_void_p), ("n1", C.c_void_p),
                ("cand_cap", C.c_int32), ("pad_", C.c_int32),
                ("kept1_ids", C.c_void_p), ("kept1_dist", C.c_void_p), ("stats", C.c_void_p)]


def reference_root() -> str:
    """Where the reference's sources lie: $REFERENCE, else a checkout named ``reference`` beside
    this repository (absent on most machines: then only the prebuilt _ref/ files are used)."""
    given = os.environ.get("REFERENCE")
    if given:
        return given
    return os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def build(force: bool = False) -> str:
    """Compile the checker (and, when the reference sources are present, oracle/_ref)."""
    so = os.path.join(_HERE, "liboctex_oracle.so")
    src = [os.path.join(_HERE, f) for f in ("octex_oracle.cpp", "octex_oracle.h", "e8_port.hpp")]
    stale = not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in src)
    # where the reference sources are mounted, its own code compiled into _ref/ must be there too
    reference = reference_root()
    if os.path.exists(os.path.join(reference, "cpp/src/neighbors/octex/detail/search_kernels.cuh")):
        outs = ("libe8_ref.so", "libe8_ref_fma.so", "libe8_ref_cuda.so", "libref_search.so")
        shims = [os.path.join(_HERE, f) for f in ("ref_e8_shim.cpp", "ref_e8_cuda_shim.cu", "ref_search_shim.cu")]
        for name in outs:
            p = os.path.join(_HERE, "_ref", name)
            if not os.path.exists(p) or any(os.path.getmtime(s) > os.path.getmtime(p) for s in shims):
                stale = True
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "all", "REFERENCE=" + reference],
                              stdout=subprocess.DEVNULL)
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
        _LIB.oracle_last_error.restype = C.c_char_p
    return _LIB


def ref_e8(fma: bool = False):
    """The reference's own E8 decode compiled for the host, or None when it was not built."""
    p = os.path.join(_HERE, "_ref", "libe8_ref_fma.so" if fma else "libe8_ref.so")
    return C.CDLL(p) if os.path.exists(p) else None


def ref_e8_cuda():
    """The reference's E8 decode compiled as device code (needs a GPU), or None when not built."""
    p = os.path.join(_HERE, "_ref", "libe8_ref_cuda.so")
    return C.CDLL(p) if os.path.exists(p) else None


def ref_cuda_cell_code(y: np.ndarray, blocks: int, inv_f: float) -> np.ndarray:
    lib_ = ref_e8_cuda()
    y = np.ascontiguousarray(y, np.float32)
    h = np.zeros(y.shape[0], np.int64)
    rc = lib_.ref_cuda_cell_code(_ptr(y), C.c_int64(y.shape[0]), C.c_int32(blocks),
                                 C.c_float(inv_f), _ptr(h))
    if rc != 0:
        raise RuntimeError(f"CUDA error {rc} in the reference E8 kernel")
    return h


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def cell_code(y: np.ndarray, blocks: int, inv_f: float, which=None) -> np.ndarray:
    y = np.ascontiguousarray(y, np.float32)
    n = y.shape[0]
    h = np.zeros(n, np.int64)
    fn = lib().oracle_cell_code if which is None else which.ref_cell_code
    fn(_ptr(y), C.c_int64(n), C.c_int32(blocks), C.c_float(inv_f), _ptr(h))
    return h


def e8_point(x: np.ndarray, which=None) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32).reshape(-1, 8)
    p = np.zeros_like(x)
    fn = lib().oracle_e8_point if which is None else which.ref_e8_point
    fn(_ptr(x), C.c_int64(x.shape[0]), _ptr(p))
    return p


def to_half_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    h = np.zeros(x.shape, np.uint16)
    lib().oracle_to_half(_ptr(x), C.c_int64(x.size), _ptr(h))
    return h


class Index:
    """Host arrays of an index directory bound to the checker's struct."""

    def __init__(self, arrays: dict, meta: dict):
        self.meta = meta
        a = {}
        for name, dt in (("mean", np.float32), ("proj", np.float32), ("shift", np.float32),
                         ("lists", np.int32), ("keys", np.int64), ("offsets", np.int32),
                         ("base", np.int32), ("sketch_basis", np.float32),
                         ("sketch_scale", np.float32), ("sketch", np.int8),
                         ("vectors", np.float16), ("table", np.int32)):
            if name in arrays:
                a[name] = np.ascontiguousarray(arrays[name], dtype=dt)
        a["spacings"] = np.asarray(meta["spacings"], np.float32)
        self.arrays = a
        s = OracleIndex()
        s.n, s.dim = meta["n"], meta["dim"]
        s.copies, s.blocks, s.levels = meta["copies"], meta["blocks"], len(meta["spacings"])
        s.list_len, s.log_buckets = meta["list_len"], meta["log_buckets"]
        s.sketch_width, s.table_len = meta["sketch_width"], meta.get("table_len", 0)
        s.stride, s.mmax = a["lists"].shape[1], a["keys"].shape[2]
        s.spacings, s.mean, s.proj, s.shift = map(_ptr, (a["spacings"], a["mean"], a["proj"], a["shift"]))
        s.lists, s.keys, s.offsets, s.base = map(_ptr, (a["lists"], a["keys"], a["offsets"], a["base"]))
        s.basis, s.scale, s.sketch = map(_ptr, (a["sketch_basis"], a["sketch_scale"], a["sketch"]))
        s.vectors = _ptr(a["vectors"])
        s.table = _ptr(a.get("table"))
        self.struct = s

    def search(self, queries, k=10, read=32, starts=128, waves=2, rerank=128, wave_rerank=128,
               sketch_rank=False, final_rerank=32, parts=1, threads=0, taps=(), y_in=None,
               sketch_form="product"):
        """Returns (neighbors, distances, taps dict).  ``sketch_form``: "product" evaluates the
        sketch distance in the integer form of the CUDA path (bit-comparable with it),
        "reference" as the fp32 sum of the reference's kernel."""
        q = np.ascontiguousarray(queries, np.float32)
        nq = q.shape[0]
        m = self.meta
        C_, w, L = m["copies"], 8 * m["blocks"], len(m["spacings"])
        KO = max(starts, k)
        sp = OracleParams(read, starts, waves, rerank, wave_rerank, 10000, int(sketch_rank),
                          final_rerank, parts, threads, 1 if sketch_form == "reference" else 0)
        nb = np.zeros((nq, k), np.int64)
        ds = np.zeros((nq, k), np.float32)
        out = {}
        t = OracleTaps()
        if y_in is not None:
            out["y_in"] = np.ascontiguousarray(y_in).view(np.uint16).reshape(nq, C_ * w)
            t.y_in = _ptr(out["y_in"])
        shapes = {"y": ((nq, C_ * w), np.uint16), "qs": ((nq, m["sketch_width"]), np.float32),
                  "codes": ((nq, C_, L), np.int64), "seg": ((nq, C_, 2), np.int32),
                  "kept1_ids": ((nq, KO), np.int64), "kept1_dist": ((nq, KO), np.float32),
                  "stats": ((nq, 8), np.int64)}
        for name in taps:
            if name in shapes:
                out[name] = np.zeros(*shapes[name])
                setattr(t, name, _ptr(out[name]))
        if "cand1" in taps:
            cap = C_ * min(read, m["list_len"])
            out["cand1"] = np.full((nq, cap), -1, np.int32)
            out["cand1_dist"] = np.zeros((nq, cap), np.float32)
            out["n1"] = np.zeros(nq, np.int32)
            t.cand1, t.cand1_dist, t.n1, t.cand_cap = _ptr(out["cand1"]), _ptr(out["cand1_dist"]), _ptr(out["n1"]), cap
        rc = lib().oracle_search(C.byref(self.struct), C.byref(sp), _ptr(q), C.c_int64(nq),
                                 C.c_int32(k), _ptr(nb), _ptr(ds), C.byref(t))
        if rc != 0:
            raise RuntimeError(lib().oracle_last_error().decode())
        return nb, ds, out


def brute_force(base, queries, k=10, threads=0):
    b = np.ascontiguousarray(base, np.float32)
    q = np.ascontiguousarray(queries, np.float32)
    ids = np.zeros((q.shape[0], k), np.int64)
    d = np.zeros((q.shape[0], k), np.float32)
    rc = lib().oracle_brute_force(_ptr(b), C.c_int64(b.shape[0]), C.c_int64(b.shape[1]), _ptr(q),
                                  C.c_int64(q.shape[0]), C.c_int32(k), C.c_int32(threads),
                                  _ptr(ids), _ptr(d))
    if rc != 0:
        raise RuntimeError(lib().oracle_last_error().decode())
    return ids, d


# ---- the reference's own search kernels on the GPU (oracle/_ref/libref_search.so) ----------------

class _RefSearchArgs(C.Structure):
    _fields_ = [("n", C.c_int64),
                ("dim", C.c_int32), ("copies", C.c_int32), ("blocks", C.c_int32), ("levels", C.c_int32),
                ("list_len", C.c_int32), ("log_buckets", C.c_int32), ("sketch_width", C.c_int32),
                ("table_len", C.c_int32),
                ("stride", C.c_int64), ("mmax", C.c_int64),
                ("inv_f", C.c_void_p), ("lists", C.c_void_p), ("keys", C.c_void_p),
                ("offsets", C.c_void_p), ("base", C.c_void_p), ("scale", C.c_void_p),
                ("sketch", C.c_void_p), ("vectors", C.c_void_p), ("table", C.c_void_p),
                ("m", C.c_int32), ("y", C.c_void_p), ("qs", C.c_void_p), ("q", C.c_void_p),
                ("read", C.c_int32), ("starts", C.c_int32), ("waves", C.c_int32),
                ("rerank", C.c_int32), ("wave_rerank", C.c_int32), ("k", C.c_int32),
                ("sketch_rank", C.c_int32), ("final_rerank", C.c_int32),
                ("seg", C.c_void_p), ("w1", C.c_int32), ("cand1", C.c_void_p), ("dist1", C.c_void_p),
                ("n1", C.c_void_p), ("kept1_ids", C.c_void_p), ("kept1_dist", C.c_void_p),
                ("kept_ids", C.c_void_p), ("kept_dist", C.c_void_p),
                ("best_ids", C.c_void_p), ("best_dist", C.c_void_p), ("kernel_ms", C.c_void_p),
                ("reps", C.c_int32), ("flush_mb", C.c_int32)]


def ref_search():
    """The reference's search kernels compiled as device code (needs a GPU), or None when not built."""
    p = os.path.join(_HERE, "_ref", "libref_search.so")
    return C.CDLL(p) if os.path.exists(p) else None


def ref_search_pipeline(arrays, meta, y, qs, queries, k=10, *, read=32, starts=128, waves=2,
                        rerank=128, wave_rerank=128, sketch_rank=False, final_rerank=32,
                        reps=1, flush_mb=0):
    """Run the reference's probe / gather / rerank / pick-starts kernels on this machine's GPU on a
    batch whose projected coordinates ``y`` (fp16 bits), sketch-space queries ``qs`` and queries are
    given.  The index arrays may be numpy arrays or torch tensors already on the GPU.  Returns a
    dict: seg, cand1, dist1, n1, kept1_ids, kept1_dist, kept_ids, kept_dist, best_ids, best_dist
    (the search result) and kernel_ms (device milliseconds of the first round's and of the waves'
    kernels: the median of ``reps`` runs, each stage starting after ``flush_mb`` MB were written to
    push the index out of the L2 cache when that is not 0)."""
    lib_ = ref_search()

    class _Held:  # a contiguous array or tensor with the address the C side reads
        def __init__(self, x, as_u16=False):
            if hasattr(x, "data_ptr"):
                self.x = x.contiguous()
                self.addr = self.x.data_ptr()
            else:
                self.x = np.ascontiguousarray(x)
                if as_u16:
                    self.x = self.x.view(np.uint16)
                self.addr = self.x.ctypes.data
            self.shape = tuple(self.x.shape)

    keep = {name: _Held(arrays[name], name == "vectors") for name in
            ("lists", "keys", "offsets", "base", "sketch_scale", "sketch", "vectors", "table")}
    inv_f = np.asarray([np.float32(1.0 / float(f)) for f in meta["spacings"]], np.float32)
    y = np.ascontiguousarray(y, np.uint16)
    qs = np.ascontiguousarray(qs, np.float32)
    q = np.ascontiguousarray(queries, np.float32)
    m, C_ = len(q), meta["copies"]
    KO = max(starts, k)
    w1 = 1
    while w1 < 1.5 * C_ * min(read, meta["list_len"]) or w1 < 2048:
        w1 <<= 1
    out = dict(seg=np.zeros((m, C_, 2), np.int32), cand1=np.zeros((m, w1), np.int32),
               dist1=np.zeros((m, w1), np.float32), n1=np.zeros(m, np.int32),
               kept1_ids=np.zeros((m, KO), np.int64), kept1_dist=np.zeros((m, KO), np.float32),
               kept_ids=np.zeros((m, KO), np.int64), kept_dist=np.zeros((m, KO), np.float32),
               best_ids=np.zeros((m, k), np.int64), best_dist=np.zeros((m, k), np.float32),
               kernel_ms=np.zeros(2, np.float32))
    a = _RefSearchArgs()
    a.n, a.dim, a.copies, a.blocks = meta["n"], meta["dim"], C_, meta["blocks"]
    a.levels, a.list_len, a.log_buckets = len(meta["spacings"]), meta["list_len"], meta["log_buckets"]
    a.sketch_width, a.table_len = meta["sketch_width"], meta["table_len"]
    a.stride, a.mmax = keep["lists"].shape[1], keep["keys"].shape[2]
    a.inv_f = inv_f.ctypes.data
    for field, name in (("lists", "lists"), ("keys", "keys"), ("offsets", "offsets"), ("base", "base"),
                        ("scale", "sketch_scale"), ("sketch", "sketch"), ("vectors", "vectors"),
                        ("table", "table")):
        setattr(a, field, keep[name].addr)
    a.reps, a.flush_mb = int(reps), int(flush_mb)
    a.m, a.y, a.qs, a.q = m, y.ctypes.data, qs.ctypes.data, q.ctypes.data
    a.read, a.starts, a.waves, a.rerank, a.wave_rerank, a.k = read, starts, waves, rerank, wave_rerank, k
    a.sketch_rank, a.final_rerank = int(sketch_rank), final_rerank
    a.w1 = w1
    for name, arr in out.items():
        setattr(a, name, arr.ctypes.data)
    rc = lib_.ref_search_pipeline(C.byref(a))
    if rc != 0:
        raise RuntimeError(f"the reference kernels returned {rc}")
    return out
