"""Reader and writer of the on-disk index directory (format 1).

Layout as the reference documents it (docs/design.md:27-48 of hpdic/octex; writer
cpp/src/neighbors/octex/build.cu:215-349, reader cpp/src/neighbors/octex/load.cu:215-313):
``meta.json`` plus one ``.npy`` (version 1.0, little-endian, C order) per array.  The native
loader of this package reads the same directory; this module is the Python side used by the
index builder and by tests.
"""
from __future__ import annotations

import json
import os

import numpy as np

#: array name -> dtype of a complete directory
ARRAYS = {
    "mean": np.float32, "proj": np.float32, "shift": np.float32, "lists": np.int32,
    "keys": np.int64, "offsets": np.int32, "base": np.int32, "cells": np.int64,
    "sketch_basis": np.float32, "sketch_scale": np.float32, "sketch": np.int8,
    "table": np.int32, "vectors": np.float16,
}

META_KEYS = ("format", "n", "dim", "copies", "blocks", "spacings", "list_len", "log_buckets",
             "sketch_width", "table_len", "metric")


def write_index(path: str, arrays: dict, meta: dict) -> None:
    """Write ``arrays`` (name -> ndarray) and ``meta`` to ``path``; meta.json goes last, a
    directory without it is incomplete (build.cu:423-424)."""
    os.makedirs(path, exist_ok=True)
    for name, arr in arrays.items():
        want = ARRAYS.get(name)
        a = np.ascontiguousarray(arr if want is None else np.asarray(arr, dtype=want))
        np.save(os.path.join(path, name + ".npy"), a, allow_pickle=False)
    full = {"format": 1, "metric": "sqeuclidean"}
    full.update(meta)
    full.setdefault("files", {name: name + ".npy" for name in arrays})
    with open(os.path.join(path, "meta.json"), "w") as f:
        json.dump(full, f, indent=1)


def read_meta(path: str) -> dict:
    with open(os.path.join(path, "meta.json")) as f:
        return json.load(f)


def read_index(path: str, mmap: bool = True):
    """(arrays, meta) of an index directory; arrays are memory-mapped unless ``mmap`` is False."""
    meta = read_meta(path)
    files = meta.get("files", {})
    arrays = {}
    for name in ARRAYS:
        rel = files.get(name, name + ".npy")
        p = rel if os.path.isabs(rel) else os.path.join(path, rel)
        if not os.path.exists(p):
            continue
        arrays[name] = np.load(p, mmap_mode="r" if mmap else None, allow_pickle=False)
    return arrays, meta
