"""Index directory format and the builder tooling: shapes, CSR consistency, the (bucket, code)
order of the keys, and a write/read round trip (the checks of the reference's
cpp/tests/test_build.cu:180-300 that concern what the search reads)."""
import json
import os

import numpy as np
import torch

from octex_b200 import build_index, index_dir


def test_builder_arrays_are_consistent(small_index):
    arrays, meta, base, _ = small_index
    C, L, l = meta["copies"], len(meta["spacings"]), meta["list_len"]
    T = 1 << meta["log_buckets"]
    n = meta["n"]
    assert arrays["proj"].shape == (C, meta["dim"], 8 * meta["blocks"])
    assert arrays["offsets"].shape == (C, L, T + 1)
    assert arrays["vectors"].dtype == np.float16 and arrays["sketch"].dtype == np.int8
    assert arrays["table"].shape == (n, meta["table_len"])
    for c in range(C):
        row = 0
        for j in range(L):
            M = int(arrays["cells"][c, j])
            assert int(arrays["base"][c, j]) == row
            off = arrays["offsets"][c, j]
            assert off[0] == 0 and off[-1] == M and (np.diff(off) >= 0).all()
            keys = arrays["keys"][c, j, :M]
            buckets = keys & (T - 1)
            assert (np.diff(buckets) >= 0).all(), "bucket order"
            same = np.diff(buckets) == 0
            assert (np.diff(keys)[same] > 0).all(), "codes ascending inside a bucket, distinct"
            # every key sits in the bucket its CSR bounds say
            assert (np.searchsorted(off, np.arange(M), side="right") - 1 == buckets).all()
            row += M
        rows = arrays["lists"][c, :row * l].reshape(row, l)
        assert rows.min() >= 0 and rows.max() < n
    t = arrays["table"]
    assert t.max() < n and (t[t >= 0] != np.repeat(np.arange(n), (t >= 0).sum(1))).all(), "no self edge"


def test_cells_hold_their_members(small_index):
    """A vector of the dataset hashes, at the coarsest level, to a cell that exists, and the first
    list entry of that cell lies in the same cell."""
    arrays, meta, base, _ = small_index
    b, f = meta["blocks"], meta["spacings"][-1]
    j = len(meta["spacings"]) - 1
    T = 1 << meta["log_buckets"]
    x = torch.as_tensor(arrays["vectors"][:500].astype(np.float32) - arrays["mean"])
    for c in (0, meta["copies"] - 1):
        y = x @ torch.as_tensor(arrays["proj"][c]) + torch.as_tensor(arrays["shift"][c])
        codes = build_index.cell_codes(y / f, b).numpy()
        off, keys = arrays["offsets"][c, j], arrays["keys"][c, j]
        for h in codes[:100]:
            bk = int(h) & (T - 1)
            assert int(h) in keys[off[bk]:off[bk + 1]].tolist()


def test_write_read_round_trip(small_index, tmp_path):
    arrays, meta, _, _ = small_index
    path = tmp_path / "idx"
    index_dir.write_index(str(path), arrays, meta)
    m = json.load(open(path / "meta.json"))
    for key in index_dir.META_KEYS:
        assert key in m, key
    assert m["format"] == 1 and m["metric"] == "sqeuclidean"
    back, meta2 = index_dir.read_index(str(path))
    assert meta2["n"] == meta["n"]
    for name, a in arrays.items():
        assert np.array_equal(back[name], a), name
        assert back[name].dtype == index_dir.ARRAYS[name]
    with open(path / "lists.npy", "rb") as f:
        assert f.read(8) == b"\x93NUMPY\x01\x00", ".npy version 1.0"


def test_auto_sketch_width():
    assert [build_index.auto_sketch_width(d) for d in (8, 48, 96, 128, 960)] == [8, 48, 96, 128, 128]
