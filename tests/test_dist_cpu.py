"""Two processes on the CPU (gloo): the host-side rules of the multi-process search.

Each rank restricts the CPU checker to the copies `octex_b200.dist.copies_of` deals to it, the
ranks exchange their first-round kept lists, and each merges the row slice `slice_rows` gives it
with the rule of the reference's merge_kept_kernel (nearest copy of every id, best KO,
cpp/src/neighbors/octex/detail/search_kernels.cuh:517-564).  The result has to be the checker's own
sharded first round (`parts=2`)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def merge_rows(ids, ds, KO):
    """ids, ds [sources, KO] of one query -> best KO distinct ids by (distance bits, id)."""
    best = {}
    for i, d in zip(ids.reshape(-1), ds.reshape(-1)):
        if i < 0:
            continue
        key = (np.float32(d).view(np.uint32).item(), int(i) & 0xffffffff)
        if int(i) not in best or key < best[int(i)]:
            best[int(i)] = key
    keys = sorted(best.values())[:KO]
    out_i = np.full(KO, -1, np.int64)
    out_d = np.full(KO, np.inf, np.float32)
    for j, (bits, i) in enumerate(keys):
        out_i[j] = i
        out_d[j] = np.uint32(bits).view(np.float32)
    return out_i, out_d


def worker(rank, world, port, path, out):
    sys.path.insert(0, ROOT)
    from octex_b200 import dist as odist, index_dir
    from oracle import oracle_py
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    arrays, meta = index_dir.read_index(path, mmap=False)
    queries = np.load(os.path.join(path, "queries.npy"))
    nq = len(queries)
    kw = dict(read=8, starts=24, waves=0, rerank=48)
    KO = 24
    c0, c1 = odist.copies_of(meta["copies"], rank, world)
    mine = dict(arrays)
    for name in ("lists", "keys", "offsets", "base", "proj", "shift"):
        mine[name] = arrays[name][c0:c1]
    _, _, t = oracle_py.Index(mine, dict(meta, copies=c1 - c0)).search(
        queries, 10, taps=("kept1_ids", "kept1_dist"), **kw)
    # every rank sees every rank's kept lists (the GPU path sends only the row slices)
    all_i = [torch.zeros((nq, KO), dtype=torch.int64) for _ in range(world)]
    all_d = [torch.zeros((nq, KO), dtype=torch.float32) for _ in range(world)]
    dist.all_gather(all_i, torch.as_tensor(t["kept1_ids"]))
    dist.all_gather(all_d, torch.as_tensor(t["kept1_dist"]))
    lo, hi = odist.slice_rows(nq, rank, world)
    merged_i = np.zeros((hi - lo, KO), np.int64)
    merged_d = np.zeros((hi - lo, KO), np.float32)
    for q in range(lo, hi):
        merged_i[q - lo], merged_d[q - lo] = merge_rows(
            np.stack([a[q].numpy() for a in all_i]), np.stack([a[q].numpy() for a in all_d]), KO)
    np.savez(os.path.join(out, f"rank{rank}.npz"), ids=merged_i, dist=merged_d, lo=lo, hi=hi)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_shard_rules(small_index, oracle, tmp_path):
    from octex_b200 import dist as odist, index_dir
    arrays, meta, _, queries = small_index
    queries = queries[:61]  # an odd count: the slices differ in size
    path = str(tmp_path / "idx")
    index_dir.write_index(path, arrays, meta)
    np.save(os.path.join(path, "queries.npy"), queries)
    world = 2
    assert [odist.slice_rows(61, r, 2) for r in range(2)] == [(0, 30), (30, 61)]
    assert [odist.copies_of(8, r, 3) for r in range(3)] == [(0, 2), (2, 5), (5, 8)]
    port = 29500 + os.getpid() % 400
    mp.spawn(worker, args=(world, port, path, str(tmp_path)), nprocs=world, join=True)
    _, _, t = oracle.Index(arrays, meta).search(queries, 10, read=8, starts=24, waves=0, rerank=48,
                                                parts=world, taps=("kept1_ids", "kept1_dist"))
    for r in range(world):
        got = np.load(tmp_path / f"rank{r}.npz")
        lo, hi = int(got["lo"]), int(got["hi"])
        assert np.array_equal(got["ids"], t["kept1_ids"][lo:hi])
        assert np.array_equal(got["dist"].view(np.uint32), t["kept1_dist"][lo:hi].view(np.uint32))


def rows_worker(rank, world, port, out):
    """Every rank keeps its range of a row array; a row is fetched from the rank that owns it."""
    sys.path.insert(0, ROOT)
    from octex_b200 import dist as odist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n, width = 1003, 6
    full = np.arange(n * width, dtype=np.int64).reshape(n, width)  # what a whole array would hold
    r0, r1 = odist.rows_of(n, rank, world)
    rows_per = (n + world - 1) // world
    mine = torch.as_tensor(full[r0:r1].copy())
    pad = torch.zeros((rows_per, width), dtype=torch.int64)
    pad[: r1 - r0] = mine
    everyone = [torch.zeros_like(pad) for _ in range(world)]
    dist.all_gather(everyone, pad)  # stands for mapping the other ranks' ranges
    rng = np.random.default_rng(rank)
    ids = rng.integers(0, n, size=200)
    got = np.stack([everyone[i // rows_per][i - (i // rows_per) * rows_per].numpy() for i in ids])
    assert np.array_equal(got, full[ids])
    np.save(os.path.join(out, f"rows{rank}.npy"), np.array([r0, r1]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_rows_dealt_over_ranks(tmp_path, world):
    port = 29700 + os.getpid() % 90 + world
    mp.spawn(rows_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    spans = [np.load(tmp_path / f"rows{r}.npy") for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == 1003
    assert all(spans[r][1] == spans[r + 1][0] for r in range(world - 1))
