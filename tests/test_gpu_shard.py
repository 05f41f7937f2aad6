"""Two processes, two GPUs: shard and replicate placement through NCCL, with the row arrays whole,
dealt over the GPUs (read through mapped peer memory) or in host memory, against the CPU checker
(sharded first round: `parts=2`).  Skipped with fewer than two GPUs."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def worker(rank, world, port, path, out, placement, tiers):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import octex_b200
    from octex_b200 import dist as odist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    idx = octex_b200.load(path, devices=[rank], placement=placement, rank=rank, world=world, **tiers)
    # nothing of the other processes is reachable before the processes are connected
    try:
        idx.search(np.zeros((1, idx.dim), np.float32), 1)
        raise AssertionError("a search before the connection must fail")
    except ValueError as e:
        assert "octexB200CommInit" in str(e), e
    odist.connect(idx)
    idx.set_projection(ordered=True)  # coordinates the CPU checker reproduces bit for bit
    queries = np.load(os.path.join(path, "queries.npy"))
    res = {}
    for name, kw in (("a", dict(read=8, starts=32, waves=2, rerank=64, wave_rerank=64)),
                     ("b", dict(read=8, starts=48, waves=1, sketch_rank=True, final_rerank=32)),
                     ("c", dict(read=8, starts=32, waves=1, rerank=64, wave_rerank=64, batch=37))):
        d, i = idx.search(queries, 10, **kw)
        res[name + "_i"], res[name + "_d"] = i, d
    # device arrays in and out as well
    q = torch.as_tensor(queries, device="cuda")
    d, i = idx.search(q, 10, read=8, starts=32, waves=2, rerank=64, wave_rerank=64)
    res["dev_i"], res["dev_d"] = i.cpu().numpy(), d.cpu().numpy()
    np.savez(os.path.join(out, f"{placement}{rank}.npz"), **res)
    rep = idx.memory_report()
    assert rep["device"] == rank and rep["copies"] > 0 and rep["buffers"] > 0
    # closing is a collective: a process that arrives late still finds its peers' memory mapped,
    # and the early one does not free what the late one has mapped
    if rank == 1:
        import time
        time.sleep(1.0)
    idx.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("placement,tiers", [
    ("shard", {}),                                                # table dealt by rows (always, as the reference)
    ("replicate", {}),
    ("shard", dict(shard_vectors=True, sketch="shard")),          # every row array dealt over the two GPUs
    ("replicate", dict(shard_vectors=True, sketch="shard")),
    ("shard", dict(vectors_on_host=True, table_on_host=True)),    # host tiers with dealt copies
])
def test_two_processes(wide_index, oracle, tmp_path, placement, tiers):
    import torch
    import torch.multiprocessing as mp
    from octex_b200 import index_dir
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    arrays, meta, _, queries = wide_index
    queries = queries[:151]
    path = str(tmp_path / "idx")
    index_dir.write_index(path, arrays, meta)
    np.save(os.path.join(path, "queries.npy"), queries)
    port = 29900 + os.getpid() % 90
    mp.spawn(worker, args=(2, port, path, str(tmp_path), placement, tiers), nprocs=2, join=True)
    ox = oracle.Index(arrays, meta)
    parts = 2 if placement == "shard" else 1
    want = {
        "a": ox.search(queries, 10, read=8, starts=32, waves=2, rerank=64, wave_rerank=64, parts=parts),
        "b": ox.search(queries, 10, read=8, starts=48, waves=1, sketch_rank=True, final_rerank=32, parts=parts),
        "c": ox.search(queries, 10, read=8, starts=32, waves=1, rerank=64, wave_rerank=64, parts=parts),
    }
    want["dev"] = want["a"]
    for r in range(2):
        got = np.load(tmp_path / f"{placement}{r}.npz")
        for name, (ids, dist_, _) in want.items():
            assert np.array_equal(got[name + "_i"], ids), (placement, r, name)
            assert np.array_equal(got[name + "_d"].view(np.uint32), dist_.view(np.uint32)), (placement, r, name)
