"""One process per GPU: connecting the processes that share an index.

The reference drives every GPU from one process (cpp/src/neighbors/octex/load.cu:241-281 of
hpdic/octex); here each GPU has its own process (``torchrun``), every process loads the index with
its ``rank`` and ``world`` (``octex_b200.load(..., rank=r, world=w)``) and ``connect`` gives the
library its NCCL communicator.  After that every process calls ``Index.search`` with the same
queries and gets all results.
"""
from __future__ import annotations

import ctypes as C

from . import _lib


def slice_rows(m: int, rank: int, world: int):
    """Rows [lo, hi) of a batch of m that process ``rank`` of ``world`` answers
    (cpp/src/neighbors/octex/search.cu:671-673)."""
    return m * rank // world, m * (rank + 1) // world


def copies_of(copies: int, rank: int, world: int):
    """Copies [c0, c1) process ``rank`` holds under shard placement (load.cu:272-275)."""
    return copies * rank // world, copies * (rank + 1) // world


def rows_of(n: int, rank: int, world: int):
    """Rows [r0, r1) of an array dealt by rows that process ``rank`` holds: ranges of
    ``ceil(n / world)`` rows (load.cu:315,406-427).  The owner of row ``i`` is ``i // rows_per``."""
    rows_per = (n + world - 1) // world
    r0 = min(n, rank * rows_per)
    return r0, min(n, r0 + rows_per)


def connect(index, group=None):
    """Create the NCCL communicator of ``index`` among the processes of ``group`` (default: all of
    torch.distributed).  Collective: every process calls it."""
    import torch.distributed as dist
    ident = [None]
    if dist.get_rank(group) == 0:
        buf = (C.c_ubyte * 128)()
        _lib.check(_lib.lib().octexB200CommUniqueId(buf))
        ident[0] = bytes(buf)
    dist.broadcast_object_list(ident, src=dist.get_global_rank(group, 0) if group is not None else 0,
                               group=group)
    raw = (C.c_ubyte * 128).from_buffer_copy(ident[0])
    _lib.check(_lib.lib().octexB200CommInit(index._h, raw))
    index._connected = True  # Index.close() is a collective from here on
    return index
