"""Index builder (tooling): dataset -> format-1 index arrays / directory.

The search path of this package reads an index; this module makes one so that tests and the
benchmark have something to read.  It restates the reference's build pipeline with torch
tensor ops (CPU or CUDA device), following

* sample PCA and seeded projections: cpp/src/neighbors/octex/detail/build_setup.cuh:40-175
* cells per copy and spacing (hash, unique, ``min_cell`` filter, centres), lists from the
  members of each cell, (bucket, hash) order and CSR offsets:
  cpp/src/neighbors/octex/detail/build_cells.cuh:62-127,134-253,384-449,519-605
* int8 sketch: build_setup.cuh:177-264
* exact neighbor table with reverse edges merged in: build_table.cuh:60-74,171-251,529-554

Deviations, all on the build side (the search reads whatever directory it is given):
projections are drawn from ``numpy.random.default_rng((seed, copy))`` rather than the
reference's ``std::mt19937_64`` stream; lists are always "member lists" (the reference's
``member_lists=true`` mode) because its default list construction needs the cuVS IVF-Flat
library.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass, field

import numpy as np
import torch

from . import index_dir

_PRIMES = [1000003, 998244353, 1000000007, 2147483647, 1099511627791, 4398042316799,
           70368744177643, 1125899906842597]
_MIX = 0x9E3779B97F4A7C15 - (1 << 64)  # the 64-bit mixer as a signed value
_SAMPLE_ROWS = 200_000


@dataclass
class IndexParams:
    """Build parameters; names and defaults of ``index_params``
    (cpp/include/cuvs/neighbors/octex.hpp:32-92) except ``min_cell``/``log_buckets`` which
    callers of this tooling usually override for small data."""
    copies: int = 200
    blocks: int = 4
    pca_dims: int = 64
    spacings: list = field(default_factory=lambda: [2.0, 2.5, 3.2, 4.0, 5.0])
    list_len: int = 64
    min_cell: int = 1
    log_buckets: int = 20
    sketch_width: int = 0
    table_len: int = 64
    reverse_edges: bool = True
    seed: int = 0


def _nearest_d8(v: torch.Tensor) -> torch.Tensor:
    f = torch.round(v)
    e = v - f
    at = e.abs().argmax(-1, keepdim=True)  # first index of the largest |error|
    e_at = e.gather(-1, at)
    odd = (torch.remainder(f.sum(-1, keepdim=True), 2.0) != 0).to(v.dtype)
    step = torch.where(e_at >= 0, torch.ones_like(e_at), -torch.ones_like(e_at)) * odd
    return f.scatter_add(-1, at, step)


def e8_nearest(x: torch.Tensor) -> torch.Tensor:
    """Nearest point of E8 = D8 u (D8 + 1/2) to every row of ``x`` [..., 8] (e8.cuh:45-63)."""
    a = _nearest_d8(x)
    c = _nearest_d8(x - 0.5) + 0.5
    da = ((x - a) ** 2).sum(-1, keepdim=True)
    dc = ((x - c) ** 2).sum(-1, keepdim=True)
    return torch.where(da <= dc, a, c)


def cell_codes(x: torch.Tensor, blocks: int) -> torch.Tensor:
    """64-bit cell code of every row of ``x`` [n, 8*blocks] (already divided by the spacing),
    e8.cuh:66-85."""
    n = x.shape[0]
    p = e8_nearest(x.reshape(n, blocks, 8))
    twice = (2.0 * p).to(torch.int64)
    primes = torch.tensor(_PRIMES, dtype=torch.int64, device=x.device)
    hb = (twice * primes).sum(-1)
    h = hb[:, 0]
    for j in range(1, blocks):
        h = h * _MIX + hb[:, j]
    h = (h ^ (h >> 31)) * _MIX
    return h ^ (h >> 29)


def sample_pca(x16: torch.Tensor):
    """Mean, eigenvalues (descending, of the unnormalised scatter) and eigenvectors of a strided
    sample of at most 200 000 rows, in float64 (build_setup.cuh:40-103)."""
    n = x16.shape[0]
    step = max(1, n // _SAMPLE_ROWS)
    s = x16[::step].to(torch.float64).cpu()
    mean = s.mean(0)
    a = s - mean.to(torch.float32).to(torch.float64)
    vals, vecs = torch.linalg.eigh(a.T @ a)
    order = torch.arange(vals.numel() - 1, -1, -1)
    return mean.to(torch.float32), vals[order].clamp_min(0), vecs[:, order], s.shape[0]


def make_projections(vals, vecs, ns, dim, p, w, copies, seed):
    """proj [C, dim, w], shift [C, w]: each copy rotates the top-p principal subspace into w
    dimensions by an orthonormal random [p, w] matrix and divides by the mean projected
    standard deviation; shifts are uniform in [0, 2) (build_setup.cuh:113-175)."""
    if p < w:
        raise ValueError("octex: pca_dims must be at least 8 * blocks")
    if p > dim:
        raise ValueError("octex: pca_dims exceeds the dimension")
    proj = np.empty((copies, dim, w), np.float32)
    shift = np.empty((copies, w), np.float32)
    lam = vals[:p].numpy()
    top = vecs[:, :p].numpy()
    for c in range(copies):
        rng = np.random.default_rng((seed, c))
        q, _ = np.linalg.qr(rng.standard_normal((p, w)))
        sd = np.sqrt((lam[:, None] * q * q).sum(0) / max(ns - 1, 1)).mean()
        proj[c] = (top @ q / sd).astype(np.float32)
        shift[c] = rng.uniform(0.0, 2.0, size=w).astype(np.float32)
    return proj, shift


def _copy_cells(y, params: IndexParams):
    """Lists, keys, offsets, base, cells of one copy from its projected rows y [n, w] fp32."""
    dev = y.device
    n, w = y.shape
    b, l = params.blocks, params.list_len
    T = 1 << params.log_buckets
    L = len(params.spacings)
    lists_all, keys_all, offs_all, base, cells = [], [], [], [], []
    row = 0
    for j, f in enumerate(params.spacings):
        codes = cell_codes(y / f, b)
        hs, order = torch.sort(codes, stable=True)
        ukeys, pop = torch.unique_consecutive(hs, return_counts=True)
        start = torch.cumsum(pop, 0) - pop
        keep = pop >= params.min_cell if (params.min_cell > 1 and j < L - 1) else torch.ones_like(pop, dtype=torch.bool)
        first = order[start[keep]]
        M = int(first.numel())
        z = f * e8_nearest((y[first] / f).reshape(M, b, 8)).reshape(M, w)
        # members of the kept cells, nearest to the centre first
        kept_index = torch.cumsum(keep.to(torch.int64), 0) - 1
        cell_of_pos = torch.repeat_interleave(torch.arange(pop.numel(), device=dev), pop)
        pos = torch.nonzero(keep[cell_of_pos]).squeeze(1)
        cidx = kept_index[cell_of_pos[pos]]
        ids = order[pos]
        d = ((y[ids] - z[cidx]) ** 2).sum(-1)
        by_d = torch.argsort(d, stable=True)
        by_cell = torch.argsort(cidx[by_d], stable=True)
        perm = by_d[by_cell]
        cidx, ids = cidx[perm], ids[perm]
        kpop = pop[keep]
        kstart = torch.cumsum(kpop, 0) - kpop
        rank = torch.arange(ids.numel(), device=dev) - kstart[cidx]
        sel = rank < l
        lists = torch.full((M, l), -1, dtype=torch.int32, device=dev)
        lists[cidx[sel], rank[sel]] = ids[sel].to(torch.int32)
        lists = torch.where(lists < 0, lists[:, :1].expand(-1, l), lists)  # repeat the nearest
        # (bucket, hash) order and CSR offsets over the buckets
        keys = ukeys[keep]
        bucket = keys & (T - 1)
        sb, bperm = torch.sort(bucket, stable=True)
        offs = torch.searchsorted(sb, torch.arange(T + 1, device=dev, dtype=sb.dtype))
        lists_all.append(lists[bperm])
        keys_all.append(keys[bperm])
        offs_all.append(offs.to(torch.int32))
        base.append(row)
        cells.append(M)
        row += M
    return lists_all, keys_all, offs_all, base, cells


def exact_table(x16: torch.Tensor, k: int, reverse: bool, chunk: int = 4096) -> torch.Tensor:
    """Neighbor table [n, k] int32: exact k nearest rows (self dropped), then the reverse-edge
    merge by the half rule: first k/2 forward, up to k/2 nearest reverse edges whose source lists
    the row among its first k/2, then the remaining forward ones; duplicates dropped, first k
    kept, ordered nearest first (build_table.cuh:171-251,529-554)."""
    dev = x16.device
    n, _ = x16.shape
    xf = x16.to(torch.float32)
    sq = (xf * xf).sum(1)
    ids = torch.empty((n, k), dtype=torch.int64, device=dev)
    dist = torch.empty((n, k), dtype=torch.float32, device=dev)
    for r0 in range(0, n, chunk):
        q = xf[r0:r0 + chunk]
        d = sq[r0:r0 + chunk, None] - 2.0 * (q @ xf.T) + sq[None, :]
        d[torch.arange(q.shape[0], device=dev), torch.arange(r0, r0 + q.shape[0], device=dev)] = float("inf")
        dd, ii = torch.topk(d, k, dim=1, largest=False, sorted=True)
        ids[r0:r0 + chunk] = ii
        dist[r0:r0 + chunk] = dd.clamp_min(0)
    if not reverse:
        return ids.to(torch.int32)
    h = max(1, k // 2)
    # reverse edges v -> u for u among the first h neighbors of v, nearest h per target
    src = torch.arange(n, device=dev).repeat_interleave(h)
    dst = ids[:, :h].reshape(-1)
    dd = dist[:, :h].reshape(-1)
    by_d = torch.argsort(dd, stable=True)
    by_dst = torch.argsort(dst[by_d], stable=True)
    perm = by_d[by_dst]
    src, dst, dd = src[perm], dst[perm], dd[perm]
    cnt = torch.bincount(dst, minlength=n)
    startp = torch.cumsum(cnt, 0) - cnt
    rank = torch.arange(dst.numel(), device=dev) - startp[dst]
    sel = rank < h
    rev = torch.full((n, h), -1, dtype=torch.int64, device=dev)
    rdist = torch.zeros((n, h), dtype=torch.float32, device=dev)
    rev[dst[sel], rank[sel]] = src[sel]
    rdist[dst[sel], rank[sel]] = dd[sel]
    cand = torch.cat([ids[:, :h], rev, ids[:, h:]], 1)          # priority order
    cdist = torch.cat([dist[:, :h], rdist, dist[:, h:]], 1)
    p = cand.shape[1]
    out = torch.empty((n, k), dtype=torch.int32, device=dev)
    big = torch.iinfo(torch.int64).max
    for r0 in range(0, n, 1 << 16):
        c = cand[r0:r0 + (1 << 16)]
        cd = cdist[r0:r0 + (1 << 16)]
        m = c.shape[0]
        slot = torch.arange(p, device=dev).expand(m, p)
        # keep the first slot of every id
        key = torch.where(c >= 0, c * p + slot, torch.full_like(c, big))
        skey, sidx = torch.sort(key, dim=1)
        sid = torch.where(skey == big, torch.full_like(skey, -1), skey // p)
        dup = torch.zeros_like(sid, dtype=torch.bool)
        dup[:, 1:] = (sid[:, 1:] == sid[:, :-1]) & (sid[:, 1:] >= 0)
        valid = (sid >= 0) & ~dup
        vslot = torch.where(valid, sidx, torch.full_like(sidx, p))
        # first k by priority among the valid ones
        order = torch.argsort(vslot, dim=1, stable=True)[:, :k]
        pick_slot = vslot.gather(1, order)
        ok = pick_slot < p
        pick_slot = pick_slot.clamp_max(p - 1)
        pid = torch.where(ok, c.gather(1, pick_slot), torch.full_like(pick_slot, -1))
        pdist = torch.where(ok, cd.gather(1, pick_slot), torch.full_like(cd[:, :k], float("inf")))
        # nearest first, then id
        o2 = torch.argsort(pid, dim=1, stable=True)
        o3 = torch.argsort(pdist.gather(1, o2), dim=1, stable=True)
        fin = o2.gather(1, o3)
        res = pid.gather(1, fin)
        out[r0:r0 + m] = res.to(torch.int32)
    return out


def make_sketch(x16, mean, basis, chunk: int = 1 << 18):
    """int8 codes = round(((x - mean) @ basis) / scale) clipped to +-127, scale = amax / 127
    per coordinate over the dataset (build_setup.cuh:177-264)."""
    dev = x16.device
    n = x16.shape[0]
    S = basis.shape[1]
    amax = torch.zeros(S, device=dev)
    for r0 in range(0, n, chunk):
        v = (x16[r0:r0 + chunk].to(torch.float32) - mean) @ basis
        amax = torch.maximum(amax, v.abs().amax(0))
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    codes = torch.empty((n, S), dtype=torch.int8, device=dev)
    for r0 in range(0, n, chunk):
        v = (x16[r0:r0 + chunk].to(torch.float32) - mean) @ basis
        codes[r0:r0 + chunk] = torch.round(v / scale).clamp(-127, 127).to(torch.int8)
    return scale, codes


def auto_sketch_width(dim: int) -> int:
    """build.cu:118-121: the dimension rounded down to a multiple of 16, at most 128."""
    return max(min(dim // 16 * 16, 128), min(dim, 16))


def build_arrays(dataset, params: IndexParams, device: str | torch.device = "cpu",
                 keep_on_device: bool = False, verbose: bool = False):
    """Build every array of an index.  Returns (arrays, meta); arrays are numpy unless
    ``keep_on_device`` (then torch tensors on ``device``, for indexes that should never touch
    the host)."""
    dev = torch.device(device)
    prev_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        src = dataset.detach() if torch.is_tensor(dataset) else torch.as_tensor(np.asarray(dataset))
        x16 = src.to(dev).to(torch.float16)
        n, dim = x16.shape
        if dim % 2:
            raise ValueError("octex: the dimension must be even")
        w = 8 * params.blocks
        L = len(params.spacings)
        S = min(params.sketch_width, dim) if params.sketch_width > 0 else auto_sketch_width(dim)
        mean, vals, vecs, ns = sample_pca(x16)
        p = min(params.pca_dims, dim)
        proj, shift = make_projections(vals, vecs, ns, dim, p, w, params.copies, params.seed)
        mean_d = mean.to(dev)
        per_copy = []
        xc = None
        if n * dim * 4 <= (8 << 30):
            xc = x16.to(torch.float32) - mean_d
        for c in range(params.copies):
            u = torch.as_tensor(proj[c], device=dev)
            sh = torch.as_tensor(shift[c], device=dev)
            if xc is not None:
                y = xc @ u + sh
            else:
                y = torch.cat([(x16[r0:r0 + (1 << 18)].to(torch.float32) - mean_d) @ u
                               for r0 in range(0, n, 1 << 18)]) + sh
            per_copy.append(_copy_cells(y, params))
            if verbose and (c % 10 == 0 or c == params.copies - 1):
                print(f"  copy {c}: cells per level {per_copy[-1][4]}", file=sys.stderr, flush=True)
        del xc
        rows = [sum(pc[4]) for pc in per_copy]
        Lmax = max(rows) * params.list_len
        Mmax = max(max(pc[4]) for pc in per_copy)
        T1 = (1 << params.log_buckets) + 1
        C = params.copies
        lists = torch.zeros((C, Lmax), dtype=torch.int32, device=dev)
        keys = torch.zeros((C, L, Mmax), dtype=torch.int64, device=dev)
        offsets = torch.empty((C, L, T1), dtype=torch.int32, device=dev)
        base = torch.zeros((C, L), dtype=torch.int32)
        cells = torch.zeros((C, L), dtype=torch.int64)
        for c, (ls, ks, os_, bs, cs) in enumerate(per_copy):
            flat = torch.cat([x.reshape(-1) for x in ls])
            lists[c, :flat.numel()] = flat
            for j in range(L):
                keys[c, j, :cs[j]] = ks[j]
                offsets[c, j] = os_[j]
                base[c, j] = bs[j]
                cells[c, j] = cs[j]
            per_copy[c] = None
        basis = vecs[:, :S].to(torch.float32).to(dev).contiguous()
        scale, codes = make_sketch(x16, mean_d, basis)
        arrays = {
            "mean": mean_d, "proj": torch.as_tensor(proj), "shift": torch.as_tensor(shift),
            "lists": lists, "keys": keys, "offsets": offsets, "base": base, "cells": cells,
            "sketch_basis": basis, "sketch_scale": scale, "sketch": codes, "vectors": x16,
        }
        if params.table_len > 0:
            if not 1 <= params.table_len < n:
                raise ValueError("octex: table_len must be in [1, n)")
            arrays["table"] = exact_table(x16, params.table_len, params.reverse_edges)
        meta = {
            "format": 1, "n": int(n), "dim": int(dim), "copies": C, "blocks": params.blocks,
            "spacings": [float(f) for f in params.spacings], "list_len": params.list_len,
            "log_buckets": params.log_buckets, "sketch_width": int(S),
            "table_len": params.table_len, "metric": "sqeuclidean",
        }
        if keep_on_device:
            arrays = {k_: v.to(dev) for k_, v in arrays.items()}
        else:
            arrays = {k_: v.cpu().numpy() for k_, v in arrays.items()}
        return arrays, meta
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev_tf32


def build(dataset, path: str, params: IndexParams | None = None, device="cpu", verbose=False):
    """Build an index of ``dataset`` [n, dim] and write it to the directory ``path``."""
    arrays, meta = build_arrays(dataset, params or IndexParams(), device=device, verbose=verbose)
    index_dir.write_index(path, arrays, meta)
    return meta
