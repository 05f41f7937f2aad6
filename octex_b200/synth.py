"""Seeded synthetic datasets standing in for the public sets the reference is measured on.

The reference quotes its numbers on SIFT1M, GIST1M, Deep10M and Deep1B (README.md:23-31 of
hpdic/octex); none of those files can be used here, so each generator below draws vectors with
the shape, value range and rough cluster structure of one of them from a seeded
``numpy.random.Generator``.  Nothing here is copied from any dataset.

Every generator returns ``float32`` rows; ``chunk`` keeps peak memory bounded for the large ones.
"""
from __future__ import annotations

import numpy as np

__all__ = ["plumbing", "descriptor_like", "global_descriptor_like", "embedding_like", "CONFIGS",
           "make"]


def plumbing(n: int, dim: int = 128, seed: int = 0, centers_seed: int = 1234) -> np.ndarray:
    """64-component Gaussian mixture: centres ~ N(0, 4 I), per-point noise ~ N(0, I).

    Same family as the reference's own ``clustered()`` test fixture (tests/conftest.py:55-63).
    """
    centers = np.random.default_rng(centers_seed).normal(0.0, 2.0, size=(64, dim))
    rng = np.random.default_rng(seed)
    which = rng.integers(0, 64, size=n)
    out = centers[which] + rng.normal(0.0, 1.0, size=(n, dim))
    return out.astype(np.float32)


def descriptor_like(n: int, dim: int = 128, seed: int = 0, centers_seed: int = 4321,
                    chunk: int = 1 << 18) -> np.ndarray:
    """Non-negative integer-valued local-descriptor-like rows (values 0..255).

    Each coordinate is ``round(clip(|N(0,1)| * 40 + offset, 0, 255))`` where the offset comes
    from one of 1 024 cluster centres drawn uniformly in [0, 120].
    """
    centers = np.random.default_rng(centers_seed).uniform(0.0, 120.0, size=(1024, dim))
    rng = np.random.default_rng(seed)
    out = np.empty((n, dim), np.float32)
    for r0 in range(0, n, chunk):
        m = min(chunk, n - r0)
        which = rng.integers(0, 1024, size=m)
        v = np.abs(rng.standard_normal(size=(m, dim), dtype=np.float32)) * 40.0
        v += centers[which].astype(np.float32)
        out[r0:r0 + m] = np.rint(np.clip(v, 0.0, 255.0))
    return out


def global_descriptor_like(n: int, dim: int = 960, seed: int = 0, centers_seed: int = 999,
                           chunk: int = 1 << 16) -> np.ndarray:
    """Non-negative global-descriptor-like rows: 256-centre mixture, centres |N(0,1)|*0.1,
    per-point noise |N(0, 0.02^2)| added."""
    centers = (np.abs(np.random.default_rng(centers_seed).standard_normal((256, dim))) * 0.1)
    centers = centers.astype(np.float32)
    rng = np.random.default_rng(seed)
    out = np.empty((n, dim), np.float32)
    for r0 in range(0, n, chunk):
        m = min(chunk, n - r0)
        which = rng.integers(0, 256, size=m)
        noise = np.abs(rng.standard_normal(size=(m, dim), dtype=np.float32)) * np.float32(0.02)
        out[r0:r0 + m] = centers[which] + noise
    return out


def _anisotropic_matrix(dim: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    a, _ = np.linalg.qr(rng.standard_normal((dim, dim)))
    b, _ = np.linalg.qr(rng.standard_normal((dim, dim)))
    sv = 1.0 / np.sqrt(np.arange(1, dim + 1, dtype=np.float64))
    return ((a * sv) @ b.T).astype(np.float32)


def embedding_like(n: int, dim: int = 96, seed: int = 0, matrix_seed: int = 77,
                   chunk: int = 1 << 20) -> np.ndarray:
    """Anisotropic unit-norm embedding-like rows: z ~ N(0, I) times a fixed random matrix with
    singular values 1/sqrt(i), then L2-normalised."""
    mat = _anisotropic_matrix(dim, matrix_seed)
    rng = np.random.default_rng(seed)
    out = np.empty((n, dim), np.float32)
    for r0 in range(0, n, chunk):
        m = min(chunk, n - r0)
        z = rng.standard_normal(size=(m, dim), dtype=np.float32) @ mat
        z /= np.linalg.norm(z, axis=1, keepdims=True)
        out[r0:r0 + m] = z
    return out


#: name -> (generator, dim, base rows, query rows) of the five benchmark configurations
CONFIGS = {
    "plumbing-100k": (plumbing, 128, 100_000, 1_000),
    "descriptor-1m": (descriptor_like, 128, 1_000_000, 10_000),
    "global-1m": (global_descriptor_like, 960, 1_000_000, 1_000),
    "embedding-10m": (embedding_like, 96, 10_000_000, 10_000),
    "embedding-1b": (embedding_like, 96, 1_000_000_000, 10_000),
}


def make(name: str, n: int | None = None, nq: int | None = None, base_seed: int = 0,
         query_seed: int = 1):
    """(base rows, query rows) of a named configuration; ``n`` / ``nq`` shrink it for tests."""
    gen, dim, n0, q0 = CONFIGS[name]
    return gen(n or n0, dim, seed=base_seed), gen(nq or q0, dim, seed=query_seed)
