"""Seeded synthetic corpora with the shapes of the reference's training inputs.

The reference is trained on ``encodings.npy`` (int32 token ids) and
``offsets.npy`` (uint64 chunk boundaries, first entry 0, last entry = number of
tokens; flyvec/train_flyvec.py:155-176).  No corpus ships with it, so the
benchmarks and parity tests draw one: token ids follow a bounded Zipf law over
the vocabulary and chunk lengths are geometric above a minimum.
"""
from __future__ import annotations

import numpy as np


def zipf_ids(n: int, vocab: int, s: float, rng: np.random.Generator, lo: int = 0) -> np.ndarray:
    """``n`` ids in ``[lo, vocab)`` with ``P(rank r) ~ r**-s`` (rank 1 = id ``lo``).

    Inverse-CDF sampling on the cumulative weights (numpy's own ``zipf`` needs
    ``s > 1`` and is unbounded)."""
    ranks = np.arange(1, vocab - lo + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** (-s))
    cdf /= cdf[-1]
    out = np.empty(n, dtype=np.int32)
    CH = 1 << 24
    for a in range(0, n, CH):
        u = rng.random(min(CH, n - a))
        out[a:a + len(u)] = (np.searchsorted(cdf, u, side="right") + lo).astype(np.int32)
    np.minimum(out, vocab - 1, out=out)
    return out


def chunk_offsets(ntok: int, mean_len: float, min_len: int, rng: np.random.Generator) -> np.ndarray:
    """uint64 boundaries ``[0, ..., ntok]`` of chunks with length
    ``min_len + Geometric - 1`` and the given mean; the last chunk is whatever
    remains."""
    p = 1.0 / max(mean_len - min_len + 1.0, 1.0)
    est = int(ntok / mean_len * 1.1) + 16
    lens = []
    total = 0
    while total < ntok:
        part = (min_len + rng.geometric(p, est) - 1).astype(np.int64)
        lens.append(part)
        total += int(part.sum())
    lens = np.concatenate(lens)
    ends = np.cumsum(lens)
    ncut = int(np.searchsorted(ends, ntok, side="left"))
    bounds = np.concatenate(([0], ends[:ncut], [ntok])).astype(np.uint64)
    return np.unique(bounds)


def make_corpus(ntok: int, vocab: int, s: float = 1.0, mean_len: float = 25.0, min_len: int = 11,
                seed: int = 101):
    """``(encodings int32[ntok], offsets uint64[C+1])``; id ``vocab-1`` is forced to
    occur so that ``max(encodings)+1 == vocab`` (flyvec/train_flyvec.py:168)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    enc = zipf_ids(ntok, vocab, s, rng)
    enc[int(rng.integers(0, ntok))] = vocab - 1
    off = chunk_offsets(ntok, mean_len, min_len, rng)
    return enc, off


def make_weights(K: int, N: int, seed: int = 1, mu: float = 0.0, sigma: float = 1.0) -> np.ndarray:
    """Initial synapses ``float32[K][N] ~ N(mu, sigma)`` (flyvec/train_flyvec.py:240)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    return (mu + sigma * rng.standard_normal((K, N))).astype(np.float32)


def make_hash_ids(n: int, vocab: int, s: float = 1.0, unk_frac: float = 0.01, seed: int = 100) -> np.ndarray:
    """Token ids for the hashing benchmark: Zipf over ``1..vocab-1`` with a
    fraction forced to id 0 (the unknown token, flyvec/core.py:130-137)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    ids = zipf_ids(n, vocab, s, rng, lo=1)
    ids[rng.random(n) < unk_frac] = 0
    return ids
