"""Token batchers, restated.  Test infrastructure only.

FifoU16 follows src/data/loader.zig:555-589 (U16TokenDatasetFifo.getBatchImpl) exactly: each call
consumes B*T+1 tokens at the cursor; inputs are window[0:B*T], targets window[1:B*T+1], both widened
to i64 and shaped [B, T]; the cursor then moves by B*T+1.  Errors keep the reference's names.

RandomU16 follows src/data/loader.zig:457-486 in structure (one uniformly drawn window start per row,
start in [0, len-T-1]); the reference draws from Zig 0.13's std.Random.DefaultPrng, which is not part
of the reference tree, so the start positions here come from a caller-supplied generator and are
UNPINNED against the reference.
"""
from __future__ import annotations

import numpy as np


class ChunkTooSmall(Exception):
    pass


class ChunkExhausted(Exception):
    pass


class FifoU16:
    def __init__(self, tokens):
        self.tokens = np.ascontiguousarray(tokens, dtype=np.uint16)
        self.cursor = 0

    def get_batch(self, batch_size: int, block_size: int):
        needed = batch_size * block_size + 1
        if self.tokens.size < needed:
            raise ChunkTooSmall()
        if self.cursor + needed > self.tokens.size:
            raise ChunkExhausted()
        w = self.tokens[self.cursor:self.cursor + needed].astype(np.int64)
        self.cursor += needed
        x = w[:-1].reshape(batch_size, block_size).copy()
        y = w[1:].reshape(batch_size, block_size).copy()
        return x, y


class RandomU16:
    def __init__(self, tokens, rng: np.random.Generator):
        self.tokens = np.ascontiguousarray(tokens, dtype=np.uint16)
        self.rng = rng

    def get_batch(self, batch_size: int, block_size: int):
        if self.tokens.size < block_size + 1:
            raise ChunkTooSmall()
        hi = self.tokens.size - block_size - 1
        x = np.empty((batch_size, block_size), np.int64)
        y = np.empty((batch_size, block_size), np.int64)
        for i in range(batch_size):
            s = int(self.rng.integers(0, hi + 1))
            x[i] = self.tokens[s:s + block_size]
            y[i] = self.tokens[s + 1:s + block_size + 1]
        return x, y


def zipf_tokens(n: int, vocab: int, s: float, seed: int) -> np.ndarray:
    """Seeded synthetic token stream: rank r in [1, vocab] with probability ~ r^-s, token = r-1.
    Stands in for the tokenised corpora the reference trains on (not shipped)."""
    rng = np.random.default_rng(seed)
    p = 1.0 / np.power(np.arange(1, vocab + 1, dtype=np.float64), s)
    cdf = np.cumsum(p / p.sum())
    u = rng.random(n)
    return np.minimum(np.searchsorted(cdf, u), vocab - 1).astype(np.uint16)


def uniform_tokens(n: int, vocab: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return rng.integers(0, vocab, size=n, dtype=np.int64).astype(np.uint16)
