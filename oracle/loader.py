"""Token batchers, restated.  Test infrastructure only.

FifoU16 follows src/data/loader.zig:555-589 (U16TokenDatasetFifo.getBatchImpl) exactly: each call
consumes B*T+1 tokens at the cursor; inputs are window[0:B*T], targets window[1:B*T+1], both widened
to i64 and shaped [B, T]; the cursor then moves by B*T+1.  Errors keep the reference's names.

RandomU16 follows src/data/loader.zig:457-486 in structure (one uniformly drawn window start per row,
start in [0, len-T-1]); the reference draws from Zig 0.13's std.Random.DefaultPrng, which is not part
of the reference tree.  Xoshiro256pp below is the published construction that generator is documented
to be (xoshiro256++ seeded through SplitMix64, Lemire's bounded integer); without the Zig sources or a
Zig run to compare with, its sequences are UNPINNED against the reference.  RandomWindows (u16 / u32
tokens), CharTokenizer (src/data/loader.zig:12-89) and init_master (src/algorithms/diloco.zig:513-586)
are what the library's host functions are checked against bit for bit.
"""
from __future__ import annotations

import math

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


# ---------------------------------------------------------------------------------------------------------
# Generator of the random-window datasets and of the master initialisation (pure Python: small cases only)
# ---------------------------------------------------------------------------------------------------------
_M64 = (1 << 64) - 1


class Xoshiro256pp:
    """xoshiro256++ with the state filled by SplitMix64 from a 64-bit seed."""

    def __init__(self, seed: int):
        s = seed & _M64
        self.s = []
        for _ in range(4):
            s = (s + 0x9E3779B97F4A7C15) & _M64
            z = s
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
            self.s.append(z ^ (z >> 31))

    @staticmethod
    def _rotl(x, k):
        return ((x << k) | (x >> (64 - k))) & _M64

    def next(self) -> int:
        s = self.s
        result = (self._rotl((s[0] + s[3]) & _M64, 23) + s[0]) & _M64
        t = (s[1] << 17) & _M64
        s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3]
        s[2] ^= t
        s[3] = self._rotl(s[3], 45)
        return result

    def uint_at_most(self, at_most: int) -> int:
        """Uniform in [0, at_most]: multiply-shift, rejecting the low products that would bias the result."""
        if at_most == _M64:
            return self.next()
        rng = at_most + 1
        m = self.next() * rng
        low = m & _M64
        if low < rng:
            threshold = ((1 << 64) - rng) % rng
            while low < threshold:
                m = self.next() * rng
                low = m & _M64
        return m >> 64

    def normal_pair(self):
        """Two standard normals by the Box-Muller transform in double precision (the reference uses Zig's
        ziggurat sampler, not shipped: same distribution, other values)."""
        u1 = ((self.next() >> 11) + 1) * (1.0 / 9007199254740992.0)
        u2 = (self.next() >> 11) * (1.0 / 9007199254740992.0)
        r = math.sqrt(-2.0 * math.log(u1))
        a = 6.283185307179586476925286766559 * u2
        return r * math.cos(a), r * math.sin(a)


class RandomWindows:
    """getBatchImpl of U16TokenDataset / TextDataset / ByteTextDataset (src/data/loader.zig:457-486, 276-307,
    366-397): per row one start drawn with uintAtMost(len - T - 1); ChunkTooSmall when len <= T + 1."""

    def __init__(self, tokens, seed: int):
        self.tokens = np.ascontiguousarray(tokens)
        self.prng = Xoshiro256pp(seed)

    def get_batch(self, batch_size: int, block_size: int):
        x = np.empty((batch_size, block_size), np.int64)
        y = np.empty((batch_size, block_size), np.int64)
        for i in range(batch_size):
            if self.tokens.size <= block_size + 1:
                raise ChunkTooSmall()
            s = self.prng.uint_at_most(self.tokens.size - block_size - 1)
            x[i] = self.tokens[s:s + block_size]
            y[i] = self.tokens[s + 1:s + block_size + 1]
        return x, y


class CharTokenizer:
    """src/data/loader.zig:12-89: vocabulary = the distinct bytes of the text in ascending order, cut at 65;
    unknown bytes encode to 0; decoding an unknown token is an error."""
    MAX_VOCAB_SIZE = 65

    def __init__(self, text: bytes):
        chars = sorted(set(text))
        self.ignored = max(0, len(chars) - self.MAX_VOCAB_SIZE)
        self.chars = chars[: self.MAX_VOCAB_SIZE]
        self.char_to_int = {c: i for i, c in enumerate(self.chars)}

    @property
    def vocab_size(self):
        return len(self.chars)

    def encode(self, text: bytes) -> np.ndarray:
        return np.array([self.char_to_int.get(c, 0) for c in text], dtype=np.uint32)

    def decode(self, tokens) -> bytes:
        out = bytearray()
        for t in tokens:
            if int(t) >= len(self.chars):
                raise KeyError("UnknownToken")
            out.append(self.chars[int(t)])
        return bytes(out)


def init_master(seed: int, n: int, dtype: str = "f32") -> np.ndarray:
    """src/algorithms/diloco.zig:513-586: n elements 0.02 * N(0,1) from one generator, the product in f32;
    bf16 = the upper 16 bits of the f32 (truncation).  Returns float32 values (f32) or uint16 bit patterns (bf16)."""
    g = Xoshiro256pp(seed)
    vals = np.empty(n, np.float32)
    i = 0
    while i < n:
        for z in g.normal_pair():
            if i < n:
                vals[i] = np.float32(z) * np.float32(0.02)
                i += 1
    if dtype == "bf16":
        return (vals.view(np.uint32) >> 16).astype(np.uint16)
    return vals
