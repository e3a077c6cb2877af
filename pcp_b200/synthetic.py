"""Seeded synthetic inputs (host side): token streams with the shapes and value distributions of the
reference's training corpora (tokenised FineWeb-Edu / tiny-shakespeare are not shipped), and the bf16
truncation the reference applies to parameter / delta blobs."""
from __future__ import annotations

import numpy as np


def zipf_tokens(n: int, vocab: int, s: float, seed: int) -> np.ndarray:
    """u16 stream: rank r in [1, vocab] with probability ~ r^-s, token = r-1."""
    rng = np.random.default_rng(seed)
    p = 1.0 / np.power(np.arange(1, vocab + 1, dtype=np.float64), s)
    cdf = np.cumsum(p / p.sum())
    return np.minimum(np.searchsorted(cdf, rng.random(n)), vocab - 1).astype(np.uint16)


def uniform_tokens(n: int, vocab: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return rng.integers(0, vocab, size=n, dtype=np.int64).astype(np.uint16)


def f32_to_bf16_trunc_bits(x) -> np.ndarray:
    """f32 -> bf16 bit patterns by dropping the low 16 bits (src/algorithms/diloco.zig:547-552)."""
    return (np.ascontiguousarray(x, np.float32).view(np.uint32) >> 16).astype(np.uint16)


def bf16_bits_to_f32(u) -> np.ndarray:
    return (np.ascontiguousarray(u, np.uint16).astype(np.uint32) << 16).view(np.float32)
