"""Host-side data functions of the library (no GPU needed): the generator behind random-window batching and master
initialisation, the character tokenizer, master initialisation — against the oracle's restatements bit for bit, and the
generator against the published test vector of its algorithm."""
import os

import numpy as np
import pytest

from oracle.loader import CharTokenizer as OracleTokenizer
from oracle.loader import ChunkTooSmall, RandomWindows, Xoshiro256pp, init_master
from pcp_b200 import backend as bk

REF = os.environ.get("PCP_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))


def test_generator_known_answers():
    """SplitMix64 from seed 0 (the first four outputs fill the state) and the first xoshiro256++ outputs of that state:
    the vectors published with the two algorithms' reference implementations."""
    g = Xoshiro256pp(0)
    assert g.s == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F, 0xF88BB8A8724C81EC]
    want = [0x53175D61490B23DF, 0x61DA6F3DC380D507, 0x5C0FDF91EC9A7BFC]
    assert [g.next() for _ in range(3)] == want
    lib = bk.RandomGenerator(0)
    assert [lib.next() for _ in range(3)] == want


@pytest.mark.parametrize("seed,bound", [(0, 0), (1, 1), (7, 1000), (9, 2**63), (11, 2**64 - 1), (13, 6 * 2**61)])
def test_bounded_integers_match_oracle(seed, bound):
    a, b = Xoshiro256pp(seed), bk.RandomGenerator(seed)
    xs = [a.uint_at_most(bound) for _ in range(500)]
    assert xs == [b.uint_at_most(bound) for _ in range(500)]
    assert max(xs) <= bound


def test_window_starts_match_oracle_and_errors():
    n, B, T = 5000, 16, 64
    tokens = np.arange(n, dtype=np.uint16)
    ds = RandomWindows(tokens, seed=42)
    gen = bk.RandomGenerator(42)
    for _ in range(5):
        x, y = ds.get_batch(B, T)
        starts = gen.window_starts(n, B, T)
        assert np.array_equal(x[:, 0], starts.astype(np.int64)) and np.array_equal(y, x + 1)
        assert starts.max() <= n - T - 1
    with pytest.raises(bk.BackendError) as ei:
        gen.window_starts(T + 1, B, T)                       # len <= T + 1: ChunkTooSmall
    assert ei.value.code == bk.E_CHUNK_TOO_SMALL
    with pytest.raises(ChunkTooSmall):
        RandomWindows(tokens[: T + 1], 0).get_batch(B, T)
    assert set(gen.window_starts(T + 2, 64, T).tolist()) == {0, 1}   # the smallest accepted chunk: two admissible starts


def test_window_starts_are_uniform():
    gen = bk.RandomGenerator(3)
    starts = gen.window_starts(1000 + 9, 200000, 8)         # starts in [0, 1000]
    hist = np.bincount(starts.astype(np.int64), minlength=1001)
    assert hist.min() > 0 and abs(hist.mean() - 200000 / 1001) < 1e-9
    assert hist.std() < 3 * np.sqrt(200000 / 1001)


def _texts():
    rng = np.random.default_rng(0)
    yield b"hello, world\nhello"
    yield bytes(rng.integers(0, 256, 4000, dtype=np.uint8))          # more than 65 distinct bytes: the tail is ignored
    yield b""
    p = os.path.join(REF, "data", "tiny_shakespeare.txt")
    if os.path.exists(p):
        with open(p, "rb") as f:
            yield f.read()[:200000]


def test_char_tokenizer_matches_oracle():
    for text in _texts():
        a, b = OracleTokenizer(text), bk.CharTokenizer(text)
        assert a.vocab_size == b.vocab_size <= 65 and a.chars == b.chars and a.ignored == b.ignored
        probe = text[:3000] + bytes(range(256))
        ta, tb = a.encode(probe), b.encode(probe)
        assert tb.dtype == np.uint32 and np.array_equal(ta, tb)
        if a.vocab_size:
            known = bytes(c for c in probe if c in a.char_to_int)
            assert b.decode(b.encode(known)) == known == a.decode(a.encode(known))
        with pytest.raises(bk.BackendError):
            b.decode([a.vocab_size])                              # UnknownToken
        with pytest.raises(KeyError):
            a.decode([a.vocab_size])


def test_tiny_shakespeare_vocabulary_is_65():
    p = os.path.join(REF, "data", "tiny_shakespeare.txt")
    if not os.path.exists(p):
        pytest.skip("reference tree not present")
    with open(p, "rb") as f:
        tok = bk.CharTokenizer(f.read())
    assert tok.vocab_size == 65 and tok.ignored == 0               # the char-vocab-65 models of the reference


@pytest.mark.parametrize("dtype,code", [("f32", bk.F32), ("bf16", bk.BF16)])
def test_init_master_matches_oracle(dtype, code):
    for seed, n in [(12345, 1001), (0, 2), (7, 1)]:
        assert np.array_equal(init_master(seed, n, dtype), bk.init_master_elems(seed, n, code))
    if dtype == "bf16":                                             # truncation: the upper halves of the f32 values
        f = bk.init_master_elems(12345, 1001, bk.F32)
        assert np.array_equal(bk.init_master_elems(12345, 1001, bk.BF16), (f.view(np.uint32) >> 16).astype(np.uint16))


def test_init_master_distribution():
    x = bk.init_master_elems(12345, 400000, bk.F32).astype(np.float64)
    assert abs(x.mean()) < 2e-4 and abs(x.std() - 0.02) < 1e-4
    assert abs(np.mean(x ** 4) / x.var() ** 2 - 3.0) < 0.05         # normal kurtosis
    with pytest.raises(bk.BackendError):
        bk.init_master_elems(0, 4, bk.I64)
