"""Tensor-core GEMM (tcgen05 / TMEM / TMA) against float64 numpy on the same bf16 inputs, all three operand
layouts and every epilogue, plus agreement with the generic kernel.  Called through the C ABI (pcpb_op_gemm)."""
import numpy as np
import pytest

from helpers import HD128_BF16, bf16_bits_to_f32
from pcp_b200 import BF16, F32, Backend, NanochatConfig, nanochat_forward_mlir
from pcp_b200.export import f32_to_bf16_rne

pytestmark = pytest.mark.gpu


def _bf16(a):
    bits = f32_to_bf16_rne(np.asarray(a, np.float32))
    return bits, bf16_bits_to_f32(bits).reshape(np.shape(a))


@pytest.fixture(scope="module")
def be():
    b = Backend(0)
    b.load_session(nanochat_forward_mlir(NanochatConfig(**HD128_BF16)))
    yield b
    b.close()


def _run(be, layout, M, N, K, epi, path, seed=0):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((M, K)).astype(np.float32)
    bm = rng.standard_normal((K, N)).astype(np.float32)
    if layout == "nt":       # forward: A [M,K] k-contiguous, B stored [N,K]
        abits, av = _bf16(a); bbits, bv = _bf16(bm.T.copy()); bv = bv.T
        sa, sb = (K, 1), (1, K)
    elif layout == "nn":     # dgrad: A [M,K] k-contiguous, B stored [K,N]
        abits, av = _bf16(a); bbits, bv = _bf16(bm)
        sa, sb = (K, 1), (N, 1)
    else:                    # "tn" wgrad: A stored [K,M], B stored [K,N]
        abits, av = _bf16(a.T.copy()); av = av.T; bbits, bv = _bf16(bm)
        sa, sb = (1, M), (N, 1)
    ref = av.astype(np.float64) @ bv.astype(np.float64)
    A = be.move_to_device(abits, abits.shape, BF16)
    B = be.move_to_device(bbits, bbits.shape, BF16)
    R = C2 = None
    rv = None
    if epi in (1, 3, 6, 9):
        rbits, rv = _bf16(rng.standard_normal((M, N)))
        R = be.move_to_device(rbits, (M, N), BF16)
    if epi == 7:
        rbits, rv = _bf16(rng.standard_normal((N,)))
        R = be.move_to_device(rbits, (N,), BF16)
    if epi in (2, 5, 8):
        C2 = be.allocate_zeros_device((M, N), BF16)
    Cb = be.allocate_zeros_device((M, N), F32 if epi == 4 else BF16)
    be.op_gemm(A, sa[0], sa[1], B, sb[0], sb[1], Cb, N, M, N, K, epilogue=epi, R=R, C2=C2, path=path)
    out = be.read_to_host(Cb, F32 if epi == 4 else BF16, (M, N))
    out = out if epi == 4 else bf16_bits_to_f32(out).reshape(M, N)
    out2 = bf16_bits_to_f32(be.read_to_host(C2, BF16, (M, N))).reshape(M, N) if C2 else None
    for x in (A, B, Cb, R, C2):
        if x is not None:
            x.release()
    r32 = ref.astype(np.float32)
    rb = lambda x: _bf16(x)[1]
    if epi == 0:
        want = rb(r32)
    elif epi == 1:
        want = rb(rv + rb(r32))
    elif epi == 2:
        want = rb(r32)
    elif epi == 3:
        u = rv; r = np.maximum(u, 0)
        with np.errstate(divide="ignore", invalid="ignore"):
            q = rb(np.where(r > 0, rb(r * r) / np.where(r > 0, r, 1), 0))
        clip = lambda x: np.clip(x, -100, 100)             # the backward epilogues pass adjoint edges (clamp +-100)
        want = np.where(u > 0, clip(rb(clip(rb(r32)) * rb(2 * q))), 0).astype(np.float32)
    elif epi == 4:
        want = np.clip(rb(r32), -100, 100)
    elif epi == 5:
        want = rb(r32)
    elif epi == 6:
        want = np.where(rv > 0, np.clip(rb(r32), -100, 100), 0).astype(np.float32)
    elif epi == 7:
        want = rb(r32 + rv[None, :])
    elif epi == 8:
        want = rb(r32)
    else:
        want = np.clip(rb(np.clip(rb(r32), -100, 100).astype(np.float64) * _gelu_grad(rv)), -100, 100)
    return out, want, out2


GC1, GC2 = _bf16(np.float32(0.7978845608028654))[1], _bf16(np.float32(0.044715))[1]


def _gelu_bf16(u):
    """The nine ops of the exported tanh GELU, each rounded to bf16."""
    rb = lambda x: _bf16(np.asarray(x, np.float32))[1]
    z = rb(GC1 * rb(u + rb(GC2 * rb(rb(u * u) * u))))
    t = rb(np.tanh(z.astype(np.float64)))
    return rb(rb(np.float32(0.5) * u) * rb(t + np.float32(1)))


def _gelu_grad(u):
    u = u.astype(np.float64)
    c1, c2 = float(GC1), float(GC2)
    t = np.tanh(c1 * (u + c2 * u ** 3))
    return 0.5 * (1 + t) + 0.5 * u * (1 - t * t) * c1 * (1 + 3 * c2 * u * u)


LAYOUTS = ["nt", "nn", "tn"]
SHAPES = [(128, 256, 64), (256, 256, 256), (256, 768, 512), (384, 128, 192), (512, 1024, 256)]


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("shape", SHAPES)
def test_tc_gemm_store(be, layout, shape):
    M, N, K = shape
    out, want, _ = _run(be, layout, M, N, K, epi=0, path=2)
    # accumulation order differs from numpy: allow one bf16 ulp on the rounded result
    np.testing.assert_allclose(out, want, rtol=2 ** -7, atol=2 ** -7 * np.sqrt(K) * 0.05)
    assert np.abs(out - want).mean() < 2e-3 * np.sqrt(K)


@pytest.mark.parametrize("layout,epi", [("nt", 1), ("nt", 2), ("nn", 3), ("tn", 4), ("nn", 0), ("nt", 4), ("nt", 5),
                                        ("nn", 6), ("nt", 7), ("nt", 8), ("nn", 9)])
def test_tc_gemm_epilogues(be, layout, epi):
    M, N, K = 256, 512, 320
    out, want, out2 = _run(be, layout, M, N, K, epi=epi, path=2, seed=epi + 1)
    gen, _, gen2 = _run(be, layout, M, N, K, epi=epi, path=1, seed=epi + 1)
    np.testing.assert_allclose(out, want, rtol=2 ** -6, atol=0.15)
    # tensor-core and generic kernels round the same f32 sums up to summation order
    assert np.mean(out != gen) < 0.02
    np.testing.assert_allclose(out, gen, rtol=2 ** -6, atol=0.15)
    if epi == 2:
        r = np.maximum(out, 0)
        np.testing.assert_array_equal(out2, _bf16(r * r)[1])
    if epi == 5:
        np.testing.assert_array_equal(out2, np.maximum(out, 0))
    if epi == 8:
        # second output from the first as stored; tanh is the only op that is not exactly rounded
        want2 = _gelu_bf16(out)
        assert np.mean(out2 != want2) < 1e-3
        np.testing.assert_allclose(out2, want2, rtol=2 ** -7, atol=1e-6)
        assert np.mean(gen2 != _gelu_bf16(gen)) < 1e-3


def test_tc_gemm_split_k(be):
    """Weight-gradient shape: few output tiles and a long contraction -> split over CTAs with f32 slabs."""
    M, N, K = 256, 256, 4096
    out, want, _ = _run(be, "tn", M, N, K, epi=4, path=2, seed=11)
    np.testing.assert_allclose(out, want, rtol=2 ** -6, atol=0.5)
    out_b, _, _ = _run(be, "tn", M, N, K, epi=4, path=2, seed=11)
    np.testing.assert_array_equal(out, out_b)        # deterministic: no atomics in the reduction


# ---- f32 models on the tensor cores: operands split into three bf16 pieces, six products in one bf16 GEMM --------------
F32_TC_MODEL = dict(vocab=512, d_model=256, n_layer=1, n_head=2, n_kv_head=2, seq_len=128, batch=2, dtype="f32")


@pytest.fixture(scope="module")
def be32():
    b = Backend(0)
    b.load_session(nanochat_forward_mlir(NanochatConfig(**F32_TC_MODEL)))
    yield b
    b.close()


def _run32(be, layout, M, N, K, epi, path, seed=0, scale=1.0):
    rng = np.random.default_rng(seed)
    a = (rng.standard_normal((M, K)) * scale).astype(np.float32)
    bm = rng.standard_normal((K, N)).astype(np.float32)
    if layout == "nt":
        ah, bh, sa, sb = a, bm.T.copy(), (K, 1), (1, K)
    elif layout == "nn":
        ah, bh, sa, sb = a, bm, (K, 1), (N, 1)
    else:
        ah, bh, sa, sb = a.T.copy(), bm, (1, M), (N, 1)
    ref = a.astype(np.float64) @ bm.astype(np.float64)
    A = be.move_to_device(ah, ah.shape, F32)
    B = be.move_to_device(bh, bh.shape, F32)
    R = None
    rv = None
    if epi == 1:
        rv = rng.standard_normal((M, N)).astype(np.float32)
        R = be.move_to_device(rv, (M, N), F32)
    if epi == 7:
        rv = rng.standard_normal((N,)).astype(np.float32)
        R = be.move_to_device(rv, (N,), F32)
    Cb = be.allocate_zeros_device((M, N), F32)
    be.op_gemm(A, sa[0], sa[1], B, sb[0], sb[1], Cb, N, M, N, K, epilogue=epi, R=R, path=path)
    out = be.read_to_host(Cb, F32, (M, N)).astype(np.float64)
    for x in (A, B, Cb, R):
        if x is not None:
            x.release()
    if epi == 1:
        ref = ref + rv
    elif epi == 7:
        ref = ref + rv[None, :]
    elif epi == 4:
        ref = np.clip(ref, -100, 100)
    return out, ref


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("shape", [(256, 256, 512), (128, 128, 64), (256, 1024, 256), (128, 128, 2048)])
def test_f32_split_gemm_is_f32_accurate(be32, layout, shape):
    """path 0 = what the f32 models' GEMMs take: for these shapes the split-operand tensor-core path.  The result has to
    be as close to the float64 product as an f32 FMA chain is (the SIMT kernel, path 1), far inside the 1e-4 of the f32
    parity tests; a single bf16 product would be off by 1e-2."""
    M, N, K = shape
    n0 = be32.launch_count
    out, ref = _run32(be32, layout, M, N, K, 0, path=0)
    assert be32.launch_count - n0 >= 4                       # two packs, the GEMM (+ its split-K reduction), the epilogue
    n0 = be32.launch_count
    gen, _ = _run32(be32, layout, M, N, K, 0, path=1)
    assert be32.launch_count - n0 == 1
    # unit-variance operands: the products sum to about sqrt(K).  An f32 FMA chain rounds to nearest at every step (a
    # random walk, ~ sqrt(K)); the tensor core truncates when it adds into its accumulator, a one-sided error that grows
    # with the number of steps taken at full magnitude (~ K; measured at K = 2048: 5.5e-4 against 2.7e-4 for the FMA
    # chain, at K = 64: 4.7e-6 against 1.1e-5).  One bf16 product per term would be off by 4e-3 sqrt(K).
    tol = 2e-6 * np.sqrt(K) + 3e-7 * K
    assert np.abs(gen - ref).max() <= tol
    assert np.abs(out - ref).max() <= tol


@pytest.mark.parametrize("epi", [1, 4, 7])
def test_f32_split_gemm_epilogues(be32, epi):
    out, ref = _run32(be32, "nt", 256, 256, 256, epi, path=0, seed=3, scale=8.0 if epi == 4 else 1.0)
    assert np.abs(out - ref).max() <= (2e-3 if epi == 4 else 2e-4)          # epi 4: operands scaled by 8
    if epi == 4:
        assert (np.abs(out) <= 100).all() and (np.abs(out) == 100).any()           # the clamp was active
