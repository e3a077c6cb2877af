"""Rollout generation on the GPU (batched prefill, paged KV cache, greedy decode, through the C ABI) against the
restated reference loop (oracle/rollout.py: one token per call, dense cache, host argmax).

Token ids are compared bit for bit on a model whose head is scaled up so that the winning logit leads by far more
than bf16 rounding noise (with N(0, 0.02) weights everywhere the logits are nearly flat, and the arg-max of two
correctly rounded evaluations with different summation orders can differ); the logits themselves are compared
within the bf16 tolerance."""
import numpy as np
import pytest
import torch

from oracle.rollout import QwenConfig, generate, seeded_params
from pcp_b200 import BackendError
from pcp_b200 import backend as bk
from pcp_b200.backend import Rollout

pytestmark = pytest.mark.gpu

# Qwen3 geometry in small: head_dim 128, 4 query heads on 2 kv heads (GQA), weighted norms, SwiGLU
SMALL = QwenConfig(vocab=1024, d_model=512, n_layer=2, n_head=4, n_kv_head=2, head_dim=128, d_ff=1024, max_seq=64, dtype="bf16")
# head_dim 64, two kv heads for eight query heads, odd vocabulary size (a multiple of 8 only)
HD64 = QwenConfig(vocab=1000, d_model=512, n_layer=1, n_head=8, n_kv_head=2, head_dim=64, d_ff=512, max_seq=48, dtype="bf16")


def _engine(cfg, max_batch=16, page_tokens=4):
    return Rollout(0, cfg.vocab, cfg.d_model, cfg.n_layer, cfg.n_head, cfg.n_kv_head, cfg.head_dim, cfg.d_ff, cfg.max_seq,
                   max_batch=max_batch, max_prompt=cfg.max_seq, page_tokens=page_tokens, rope_theta=cfg.rope_theta, rms_eps=cfg.rms_eps)


def _blob_bf16(params):
    return np.concatenate([p.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16).reshape(-1) for p in params])


def _clear_prefix(rec, thr=0.02):
    """Number of leading steps whose winning logit leads the runner-up by more than thr of the largest logit."""
    n = 0
    for z in rec:
        top2 = torch.topk(z, 2).values
        if float(top2[0] - top2[1]) <= thr * float(z.abs().max()):
            break
        n += 1
    return n


@pytest.mark.parametrize("cfg", [SMALL, HD64])
def test_rollout_tokens_match_oracle(cfg):
    """Free-running greedy generation of six ragged prompts (one empty).  Arg-max over bf16 logits is decided by the
    last bit when two logits nearly tie, and two correct evaluations with different summation orders may then pick
    different tokens; so the tokens are required to be identical up to each sequence's first near-tie (and to be one of
    the oracle's two leaders there), the logits to agree within the bf16 tolerance, and the chosen token to be exactly
    the first maximum of the device's own logits."""
    from oracle.rollout import argmax_first
    params = seeded_params(cfg, seed=0, std=0.05, head_std=1.0)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (9, 1, 17, 5, 12)] + [[]]     # ragged, one empty
    new = 10
    want, logits_ref = [], []
    for p in prompts:
        rec = []
        toks, why = generate(cfg, params, p, new, record_logits=rec)
        assert why == "length"
        want.append(toks); logits_ref.append(rec)
    with _engine(cfg) as eng:
        assert eng.num_params == cfg.num_params()
        eng.ensure_device_weights(_blob_bf16(params))
        got, reasons, (pre_ms, dec_ms) = eng.generate_rollout(prompts, new)
        assert eng.launch_count > 0 and pre_ms > 0 and dec_ms > 0
        last_logits = [eng.read_logits(b) for b in range(len(prompts))]
        # one token per prompt: the logits read back are those of the prefill's last prompt row
        got1, _, _ = eng.generate_rollout(prompts, 1)
        first_logits = [eng.read_logits(b) for b in range(len(prompts))]
    assert reasons == ["length"] * len(prompts)
    compared = 0
    for b in range(len(prompts)):
        n = _clear_prefix(logits_ref[b])
        assert got[b][:n] == want[b][:n], (b, n, got[b], want[b])
        if n < new:
            assert got[b][n] in torch.topk(logits_ref[b][n], 2).indices.tolist(), (b, n)
        compared += n
        # prefill logits against the oracle's; bit-exact arg-max of the device's own logits
        ref = logits_ref[b][0].numpy()
        assert np.abs(first_logits[b] - ref).max() <= 2e-2 * np.abs(ref).max(), b
        assert got1[b] == [argmax_first(torch.from_numpy(first_logits[b]))] == got[b][:1], b
        assert got[b][-1] == argmax_first(torch.from_numpy(last_logits[b])), b
        if n == new:                                         # the whole sequence agreed: so must the last step's logits
            ref = logits_ref[b][-1].numpy()
            assert np.abs(last_logits[b] - ref).max() <= 2e-2 * np.abs(ref).max(), b
    assert compared >= 2 * len(prompts), compared             # the test compared a meaningful number of tokens


def test_rollout_stops_at_eos_and_pages_are_reused():
    """eos_token ends a sequence ("stop") while the others run to max_new_tokens ("length"); a second call reuses the
    cache pages and the captured decode graph.  The model seed is the first one for which the oracle's first three
    steps of sequence 0 and first five of sequence 1 are decided by a clear margin."""
    cfg = SMALL
    prompts = [[7, 8, 9], [100, 200]]
    for seed in range(3, 40):
        params = seeded_params(cfg, seed=seed, std=0.05, head_std=1.0)
        recs = [[], []]
        full = [generate(cfg, params, p, 8, record_logits=r)[0] for p, r in zip(prompts, recs)]
        eos = full[0][2]                                     # the third token of sequence 0
        if _clear_prefix(recs[0]) >= 3 and _clear_prefix(recs[1]) >= 5 and eos not in full[0][:2] and eos not in full[1]:
            break
    else:
        pytest.skip("no seed with clear margins")
    n1 = _clear_prefix(recs[1])
    with _engine(cfg, max_batch=2, page_tokens=16) as eng:
        eng.ensure_device_weights(np.concatenate([p.reshape(-1).numpy() for p in params]).astype(np.float32))   # f32 blob
        for _ in range(2):
            got, reasons, _ = eng.generate_rollout(prompts, 8, eos_token=eos)
            assert got[0] == full[0][:3] and reasons[0] == "stop"
            assert got[1][:n1] == full[1][:n1] and len(got[1]) == 8 and reasons[1] == "length"


def test_prefill_on_the_tensor_core_attention_kernel(monkeypatch):
    """Prompts of one length that is a multiple of 128 (head_dim 128) are prefilled with the tcgen05 attention kernel
    over a staged copy of q and of k, v shifted by one position behind a zero row -- which gives the ordinary causal
    kernel exactly the slots the exported step attends to.  Checked against the oracle and against the row kernel."""
    cfg = QwenConfig(vocab=1024, d_model=512, n_layer=2, n_head=4, n_kv_head=2, head_dim=128, d_ff=1024, max_seq=160, dtype="bf16")
    params = seeded_params(cfg, seed=5, std=0.05, head_std=1.0)
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, cfg.vocab, size=128).tolist() for _ in range(3)]
    new = 4
    recs = [[] for _ in prompts]
    want = [generate(cfg, params, p, new, record_logits=r)[0] for p, r in zip(prompts, recs)]
    out = {}
    for mode in ("", "rows"):
        monkeypatch.setenv("PCPB_ROLLOUT_PREFILL", mode)
        with _engine(cfg, max_batch=4, page_tokens=16) as eng:
            eng.ensure_device_weights(_blob_bf16(params))
            toks, _, _ = eng.generate_rollout(prompts, 1)                # the prefill's own logits
            first = [eng.read_logits(b) for b in range(len(prompts))]
            full, _, _ = eng.generate_rollout(prompts, new)
            out[mode] = (toks, first, full)
    for mode, (toks, first, full) in out.items():
        for b in range(len(prompts)):
            ref = recs[b][0].numpy()
            assert np.abs(first[b] - ref).max() <= 2e-2 * np.abs(ref).max(), (mode, b)
            n = _clear_prefix(recs[b])
            assert full[b][:n] == want[b][:n], (mode, b, n)
    # the two prefill paths differ only by rounding noise
    for b in range(len(prompts)):
        assert np.abs(out[""][1][b] - out["rows"][1][b]).max() <= 1e-2 * np.abs(out["rows"][1][b]).max()


def test_rollout_argument_errors():
    cfg = HD64
    with _engine(cfg, max_batch=2) as eng:
        with pytest.raises(BackendError) as ei:
            eng.generate_rollout([[1, 2]], 4)                # no weights yet
        assert ei.value.code == bk.E_STATE
        eng.random_weights(0, 0.02)
        with pytest.raises(BackendError) as ei:
            eng.generate_rollout([[1]] * 3, 4)               # more sequences than max_batch
        assert ei.value.code == bk.E_INVALID
        with pytest.raises(BackendError) as ei:
            eng.generate_rollout([[1] * 40], 20)             # prompt + new tokens beyond max_seq
        assert ei.value.code == bk.E_TOO_LARGE
        with pytest.raises(BackendError) as ei:
            eng.generate_rollout([[1]], 4, temperature=0.7)  # sampling with temperature stays on the host
        assert ei.value.code == bk.E_INVALID
        toks, _, _ = eng.generate_rollout([[1, 2, 3]], 4)
        assert len(toks[0]) == 4 and all(0 <= t < cfg.vocab for t in toks[0])
    with pytest.raises(BackendError):
        Rollout(0, 1000, 200, 1, 4, 1, 64, 512, 48)           # d_model not a multiple of 512
