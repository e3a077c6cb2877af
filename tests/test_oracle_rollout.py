"""The rollout oracle (oracle/rollout.py) pinned against Hugging Face's Qwen3ForCausalLM -- the model the
reference's generation export wraps (tools/export_qwen3_generation.py) -- and against the sampler's own test
(src/core/math.zig:76-89)."""
import math

import numpy as np
import pytest
import torch

from oracle.rollout import QwenConfig, argmax_first, decode_step, generate, rope_tables, seeded_params

CFG = QwenConfig(vocab=320, d_model=256, n_layer=2, n_head=4, n_kv_head=2, head_dim=64, d_ff=640, max_seq=24, dtype="f32")


def _hf_model(cfg, params):
    tr = pytest.importorskip("transformers")
    hc = tr.Qwen3Config(vocab_size=cfg.vocab, hidden_size=cfg.d_model, intermediate_size=cfg.d_ff,
                        num_hidden_layers=cfg.n_layer, num_attention_heads=cfg.n_head, num_key_value_heads=cfg.n_kv_head,
                        head_dim=cfg.head_dim, max_position_embeddings=cfg.max_seq, rope_theta=cfg.rope_theta,
                        rms_norm_eps=cfg.rms_eps, tie_word_embeddings=False, attention_bias=False)
    m = tr.Qwen3ForCausalLM(hc).eval()
    named = list(m.named_parameters())
    assert [tuple(p.shape) for _, p in named] == [tuple(s) for s in cfg.param_shapes()]      # the argument order
    with torch.no_grad():
        for (_, p), v in zip(named, params):
            p.copy_(v)
    return m


def _oracle_logits(cfg, params, tokens, include_self):
    tables = rope_tables(cfg)
    kc = [torch.zeros(cfg.n_kv_head, cfg.max_seq, cfg.head_dim) for _ in range(cfg.n_layer)]
    vc = [torch.zeros(cfg.n_kv_head, cfg.max_seq, cfg.head_dim) for _ in range(cfg.n_layer)]
    out = []
    for pos, t in enumerate(tokens):
        logits, kn, vn = decode_step(cfg, params, int(t), pos, kc, vc, tables, include_self)
        for l in range(cfg.n_layer):
            kc[l][:, pos] = kn[l]; vc[l][:, pos] = vn[l]
        out.append(logits)
    return torch.stack(out)


def test_architecture_matches_hugging_face_qwen3():
    """With the step's own key / value placed in its slot (the standard causal form) the restated step reproduces the
    Hugging Face model token by token: parameter order, weighted RMSNorm, QK-norm before RoPE, rotate-half RoPE at
    theta 1e6, GQA, SwiGLU, untied head."""
    params = seeded_params(CFG, seed=1, std=0.05)
    m = _hf_model(CFG, params)
    tokens = torch.randint(0, CFG.vocab, (1, 12), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        want = m(tokens).logits[0]
    got = _oracle_logits(CFG, params, tokens[0].tolist(), include_self=True)
    assert float((got - want).abs().max()) <= 1e-4 * float(want.abs().max()) + 1e-5


def test_reference_step_attends_to_a_zero_slot_instead_of_itself():
    """The exported step attends to the cache as it was before the step (the host writes the new rows afterwards,
    src/nodes/workers/generation_engine.zig:285-312): slot pos holds zeros, so the first token's attention output is
    exactly zero and later tokens see one extra key with score 0 and value 0."""
    params = seeded_params(CFG, seed=3, std=0.05)
    tokens = [5, 17, 200, 3]
    ref = _oracle_logits(CFG, params, tokens, include_self=False)
    std = _oracle_logits(CFG, params, tokens, include_self=True)
    assert float((ref - std).abs().max()) > 1e-3                       # the two forms differ
    # position 0 by hand: attention contributes nothing, only the MLP branches act
    from oracle.rollout import PER_LAYER, _linear, _rmsnorm
    h = params[0][tokens[0]].view(1, -1)
    for l in range(CFG.n_layer):
        wg, wu, wd, _, ln2 = params[1 + PER_LAYER * l + 6: 1 + PER_LAYER * (l + 1)]
        x = _rmsnorm(h, ln2, CFG.rms_eps)
        h = h + _linear(torch.nn.functional.silu(_linear(x, wg)) * _linear(x, wu), wd)
    want0 = _linear(_rmsnorm(h, params[-2], CFG.rms_eps), params[-1]).view(-1)
    assert float((ref[0] - want0).abs().max()) <= 1e-5


def test_sampler_greedy_known_answers():
    assert argmax_first(torch.tensor([1.0, 5.0, 2.0])) == 1               # src/core/math.zig:80-82
    assert argmax_first(torch.tensor([3.0, 7.0, 7.0, 1.0])) == 1          # strict '>': the first maximum wins
    assert argmax_first(torch.tensor([float("nan"), 2.0, float("nan")])) == 1
    assert argmax_first(torch.tensor([-math.inf, -math.inf])) == 0


def test_generate_loop_lengths_and_stop():
    cfg = QwenConfig(vocab=64, d_model=128, n_layer=1, n_head=2, n_kv_head=1, head_dim=64, d_ff=256, max_seq=16, dtype="bf16")
    params = seeded_params(cfg, seed=0, std=0.05, head_std=0.5)
    prompt = [1, 2, 3, 4]
    toks, why = generate(cfg, params, prompt, max_new_tokens=5)
    assert len(toks) == 5 and why == "length"
    # the first sampled token comes from the last prompt position; stopping on it ends the loop with one token
    toks2, why2 = generate(cfg, params, prompt, max_new_tokens=5, eos_token=toks[0])
    assert toks2 == toks[:1] and why2 == "stop"
    # an empty prompt starts from token 0 and samples from the first step on
    toks3, _ = generate(cfg, params, [], max_new_tokens=3)
    assert len(toks3) == 3
