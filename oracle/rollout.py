"""Rollout generation, restated.  Test infrastructure only.

The reference generates one token per call of a compiled decode-step function with a dense KV cache kept on the
host (src/nodes/workers/generation_engine.zig:174-332); the function is the Qwen3 forward exported by
tools/export_qwen3_generation.py, and the next token is drawn by Sampler.sample (src/core/math.zig:21-73; temperature
< 1e-6 = argmax, first maximum wins).  This module restates both:

decode_step   the exported graph's arithmetic for one token: embedding, per layer weighted RMSNorm -> q/k/v projections
              -> per-head RMSNorm of q and k (before RoPE) -> RoPE (rotate-half form, theta 1e6) -> attention over the
              cache AS IT WAS BEFORE THIS STEP -> output projection -> residual -> weighted RMSNorm -> SwiGLU MLP ->
              residual; final RMSNorm and LM head.  The step returns the new key / value rows; the host writes them into
              the cache afterwards (generation_engine.zig:285-312).  Consequence, kept here because it is what the
              reference computes: at position p the query sees the real keys of positions < p and, at slot p, the
              zero-initialised cache row (score 0, value 0) -- its own key and value are not part of its attention.
              Slots > p carry the additive mask -1e4 on a zero score and underflow to weight 0 in the f32 softmax.
generate      the host loop: prompt tokens are fed one by one, sampling starts at the last prompt token, stops at
              eos_token or after max_new_tokens.

dtype "f32" is the exported graph as the script writes it (DTYPE = float32).  dtype "bf16" is the same op sequence
with every op's result rounded to bf16 (linear layers accumulate in f32 and round once), the softmax in f32 as in the
script, and the RoPE tables computed in f32 from exact integer positions and then rounded to bf16 (the script's own
expression would round the position itself to bf16, which cannot represent positions above 256): the reference has
no bf16 generation graph, so that one point is this restatement's choice.

The architecture is pinned against Hugging Face's Qwen3ForCausalLM (the model the reference's script wraps) in
tests/test_oracle_rollout.py: with the self slot switched to the standard causal form the f32 logits agree with it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch


@dataclass
class QwenConfig:
    vocab: int = 512
    d_model: int = 256
    n_layer: int = 2
    n_head: int = 2
    n_kv_head: int = 1
    head_dim: int = 128
    d_ff: int = 768
    max_seq: int = 64
    rope_theta: float = 1_000_000.0
    rms_eps: float = 1e-6
    dtype: str = "bf16"

    def param_shapes(self):
        """Order of model.named_parameters() of the Hugging Face model, which is the order of the exported function's
        weight arguments (tools/export_qwen3_generation.py: params = dict(model.named_parameters()))."""
        d, hq, hk, f = self.d_model, self.n_head * self.head_dim, self.n_kv_head * self.head_dim, self.d_ff
        s = [(self.vocab, d)]
        for _ in range(self.n_layer):
            s += [(hq, d), (hk, d), (hk, d), (d, hq), (self.head_dim,), (self.head_dim,), (f, d), (f, d), (d, f), (d,), (d,)]
        s += [(d,), (self.vocab, d)]
        return s

    def num_params(self):
        return int(sum(int(np.prod(x)) for x in self.param_shapes()))

    @property
    def torch_dtype(self):
        return torch.float32 if self.dtype == "f32" else torch.bfloat16


PER_LAYER = 11          # q k v o q_norm k_norm gate up down input_ln post_ln


def rope_tables(cfg: QwenConfig):
    """cos / sin [max_seq, head_dim] of the model dtype (emb = cat(freqs, freqs))."""
    half = cfg.head_dim // 2
    inv = torch.tensor([1.0 / (cfg.rope_theta ** (2.0 * i / cfg.head_dim)) for i in range(half)], dtype=torch.float32)
    pos = torch.arange(cfg.max_seq, dtype=torch.float32).view(-1, 1)
    freqs = pos * inv.view(1, -1)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(cfg.torch_dtype), emb.sin().to(cfg.torch_dtype)


def _rmsnorm(x, w, eps):
    """Qwen3RMSNorm: statistics in f32, cast back, then the weight multiply in the model dtype."""
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(-1, keepdim=True)
    return w * (xf * torch.rsqrt(var + eps)).to(x.dtype)


def _rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def _linear(x, w):
    return torch.nn.functional.linear(x, w)


def decode_step(cfg: QwenConfig, params, token: int, pos: int, kcache, vcache, tables, include_self: bool = False):
    """One token at position pos.  kcache / vcache: lists (per layer) of [n_kv_head, max_seq, head_dim] tensors holding
    the rows written by earlier steps (zeros elsewhere).  -> (logits [vocab] in the model dtype, new k rows, new v rows),
    each row list entry [n_kv_head, head_dim].

    include_self=True puts this step's own key / value into slot pos before attending (the standard causal form, used
    only to pin the architecture against the Hugging Face model)."""
    H, Hk, hd = cfg.n_head, cfg.n_kv_head, cfg.head_dim
    cos, sin = tables
    c, s = cos[pos], sin[pos]
    h = params[0][token].view(1, -1)
    k_new, v_new = [], []
    scale = math.sqrt(hd)
    idx = torch.arange(cfg.max_seq)
    zero = torch.tensor(0.0, dtype=cfg.torch_dtype)
    mask = torch.where(idx <= pos, zero, torch.tensor(-1e4, dtype=cfg.torch_dtype))
    for l in range(cfg.n_layer):
        wq, wk, wv, wo, qn, kn, wg, wu, wd, ln1, ln2 = params[1 + PER_LAYER * l: 1 + PER_LAYER * (l + 1)]
        x = _rmsnorm(h, ln1, cfg.rms_eps)
        q = _rmsnorm(_linear(x, wq).view(H, hd), qn, cfg.rms_eps)
        k = _rmsnorm(_linear(x, wk).view(Hk, hd), kn, cfg.rms_eps)
        v = _linear(x, wv).view(Hk, hd)
        q = (q * c) + (_rotate_half(q) * s)
        k = (k * c) + (_rotate_half(k) * s)
        k_new.append(k.clone()); v_new.append(v.clone())
        K, V = kcache[l], vcache[l]
        if include_self:
            K, V = K.clone(), V.clone()
            K[:, pos] = k; V[:, pos] = v
        rep = H // Hk
        Kx = K[:, None].expand(Hk, rep, cfg.max_seq, hd).reshape(H, cfg.max_seq, hd)
        Vx = V[:, None].expand(Hk, rep, cfg.max_seq, hd).reshape(H, cfg.max_seq, hd)
        qs = q / scale
        att = torch.matmul(qs.view(H, 1, hd), Kx.transpose(1, 2)).view(H, cfg.max_seq)
        att = att + mask
        att = torch.softmax(att, dim=-1, dtype=torch.float32).to(q.dtype)
        o = torch.matmul(att.view(H, 1, cfg.max_seq), Vx).reshape(1, H * hd)
        h = h + _linear(o, wo)
        x = _rmsnorm(h, ln2, cfg.rms_eps)
        h = h + _linear(torch.nn.functional.silu(_linear(x, wg)) * _linear(x, wu), wd)
    h = _rmsnorm(h, params[-2], cfg.rms_eps)
    return _linear(h, params[-1]).view(-1), k_new, v_new


def argmax_first(logits) -> int:
    """Sampler.argmax (src/core/math.zig:61-73): strict '>' scan, so the first maximum wins; NaN never wins."""
    best, at = -math.inf, 0
    for i, v in enumerate(logits.to(torch.float32).tolist()):
        if v > best:
            best, at = v, i
    return at


def generate(cfg: QwenConfig, params, prompt, max_new_tokens: int, eos_token: int = -1, include_self: bool = False,
             record_logits=None):
    """generateRolloutStreaming with temperature 0 (generation_engine.zig:174-332).  -> (tokens, finish_reason)."""
    params = [p.to(cfg.torch_dtype) for p in params]
    tables = rope_tables(cfg)
    kc = [torch.zeros(cfg.n_kv_head, cfg.max_seq, cfg.head_dim, dtype=cfg.torch_dtype) for _ in range(cfg.n_layer)]
    vc = [torch.zeros(cfg.n_kv_head, cfg.max_seq, cfg.head_dim, dtype=cfg.torch_dtype) for _ in range(cfg.n_layer)]
    out = []
    pos, total = 0, len(prompt) + max_new_tokens
    while pos < total:
        if pos < len(prompt):
            tok = int(prompt[pos])
        elif out:
            tok = out[-1]
        else:
            tok = 0
        logits, kn, vn = decode_step(cfg, params, tok, pos, kc, vc, tables, include_self)
        last_prompt = len(prompt) > 0 and pos == len(prompt) - 1
        reason = None
        if last_prompt or pos >= len(prompt):
            if record_logits is not None:
                record_logits.append(logits.to(torch.float32).clone())
            nxt = argmax_first(logits)
            out.append(nxt)
            if nxt == eos_token:
                reason = "stop"
            elif len(out) >= max_new_tokens:
                reason = "length"
        for l in range(cfg.n_layer):                      # the host writes the new rows after the step
            if pos < cfg.max_seq:
                kc[l][:, pos] = kn[l]; vc[l][:, pos] = vn[l]
        pos += 1
        if reason:
            return out, reason
    return out, "length"


def seeded_params(cfg: QwenConfig, seed: int = 0, std: float = 0.02, head_std: float | None = None):
    """N(0, std) matrices (the baseline configuration's random weights), norm weights at 1 + N(0, 0.1)."""
    g = torch.Generator().manual_seed(seed)
    out = []
    shapes = cfg.param_shapes()
    for i, s in enumerate(shapes):
        if len(s) == 1:
            out.append(1.0 + 0.1 * torch.randn(s, generator=g))
        else:
            sd = head_std if (head_std is not None and i == len(shapes) - 1) else std
            out.append(torch.randn(s, generator=g) * sd)
    return out
