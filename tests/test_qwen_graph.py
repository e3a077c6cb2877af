"""A third architecture through the general front end (no GPU here): the Qwen3-style training graph of
pcp_b200/export.py:qwen_forward_mlir.  (1) The exported graph computes what an independent PyTorch implementation of
the architecture computes; (2) the oracle's reverse AD on it agrees with torch.autograd run through the same evaluator
(the reference's method for its AD engine, test/nanochat/test_pcp_gradients_parity.py:39,122-125, here without the
guard terms, which the known-answer tests pin); (3) the library's tensor program of it is exact against the oracle."""
import math

import pytest
import torch

import graph_program as gp
from oracle import stablehlo as hlo
from oracle.worker import TrainingModule
from pcp_b200.backend import graph_describe, inspect_artifact
from pcp_b200.export import QwenConfig, qwen_forward_mlir, rope_tables


def qwen_params(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    # Activations of order one (embedding rows of unit scale, weights ~ fan_in^-1/2, norm weights near 1): the oracle's
    # rsqrt rule evaluates rsqrt(ms + eps + 1e-4)^3 (src/autodiff/vjp_rules.zig:1543), which is within the 1e-4 tolerance
    # of autograd only when the mean squares the norms see are of order one.
    for i, s in enumerate(cfg.param_shapes()):
        p = torch.randn(s, generator=g)
        out.append(p * 0.05 + 1.0 if len(s) == 1 else (p if i == 0 else p * s[1] ** -0.5))
    return out


def qwen_batch(cfg, seed=1):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, cfg.vocab, (cfg.batch, cfg.seq_len), generator=g)
    tg = torch.randint(0, cfg.vocab, (cfg.batch, cfg.seq_len), generator=g)
    tg[0, :2] = -100
    return ids, tg


def _torch_forward(cfg, params, ids, tg):
    """The architecture written directly in PyTorch (f32)."""
    B, T, H, Hkv, hd = cfg.batch, cfg.seq_len, cfg.n_head, cfg.n_kv_head, cfg.head_dim
    cos_b, sin_b = rope_tables(T, hd, cfg.rope_base)
    to_f = lambda bits: torch.from_numpy((bits.astype("uint32") << 16).view("float32").copy()).reshape(1, T, 1, hd // 2)
    cos, sin = to_f(cos_b), to_f(sin_b)

    def rms(x, w):
        return w * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.eps))

    def rope(x):
        x1, x2 = x[..., : hd // 2], x[..., hd // 2:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

    it = iter(params)
    x = next(it)[ids]
    for _ in range(cfg.n_layer):
        ln1, wq, wk, wv, qn, kn, wo, ln2, wg, wu, wd = (next(it) for _ in range(11))
        h = rms(x, ln1)
        q = rope(rms((h @ wq.T).view(B, T, H, hd), qn)).transpose(1, 2)
        k = rope(rms((h @ wk.T).view(B, T, Hkv, hd), kn)).transpose(1, 2).repeat_interleave(H // Hkv, dim=1)
        v = (h @ wv.T).view(B, T, Hkv, hd).transpose(1, 2).repeat_interleave(H // Hkv, dim=1)
        s = (q @ k.transpose(-1, -2)) / math.sqrt(hd)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        o = (torch.softmax(s, -1) @ v).transpose(1, 2).reshape(B, T, H * hd)
        x = x + o @ wo.T
        h = rms(x, ln2)
        x = x + (torch.nn.functional.silu(h @ wg.T) * (h @ wu.T)) @ wd.T
    norm, head = next(it), next(it)
    logits = rms(x, norm) @ head.T
    return torch.nn.functional.cross_entropy(logits.view(B * T, -1), tg.view(-1), ignore_index=-100)


def test_exported_graph_is_the_architecture():
    cfg = QwenConfig()
    text = qwen_forward_mlir(cfg)
    params, (ids, tg) = qwen_params(cfg), qwen_batch(cfg)
    got = hlo.evaluate(hlo.parse_module(text, "main"), params + [ids, tg])
    want = _torch_forward(cfg, params, ids, tg)
    assert abs(float(got) - float(want)) <= 1e-5 * abs(float(want)), (float(got), float(want))


def test_oracle_gradients_of_the_graph_match_autograd():
    cfg = QwenConfig()
    text = qwen_forward_mlir(cfg)
    params, (ids, tg) = qwen_params(cfg), qwen_batch(cfg)
    mod = TrainingModule(text, sanitize=False, guards=False)
    grads, loss = mod.compute_gradients(params, ids, tg)
    leaves = [p.clone().requires_grad_(True) for p in params]
    loss_ag = hlo.evaluate(hlo.parse_module(text, "main"), leaves + [ids, tg])
    loss_ag.backward()
    assert abs(float(loss) - float(loss_ag.detach())) <= 1e-5 * abs(float(loss_ag.detach()))
    for i, (got, leaf) in enumerate(zip(grads, leaves)):
        ref = leaf.grad
        assert float((got - ref).abs().max()) <= 1e-4 + 1e-4 * float(ref.abs().max()), i


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_program_of_the_graph_matches_oracle_exactly(lib_built, dtype):
    cfg = QwenConfig(dtype=dtype)
    text = qwen_forward_mlir(cfg)
    f = inspect_artifact(text)
    assert f["family"] == "graph" and f["total_params"] == cfg.num_params() and f["vocab"] == cfg.vocab
    mod = TrainingModule(text)
    params, (ids, tg) = mod._model_params(qwen_params(cfg)), qwen_batch(cfg)
    loss, grads = gp.run(gp.parse(graph_describe(text)), params + [ids, tg])
    want = mod.model_forward_pass_grad(params, ids, tg, 1.0)
    assert float(loss) == float(mod.forward([p.to(torch.float32) for p in params], ids, tg))
    for a, w in zip(grads, want):
        assert torch.equal(a, w) and float(w.to(torch.float32).abs().max()) > 0
