"""tanh-GELU option of the nanoGPT family, host side (no GPU): the exported graph run by the oracle against an
independent PyTorch forward (torch.nn.functional.gelu, approximate="tanh"), and the artefact recogniser."""
import numpy as np
import pytest
import torch
import torch.nn.functional as Fn

from helpers import GPT_GELU_F32, GPT_SMALL_F32, make_model, seeded_params
from oracle.loader import uniform_tokens
from oracle.worker import TrainingModule
from pcp_b200 import backend as bk
from pcp_b200.backend import BackendError, inspect_artifact


def _torch_loss(cfg, P, x, y, act):
    d, H = cfg.d_model, cfg.n_head
    B, T = x.shape
    h = P[0][x] + P[1][None]
    for l in range(cfg.n_layer):
        l1w, l1b, wa, wo, l2w, l2b, wfc, wpr = P[2 + 8 * l:10 + 8 * l]
        q, k, v = (Fn.layer_norm(h, (d,), l1w, l1b, 1e-5) @ wa.T).split(d, dim=-1)
        q, k, v = [t.reshape(B, T, H, d // H).transpose(1, 2) for t in (q, k, v)]
        o = Fn.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, d)
        h = h + o @ wo.T
        h = h + act(Fn.layer_norm(h, (d,), l2w, l2b, 1e-5) @ wfc.T) @ wpr.T
    lw, lb, wh, bh = P[-4:]
    z = Fn.layer_norm(h, (d,), lw, lb, 1e-5) @ wh.T + bh
    return Fn.cross_entropy(z.reshape(-1, cfg.vocab), y.reshape(-1))


@pytest.mark.parametrize("cfgd,act", [(GPT_GELU_F32, lambda u: Fn.gelu(u, approximate="tanh")), (GPT_SMALL_F32, Fn.relu)])
def test_exported_activation_matches_torch(cfgd, act):
    cfg, text = make_model(cfgd)
    params = seeded_params(cfg)
    tok = np.asarray(uniform_tokens(cfg.batch * cfg.seq_len + 1, cfg.vocab, 1), dtype=np.int64)
    x = torch.from_numpy(tok[:-1].reshape(cfg.batch, cfg.seq_len).copy())
    y = torch.from_numpy(tok[1:].reshape(cfg.batch, cfg.seq_len).copy())
    g, loss = TrainingModule(text).compute_gradients(params, x, y)
    P = [p.clone().requires_grad_(True) for p in params]
    ref = _torch_loss(cfg, P, x, y, act)
    ref.backward()
    # the exported graph carries the sanitiser's 1e-4 guards (LayerNorm, softmax, loss), PyTorch does not: the loss
    # agrees to 1e-5, the gradients to a few per cent of each tensor's largest entry
    assert abs(float(loss) - float(ref.detach())) < 1e-5 * abs(float(ref.detach()))
    for a, b in zip(g, P):
        assert float((a - b.grad).abs().max()) <= 5e-2 * float(b.grad.abs().max()) + 1e-7


def test_gelu_changes_the_loss():
    cfg_r, text_r = make_model(GPT_SMALL_F32)
    cfg_g, text_g = make_model(GPT_GELU_F32)
    assert text_g.count("stablehlo.tanh") == cfg_g.n_layer and "stablehlo.tanh" not in text_r
    params = seeded_params(cfg_r, std=0.2)
    tok = np.asarray(uniform_tokens(cfg_r.batch * cfg_r.seq_len + 1, cfg_r.vocab, 1), dtype=np.int64)
    x = torch.from_numpy(tok[:-1].reshape(cfg_r.batch, cfg_r.seq_len).copy())
    y = torch.from_numpy(tok[1:].reshape(cfg_r.batch, cfg_r.seq_len).copy())
    _, lr = TrainingModule(text_r).compute_gradients(params, x, y)
    _, lg = TrainingModule(text_g).compute_gradients(params, x, y)
    assert abs(float(lr) - float(lg)) > 1e-4


def test_recogniser_accepts_gelu_and_refuses_other_activations(lib_built, monkeypatch):
    cfg, text = make_model(GPT_GELU_F32)
    f = inspect_artifact(text)
    assert (f["d_model"], f["n_layer"], f["d_ff"], f["total_params"]) == (cfg.d_model, cfg.n_layer, 4 * cfg.d_model, cfg.num_params())
    assert f["family"] == "fused"
    # a different cubic coefficient is not the activation the fused kernels implement, nor is a graph with one tanh
    # removed (the count no longer matches the layer count): the fused recogniser refuses both ...
    others = (text.replace("4.47149985e-02", "5.00000000e-02"), text.replace("stablehlo.tanh", "stablehlo.negate", 1))
    monkeypatch.setenv("PCPB_FRONTEND", "fused")
    for other in others:
        with pytest.raises(BackendError) as ei:
            inspect_artifact(other)
        assert ei.value.code == bk.E_ARTIFACT
    # ... and without that restriction they run op by op on the general front end
    monkeypatch.delenv("PCPB_FRONTEND")
    for other in others:
        assert inspect_artifact(other)["family"] == "graph"
