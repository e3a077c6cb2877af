"""GPU parity of the general StableHLO front end (one kernel per op of the library's tensor program) against the CPU
oracle, called through the C ABI.  PCPB_FRONTEND=graph sends graphs of the fused families down the general path too,
so the same oracle cases check it; a graph of neither family takes it by itself.  Tolerances as for the fused path:
f32 1e-4 relative, bf16 2e-2 on the loss and 4e-2 on the gradients."""
import numpy as np
import pytest
import torch

import helpers
from helpers import flat, make_model, rel_err, seeded_params, tokens_for
from oracle.loader import FifoU16
from oracle.optim import AdamConf
from oracle.worker import TrainingModule, inner_loop
from pcp_b200 import BF16, F32, I64, Backend
from pcp_b200.backend import inspect_artifact
from test_gpu_branches import _forward_pass_grad
from test_gpu_parity import _grads_via_abi

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["SMALL_F32", "GQA_F32", "GPT_SMALL_F32", "GPT_GELU_F32", "SMALL_BF16", "GPT_SMALL_BF16",
                                  "HD128_BF16"])
def test_general_path_gradients_match_oracle(name, monkeypatch):
    """HD128_BF16 has products of tensor-core shape: those leave the per-op GEMM kernel for the tcgen05 one."""
    monkeypatch.setenv("PCPB_FRONTEND", "graph")
    cfgd = getattr(helpers, name)
    cfg, text = make_model(cfgd)
    assert inspect_artifact(text)["family"] == "graph"
    mod = TrainingModule(text)
    params = seeded_params(cfg, seed=0, std=0.05)
    x, y = FifoU16(tokens_for(cfg, 1, seed=1)).get_batch(cfg.batch, cfg.seq_len)
    y[0, :2] = -1 if "n_kv_head" in cfgd else -100
    g_ref, loss_ref = mod.compute_gradients(params, torch.from_numpy(x), torch.from_numpy(y))
    with Backend(0) as be:
        be.load_session(text)
        assert be.param_shapes() == [tuple(s) for s in cfg.param_shapes()]
        n0 = be.launch_count
        g, loss = _grads_via_abi(be, cfg, params, x, y)
        assert be.launch_count - n0 > 100              # one kernel per op
        g2, loss2 = _grads_via_abi(be, cfg, params, x, y)        # the arena is reused; no float atomics on the way: same bits
        assert loss2 == loss and all(np.array_equal(a, b) for a, b in zip(g, g2))
    f32 = cfg.dtype == "f32"
    assert abs(loss - float(loss_ref)) <= (1e-4 if f32 else 2e-2) * abs(float(loss_ref)), (loss, float(loss_ref))
    worst = max(rel_err(a, b.numpy()) for a, b in zip(g, g_ref))
    l2 = max(float(np.linalg.norm(a - b.numpy()) / (np.linalg.norm(b.numpy()) + 1e-30)) for a, b in zip(g, g_ref))
    if f32:
        assert worst <= 1e-4, worst
    else:
        assert l2 <= 4e-2 and worst <= 0.25, (l2, worst)
    print(f"{name}: loss {loss:.6f} vs {float(loss_ref):.6f}, worst {worst:.2e}, l2 {l2:.2e}")


def test_general_path_forward_and_seeded_gradients(monkeypatch):
    """model_forward_pass (forward ops only) and model_forward_pass_grad with d(loss) = 500, where the oracle's clamp of
    the adjoint edges is active."""
    monkeypatch.setenv("PCPB_FRONTEND", "graph")
    cfg, text = make_model(helpers.SMALL_F32)
    mod = TrainingModule(text)
    params = seeded_params(cfg, seed=0, std=0.05)
    x, y = FifoU16(tokens_for(cfg, 1, seed=1)).get_batch(cfg.batch, cfg.seq_len)
    tx, ty = torch.from_numpy(x), torch.from_numpy(y)
    ref500 = mod.model_forward_pass_grad(params, tx, ty, 500.0)
    ref_loss = float(mod.forward(params, tx, ty))
    with Backend(0) as be:
        be.load_session(text)
        bufs = [be.move_to_device(p.numpy(), p.shape, F32) for p in params]
        bufs += [be.move_to_device(x, x.shape, I64), be.move_to_device(y, y.shape, I64)]
        outs = be.execute_with_device_buffers(None, "model_forward_pass", bufs)
        loss = float(be.read_to_host(outs[0], F32, ())[()])
        for b in bufs + outs:
            b.release()
        assert abs(loss - ref_loss) <= 1e-5 * abs(ref_loss)
        g500 = _forward_pass_grad(be, params, x, y, 500.0)
    assert max(rel_err(a, b.numpy()) for a, b in zip(g500, ref500)) <= 1e-4


@pytest.mark.parametrize("name,tol", [("SMALL_F32", 1e-4), ("GPT_SMALL_BF16", 2e-2)])
def test_graph_of_neither_family_trains_like_the_oracle(name, tol):
    """A graph the fused recogniser refuses (logistic where the family has tanh): the worker round runs it op by op —
    three AdamW steps, the per-step losses and the round's delta against the oracle's inner loop."""
    cfgd = getattr(helpers, name)
    cfg, text = make_model(cfgd)
    text = text.replace("stablehlo.tanh ", "stablehlo.logistic ", 1) if "n_kv_head" in cfgd else \
        text.replace("= stablehlo.maximum ", "= stablehlo.minimum ", 1)
    assert inspect_artifact(text)["family"] == "graph"
    mod = TrainingModule(text)
    dt = F32 if cfg.dtype == "f32" else BF16
    master = seeded_params(cfg, seed=0, std=0.02)
    if dt == BF16:
        master = [torch.from_numpy(helpers.bf16_bits_to_f32(helpers.f32_to_bf16_trunc_bits(p.numpy())).reshape(p.shape)) for p in master]
    tau = 3
    toks = tokens_for(cfg, tau, seed=7)
    conf = AdamConf(learning_rate=1e-3)
    rec = []
    d_ref, _, _, _ = inner_loop(mod, master, FifoU16(toks), tau, cfg.batch, cfg.seq_len, conf, record=rec)
    with Backend(0) as be:
        be.load_session(text)
        be.set_adam(conf.learning_rate, conf.beta1, conf.beta2, conf.epsilon, conf.weight_decay, conf.max_grad_norm)
        blob = flat(master) if dt == F32 else helpers.f32_to_bf16_trunc_bits(flat(master))
        be.worker_begin_round(tau, blob, param_dtype=dt)
        be.worker_set_tokens(toks)
        for _ in range(tau):
            be.worker_step()
        delta, losses = be.worker_end_round(tau, param_dtype=dt)
    np.testing.assert_allclose(losses, [r[0] for r in rec], rtol=tol)
    dgpu = delta if dt == F32 else helpers.bf16_bits_to_f32(delta)
    after, after_ref = flat(master) - dgpu, flat(master) - flat(d_ref)
    assert rel_err(after, after_ref) <= tol


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_op_zoo_on_the_gpu(dtype):
    """The hand-written graph of tests/graph_zoo.py (sine, cosine, logistic, strided slices, three-way concatenate,
    rank-3 transpose, batched dot_general, reductions over middle and leading dimensions, broadcasts into non-adjacent
    dimensions, integer converts, compare + select, ops without a gradient rule) against the oracle."""
    from graph_zoo import ZOO_BATCH, ZOO_BLOCK, ZOO_MLIR, ZOO_PARAM_SHAPES, ZOO_VOCAB
    text = ZOO_MLIR.replace("f32", dtype)
    mod = TrainingModule(text)
    g = torch.Generator().manual_seed(0)
    params = [torch.randn(s, generator=g) * 0.5 for s in ZOO_PARAM_SHAPES]
    x = torch.randint(0, ZOO_VOCAB, (ZOO_BATCH, ZOO_BLOCK), generator=g).numpy()
    y = torch.randint(0, ZOO_VOCAB, (ZOO_BATCH, ZOO_BLOCK), generator=g).numpy()
    g_ref, loss_ref = mod.compute_gradients(params, torch.from_numpy(x), torch.from_numpy(y))
    with Backend(0) as be:
        be.load_session(text)
        assert be.param_shapes() == [tuple(s) for s in ZOO_PARAM_SHAPES]
        got, loss = _grads_via_abi(be, None, params, x, y)
    assert abs(loss - float(loss_ref)) <= (1e-5 if dtype == "f32" else 2e-2) * abs(float(loss_ref))
    assert max(rel_err(a, b.numpy()) for a, b in zip(got, g_ref)) <= (1e-4 if dtype == "f32" else 4e-2)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_a_third_architecture_trains_like_the_oracle(dtype):
    """The Qwen3-style training graph (weighted RMSNorm, per-head q / k norm before RoPE, GQA, SwiGLU, plain cross
    entropy): no fused kernel knows it; the general front end runs it — gradients against the oracle, then a worker
    round of three AdamW steps (losses and parameters after the round)."""
    from pcp_b200.export import QwenConfig, qwen_forward_mlir
    from test_qwen_graph import qwen_batch, qwen_params
    cfg = QwenConfig(dtype=dtype)
    text = qwen_forward_mlir(cfg)
    mod = TrainingModule(text)
    f32 = dtype == "f32"
    params = qwen_params(cfg)
    ids, tg = qwen_batch(cfg)
    g_ref, loss_ref = mod.compute_gradients(params, ids, tg)
    dt = F32 if f32 else BF16
    master = params if f32 else [torch.from_numpy(helpers.bf16_bits_to_f32(helpers.f32_to_bf16_trunc_bits(p.numpy())).reshape(p.shape)) for p in params]
    tau = 3
    toks = helpers.uniform_tokens(tau * (cfg.batch * cfg.seq_len + 1), cfg.vocab, 7)
    conf = AdamConf(learning_rate=1e-3)
    rec = []
    d_ref, _, _, _ = inner_loop(mod, master, FifoU16(toks), tau, cfg.batch, cfg.seq_len, conf, record=rec)
    with Backend(0) as be:
        be.load_session(text)
        assert be.param_shapes() == [tuple(s) for s in cfg.param_shapes()]
        got, loss = _grads_via_abi(be, None, params, ids.numpy(), tg.numpy())
        be.set_adam(conf.learning_rate, conf.beta1, conf.beta2, conf.epsilon, conf.weight_decay, conf.max_grad_norm)
        blob = flat(master) if f32 else helpers.f32_to_bf16_trunc_bits(flat(master))
        be.worker_begin_round(tau, blob, param_dtype=dt)
        be.worker_set_tokens(toks)
        for _ in range(tau):
            be.worker_step()
        delta, losses = be.worker_end_round(tau, param_dtype=dt)
    assert abs(loss - float(loss_ref)) <= (1e-4 if f32 else 2e-2) * abs(float(loss_ref))
    worst = max(rel_err(a, b.numpy()) for a, b in zip(got, g_ref))
    l2 = max(float(np.linalg.norm(a - b.numpy()) / (np.linalg.norm(b.numpy()) + 1e-30)) for a, b in zip(got, g_ref))
    assert (worst <= 1e-4) if f32 else (l2 <= 4e-2 and worst <= 0.25), (worst, l2)
    np.testing.assert_allclose(losses, [r[0] for r in rec], rtol=1e-4 if f32 else 2e-2)
    dgpu = delta if f32 else helpers.bf16_bits_to_f32(delta)
    assert rel_err(flat(master) - dgpu, flat(master) - flat(d_ref)) <= (1e-4 if f32 else 2e-2)
