"""The oracle against the committed golden fixture (made from the reference's shipped graph) and, where the
reference tree is present, the exporter against the shipped graphs."""
import os

import numpy as np
import pytest
import torch

from helpers import flat, split
from oracle import sanitizer
from oracle.loader import ChunkExhausted, ChunkTooSmall, FifoU16
from oracle.optim import AdamConf
from oracle.worker import TrainingModule, inner_loop
from pcp_b200 import NanochatConfig, NanoGPTConfig, nanochat_forward_mlir, nanogpt_forward_mlir
from pcp_b200.export import rope_tables

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
REF = os.environ.get("PCP_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))
SMALL = NanochatConfig(vocab=65, d_model=64, n_layer=2, n_head=4, n_kv_head=4, seq_len=32, batch=64, dtype="f32")


def test_oracle_reproduces_golden_on_exported_graph():
    gold = np.load(os.path.join(GOLDEN, "nanochat_small.npz"))
    mod = TrainingModule(nanochat_forward_mlir(SMALL))
    params = [torch.from_numpy(p.copy()) for p in split(gold["params"], SMALL)]
    grads, loss = mod.compute_gradients(params, torch.from_numpy(gold["ids"]), torch.from_numpy(gold["targets"]))
    assert float(loss) == float(gold["loss"])
    np.testing.assert_array_equal(flat(grads), gold["grads"])
    deltas, _, _, _ = inner_loop(mod, params, FifoU16(gold["tokens"]), 2, 64, 32, AdamConf(learning_rate=1e-3))
    np.testing.assert_allclose(flat(deltas), gold["delta_after_2"], rtol=0, atol=0)


def test_fifo_batcher_exact():
    toks = np.arange(0, 40, dtype=np.uint16)
    ds = FifoU16(toks)
    x, y = ds.get_batch(2, 4)
    assert x.dtype == np.int64 and x.tolist() == [[0, 1, 2, 3], [4, 5, 6, 7]] and y.tolist() == [[1, 2, 3, 4], [5, 6, 7, 8]]
    x, y = ds.get_batch(2, 4)                       # the cursor moved by B*T+1, the boundary token is consumed
    assert x[0, 0] == 9 and y[-1, -1] == 17 and ds.cursor == 18
    with pytest.raises(ChunkTooSmall):
        FifoU16(toks[:8]).get_batch(2, 4)
    ds.cursor = 36
    with pytest.raises(ChunkExhausted):
        ds.get_batch(2, 4)


def test_sanitizer_patches():
    src = ("    %11 = stablehlo.divide %7, %10 : tensor<4x1xf32>\n"
           "    %12 = stablehlo.log %11 : tensor<4x1xf32>\n"
           "    %13 = stablehlo.logistic %12 : tensor<4x1xf32>\n"
           "    %c = stablehlo.constant dense<0xFF800000> : tensor<f32>\n")
    out = sanitizer.apply_stability_patches(src)
    assert "%safe_denom_0 = stablehlo.add %10, %eps_div_0 : tensor<4x1xf32>" in out
    assert "%11 = stablehlo.divide %7, %safe_denom_0 : tensor<4x1xf32>" in out
    assert "%12 = stablehlo.log %safe_log_1 : tensor<4x1xf32>" in out
    assert "%13 = stablehlo.logistic %12" in out            # not rewritten (the reference's substring match would)
    assert "-6.550400e+04" in sanitizer.sanitize_hex_floats(src)


def test_softmax_denominators_carry_the_guard():
    """Every forward divide and log of the exported graph is patched (softmax /sum, RMSNorm /d, soft-cap /15,
    loss /count): the sanitised loss differs from the raw one by the expected small amount."""
    cfg = NanochatConfig(vocab=65, d_model=32, n_layer=1, n_head=2, n_kv_head=2, seq_len=8, batch=2, dtype="f32")
    text = nanochat_forward_mlir(cfg)
    assert sanitizer.sanitize(text).count("%safe_denom_") // 2 == text.count("stablehlo.divide")
    g = torch.Generator().manual_seed(0)
    params = [torch.randn(s, generator=g) * 0.1 for s in cfg.param_shapes()]
    ids = torch.randint(0, 65, (2, 8), generator=g)
    a = TrainingModule(text, sanitize=True).forward(params, ids, ids)
    b = TrainingModule(text, sanitize=False).forward(params, ids, ids)
    assert 0 < abs(float(a) - float(b)) < 1e-3


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "models")), reason="reference tree not present")
@pytest.mark.parametrize("name,cfgd", [
    ("nanochat_small", dict(vocab=65, d_model=64, n_layer=2, n_head=4, n_kv_head=4, seq_len=32, batch=64, dtype="f32")),
    ("nanochat_smoke_d1_128", dict(vocab=65536, d_model=64, n_layer=1, n_head=4, n_kv_head=4, seq_len=128, batch=1, dtype="f32")),
])
def test_exporter_equals_shipped_graph(name, cfgd):
    cfg = NanochatConfig(**cfgd)
    shipped = TrainingModule(open(os.path.join(REF, "models", name + ".mlir")).read())
    mine = TrainingModule(nanochat_forward_mlir(cfg))
    assert shipped.param_shapes == mine.param_shapes
    g = torch.Generator().manual_seed(1)
    params = [torch.randn(s, generator=g) * 0.05 for s in cfg.param_shapes()]
    ids = torch.randint(0, cfg.vocab, (cfg.batch, cfg.seq_len), generator=g)
    tg = torch.randint(0, cfg.vocab, (cfg.batch, cfg.seq_len), generator=g)
    tg[0, :2] = -1
    ga, la = shipped.compute_gradients(params, ids, tg)
    gb, lb = mine.compute_gradients(params, ids, tg)
    assert float(la) == float(lb)
    for x, y in zip(ga, gb):
        assert torch.equal(x, y)
    cos, sin = rope_tables(cfg.seq_len, cfg.head_dim)
    blobs = sorted(shipped.fn.resources.items())
    assert [v for k, v in blobs if not k.endswith("_1")][0] == cos.astype("<u2").tobytes()
    assert [v for k, v in blobs if k.endswith("_1")][0] == sin.astype("<u2").tobytes()


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "models")), reason="reference tree not present")
def test_recorded_forward_loss_scale():
    """The reference records 4.3792643547 (PyTorch) vs 4.3792648315 (IREE llvm-cpu) for this graph with its own
    seeded nanochat weights (test/nanochat/test_generate_nanochat_mlir_forward_loss.py:27-32).  The weights come
    from the `nanochat` package, which is not part of the tree, so the number itself cannot be reproduced; the
    oracle is checked to give a loss in the same range (ln 65 = 4.174 for near-uniform logits)."""
    mod = TrainingModule(open(os.path.join(REF, "models", "nanochat_small.mlir")).read())
    g = torch.Generator().manual_seed(0)
    params = [torch.randn(s, generator=g) * 0.02 for s in mod.param_shapes]
    ids = torch.randint(0, 65, (64, 32), generator=g)
    loss = float(mod.forward(params, ids, ids))
    assert 4.0 < loss < 4.5


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "models")), reason="reference tree not present")
def test_nanogpt_exporter_equals_shipped_graph():
    """models/nanogpt_small.mlir (f32, LayerNorm variance in f64, ReLU MLP, lm_head bias, ignore_index -100): loss and
    all 22 gradients bit-identical between the shipped graph and the exporter's.  (The bf16 graph
    models/nanogpt_medium_bf16.mlir was checked the same way once; it takes 20 s on the CPU.)"""
    cfg = NanoGPTConfig(vocab=65, d_model=64, n_layer=2, n_head=4, seq_len=32, batch=64, dtype="f32")
    shipped = TrainingModule(open(os.path.join(REF, "models", "nanogpt_small.mlir")).read())
    mine = TrainingModule(nanogpt_forward_mlir(cfg))
    assert shipped.param_shapes == mine.param_shapes and cfg.num_params() == 109377
    g = torch.Generator().manual_seed(4)
    params = [torch.randn(s, generator=g) * 0.05 for s in cfg.param_shapes()]
    ids = torch.randint(0, 65, (64, 32), generator=g)
    tg = torch.randint(0, 65, (64, 32), generator=g)
    tg[1, :4] = -100
    ga, la = shipped.compute_gradients(params, ids, tg)
    gb, lb = mine.compute_gradients(params, ids, tg)
    assert float(la) == float(lb)
    for x, y in zip(ga, gb):
        assert torch.equal(x, y)
