"""Shared helpers of the test-suite: seeded inputs and the oracle-side replay."""
import numpy as np
import torch

from oracle.loader import FifoU16, uniform_tokens, zipf_tokens
from oracle.optim import AdamConf, NesterovConf
from oracle.worker import TrainingModule, inner_loop, outer_step
from pcp_b200.export import NanochatConfig, NanoGPTConfig, nanochat_forward_mlir, nanogpt_forward_mlir

SMALL_F32 = dict(vocab=65, d_model=64, n_layer=2, n_head=4, n_kv_head=4, seq_len=32, batch=8, dtype="f32")
GQA_F32 = dict(vocab=97, d_model=64, n_layer=2, n_head=4, n_kv_head=2, seq_len=24, batch=3, dtype="f32")
SMALL_BF16 = dict(vocab=65, d_model=64, n_layer=2, n_head=4, n_kv_head=4, seq_len=32, batch=8, dtype="bf16")
HD128_BF16 = dict(vocab=512, d_model=256, n_layer=2, n_head=2, n_kv_head=2, seq_len=128, batch=2, dtype="bf16")
HD128_GQA_BF16 = dict(vocab=512, d_model=512, n_layer=1, n_head=4, n_kv_head=2, seq_len=256, batch=1, dtype="bf16")
# 160 (batch x head x row tile) work items: more than the 148 SMs, so the persistent attention kernels take several
# items per CTA (resident-tile reload and accumulator hand-over between items)
HD128_MANY_BF16 = dict(vocab=512, d_model=256, n_layer=1, n_head=2, n_kv_head=2, seq_len=256, batch=40, dtype="bf16")
# head dim 64 (what the nanoGPT configurations of the baseline use): the mma.sync tiled attention kernels, GQA
HD64_GQA_BF16 = dict(vocab=512, d_model=256, n_layer=2, n_head=4, n_kv_head=2, seq_len=256, batch=2, dtype="bf16")
# 32-wide heads, 8 query / 4 kv heads: the head layout of the shipped models/nanochat_d8_b*_t2048_bf16.mlir graphs; and
# 16-wide heads (the shipped f32 test graphs' layout, here in bf16)
HD32_GQA_BF16 = dict(vocab=512, d_model=256, n_layer=2, n_head=8, n_kv_head=4, seq_len=256, batch=2, dtype="bf16")
HD16_BF16 = dict(vocab=512, d_model=64, n_layer=1, n_head=4, n_kv_head=4, seq_len=128, batch=2, dtype="bf16")
# The kernel shapes of BASELINE config 3 (nanochat d20: d_model 1280, 10 heads x 128, T = 2048, vocabulary 65536) at two
# layers and batch 1: the two-CTA GEMM at K = 1280 / 5120 and N = 65536 with grouped tile order and split-K, the
# tcgen05 attention with 16 row tiles per head, the loss kernel over 65536-wide rows, the vector-reduction embedding
# scatter under Zipf tokens.  The oracle needs about two minutes and 25 GB of host memory for it.
D20_SHAPES_BF16 = dict(vocab=65536, d_model=1280, n_layer=2, n_head=10, n_kv_head=10, seq_len=2048, batch=1, dtype="bf16")
HD128_F32 = dict(vocab=512, d_model=256, n_layer=1, n_head=2, n_kv_head=1, seq_len=64, batch=2, dtype="f32")
# f32 with 64-wide heads, T a multiple of 64 and GEMM dimensions that are multiples of 128: the tiled f32 attention
# kernels (two query tiles per head, grouped-query heads) and the split-operand tensor-core GEMM path
HD64_F32 = dict(vocab=512, d_model=256, n_layer=2, n_head=4, n_kv_head=2, seq_len=128, batch=2, dtype="f32")
# the other head widths of the tiled f32 attention: 32 (grouped-query) and 16 (the shipped f32 nanochat graphs' widths)
HD32_F32 = dict(vocab=512, d_model=128, n_layer=1, n_head=4, n_kv_head=2, seq_len=128, batch=2, dtype="f32")
HD16_F32 = dict(vocab=256, d_model=64, n_layer=1, n_head=4, n_kv_head=4, seq_len=64, batch=2, dtype="f32")


GPT_SMALL_F32 = dict(vocab=65, d_model=64, n_layer=2, n_head=4, seq_len=32, batch=8, dtype="f32")
GPT_ODD_F32 = dict(vocab=97, d_model=48, n_layer=1, n_head=3, seq_len=20, batch=3, dtype="f32")
GPT_SMALL_BF16 = dict(vocab=256, d_model=64, n_layer=2, n_head=4, seq_len=32, batch=4, dtype="bf16")
# tanh-GELU MLP (the activation the larger nanoGPT configurations name; no shipped graph has it).  The bf16 one is
# sized for the tensor-core GEMM path (every GEMM dimension a multiple of 128) and the tiled attention (head dim 64).
GPT_GELU_F32 = dict(GPT_SMALL_F32, activation="gelu")
GPT_GELU_BF16 = dict(vocab=256, d_model=256, n_layer=2, n_head=4, seq_len=128, batch=4, dtype="bf16", activation="gelu")
# d_model a multiple of 256: the vectorised LayerNorm backward, f32
GPT_D256_F32 = dict(vocab=97, d_model=256, n_layer=1, n_head=4, seq_len=32, batch=4, dtype="f32")
# nanoGPT-small's kernel shapes in small (the fp32 benchmark configuration: 64-wide heads): tiled f32 attention over three query
# tiles, split-operand tensor-core GEMMs, GELU
# the shipped models/nanogpt_medium.mlir layout in small: f32, 8 heads x 32
GPT_HD32_F32 = dict(vocab=256, d_model=256, n_layer=1, n_head=8, seq_len=128, batch=2, dtype="f32")
GPT_HD64_F32 = dict(vocab=65, d_model=128, n_layer=2, n_head=2, seq_len=192, batch=2, dtype="f32", activation="gelu")


def make_model(cfgd):
    """(config, forward graph text) of either family; nanoGPT configs have no n_kv_head."""
    if "n_kv_head" in cfgd:
        cfg = NanochatConfig(**cfgd)
        return cfg, nanochat_forward_mlir(cfg)
    cfg = NanoGPTConfig(**cfgd)
    return cfg, nanogpt_forward_mlir(cfg)


def seeded_params(cfg, seed=0, std=0.02):
    g = torch.Generator().manual_seed(seed)
    out = []
    for s in cfg.param_shapes():
        p = torch.randn(s, generator=g) * std
        if len(s) == 1 and isinstance(cfg, NanoGPTConfig):
            p = p + 1.0 if len(out) % 2 == 0 else p        # LayerNorm weights near 1 (even slots are .w in every group)
        out.append(p)
    return out


def flat(ts):
    return np.concatenate([np.asarray(t, dtype=np.float32).reshape(-1) if not torch.is_tensor(t)
                           else t.detach().to(torch.float32).reshape(-1).numpy() for t in ts])


def split(flat_arr, cfg):
    out, at = [], 0
    for s in cfg.param_shapes():
        n = int(np.prod(s))
        out.append(flat_arr[at:at + n].reshape(s))
        at += n
    return out


def rel_err(a, b):
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-30))


def tokens_for(cfg, steps, seed, zipf=False):
    n = steps * (cfg.batch * cfg.seq_len + 1)
    return zipf_tokens(n, cfg.vocab, 1.1, seed) if zipf else uniform_tokens(n, cfg.vocab, seed)


def f32_to_bf16_trunc_bits(x):
    return (np.ascontiguousarray(x, np.float32).view(np.uint32) >> 16).astype(np.uint16)


def bf16_bits_to_f32(u):
    return (np.ascontiguousarray(u, np.uint16).astype(np.uint32) << 16).view(np.float32)
