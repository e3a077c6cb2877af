"""Forward-graph exporter for the nanochat model family (StableHLO text).

The reference gets its forward graphs by exporting PyTorch modules through torch_mlir
(tools/generate_nanochat.py) and ships the results as models/*.mlir; the worker artefact is
derived from that text.  Neither torch_mlir nor the `nanochat` package can be installed offline,
so for model shapes the reference does not ship this module writes the same graph directly:
same argument order (wte, per layer c_q c_k c_v c_proj c_fc mlp.c_proj, lm_head, idx, targets),
same op sequence and cast points per value as models/nanochat_small.mlir (f32) and
models/nanochat_d8_b8_t2048_bf16.mlir (bf16):

  x = norm(wte[idx]);  per layer: q,k,v = norm(x).W^T -> RoPE(half split, bf16 tables) ->
  norm(q), norm(k) -> GQA broadcast -> (q.k^T)*1/sqrt(hd) in model dtype -> causal select ->
  softmax in f32 -> model dtype -> .v -> c_proj -> +x ; norm -> c_fc -> max(.,0) -> power(.,2)
  -> c_proj -> +x ;  norm -> lm_head -> f32 -> 15*tanh(z/15) -> log-softmax -> NLL gather ->
  mean over targets != -1.

norm is the parameter-free RMSNorm: f32(x)^2 summed, /d, +1e-5, rsqrt, cast to model dtype,
multiply in model dtype.  SSA numbering and constant hoisting differ from torch_mlir's output;
values are identical op for op.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np


@dataclass
class NanochatConfig:
    vocab: int = 65
    d_model: int = 64
    n_layer: int = 2
    n_head: int = 4
    n_kv_head: int = 4
    seq_len: int = 32
    batch: int = 64
    dtype: str = "f32"            # "f32" | "bf16"
    rope_base: float = 10000.0
    softcap: int = 15
    mlp_ratio: int = 4

    @property
    def head_dim(self):
        return self.d_model // self.n_head

    @property
    def d_kv(self):
        return self.n_kv_head * self.head_dim

    def param_shapes(self):
        d, dkv, f = self.d_model, self.d_kv, self.mlp_ratio * self.d_model
        s = [(self.vocab, d)]
        for _ in range(self.n_layer):
            s += [(d, d), (dkv, d), (dkv, d), (d, d), (f, d), (d, f)]
        s.append((self.vocab, d))
        return s

    def num_params(self):
        return sum(a * b for a, b in self.param_shapes())


def rope_tables(seq_len: int, head_dim: int, base: float = 10000.0):
    """cos, sin of shape [seq_len, head_dim/2] as bf16 bit patterns (uint16), computed in f32 and
    rounded to nearest-even — the tables the exports embed as `dense_resource` blobs."""
    ch = np.arange(0, head_dim, 2, dtype=np.float32)
    inv_freq = (np.float32(1.0) / np.power(np.float32(base), ch / np.float32(head_dim))).astype(np.float32)
    t = np.arange(seq_len, dtype=np.float32)
    freqs = np.outer(t, inv_freq).astype(np.float32)
    return f32_to_bf16_rne(np.cos(freqs).astype(np.float32)), f32_to_bf16_rne(np.sin(freqs).astype(np.float32))


def f32_to_bf16_rne(x: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    return r


class _Emitter:
    def __init__(self):
        self.lines = []
        self.n = 0

    @staticmethod
    def ty(shape, dt):
        return "tensor<" + "".join(f"{s}x" for s in shape) + dt + ">"

    def emit(self, text, shape, dt, sig=None):
        name = f"%{self.n}"
        self.n += 1
        self.lines.append(f"    {name} = {text} : {sig if sig else self.ty(shape, dt)}")
        return (name, tuple(shape), dt)

    def const(self, lit, shape, dt, arith=False):
        op = "arith.constant" if arith else "stablehlo.constant"
        return self.emit(f"{op} dense<{lit}>", shape, dt)

    def resource(self, key, shape, dt):
        return self.emit(f"stablehlo.constant dense_resource<{key}>", shape, dt)

    def convert(self, x, dt):
        return self.emit(f"stablehlo.convert {x[0]}", x[1], dt, f"({self.ty(x[1], x[2])}) -> {self.ty(x[1], dt)}")

    def reshape(self, x, shape):
        return self.emit(f"stablehlo.reshape {x[0]}", shape, x[2], f"({self.ty(x[1], x[2])}) -> {self.ty(shape, x[2])}")

    def bcast(self, x, shape, dims):
        return self.emit(f"stablehlo.broadcast_in_dim {x[0]}, dims = [{', '.join(map(str, dims))}]", shape, x[2],
                         f"({self.ty(x[1], x[2])}) -> {self.ty(shape, x[2])}")

    def bin(self, op, a, b):
        assert a[1] == b[1] and a[2] == b[2], (op, a, b)
        return self.emit(f"stablehlo.{op} {a[0]}, {b[0]}", a[1], a[2])

    def un(self, op, a):
        return self.emit(f"stablehlo.{op} {a[0]}", a[1], a[2])

    def reduce(self, kind, x, init, dims):
        shape = tuple(s for i, s in enumerate(x[1]) if i not in dims)
        return self.emit(f"stablehlo.reduce({x[0]} init: {init[0]}) applies stablehlo.{kind} across dimensions = "
                         f"[{', '.join(map(str, dims))}]", shape, x[2],
                         f"({self.ty(x[1], x[2])}, {self.ty((), x[2])}) -> {self.ty(shape, x[2])}")

    def transpose(self, x, perm):
        shape = tuple(x[1][p] for p in perm)
        return self.emit(f"stablehlo.transpose {x[0]}, dims = [{', '.join(map(str, perm))}]", shape, x[2],
                         f"({self.ty(x[1], x[2])}) -> {self.ty(shape, x[2])}")

    def dot(self, a, b, batched=False):
        if batched:
            shape = (a[1][0], a[1][1], b[1][2])
            txt = f"stablehlo.dot_general {a[0]}, {b[0]}, batching_dims = [0] x [0], contracting_dims = [2] x [1]"
        else:
            shape = (a[1][0], b[1][1])
            txt = f"stablehlo.dot_general {a[0]}, {b[0]}, contracting_dims = [1] x [0]"
        return self.emit(txt, shape, a[2], f"({self.ty(a[1], a[2])}, {self.ty(b[1], b[2])}) -> {self.ty(shape, a[2])}")

    def slice(self, x, ranges):
        shape = tuple(b - a for a, b in ranges)
        return self.emit(f"stablehlo.slice {x[0]} [{', '.join(f'{a}:{b}' for a, b in ranges)}]", shape, x[2],
                         f"({self.ty(x[1], x[2])}) -> {self.ty(shape, x[2])}")

    def concat(self, a, b, dim):
        shape = list(a[1]); shape[dim] += b[1][dim]
        return self.emit(f"stablehlo.concatenate {a[0]}, {b[0]}, dim = {dim}", shape, a[2],
                         f"({self.ty(a[1], a[2])}, {self.ty(b[1], b[2])}) -> {self.ty(shape, a[2])}")

    def compare(self, d, a, b, kind="SIGNED"):
        return self.emit(f"stablehlo.compare  {d}, {a[0]}, {b[0]},  {kind}", a[1], "i1",
                         f"({self.ty(a[1], a[2])}, {self.ty(b[1], b[2])}) -> {self.ty(a[1], 'i1')}")

    def select(self, p, a, b):
        return self.emit(f"stablehlo.select {p[0]}, {a[0]}, {b[0]}", a[1], a[2],
                         f"{self.ty(p[1], 'i1')}, {self.ty(a[1], a[2])}")

    def iota(self, shape, dim):
        return self.emit(f"stablehlo.iota dim = {dim}", shape, "i64")

    def scalar(self, lit, src_dt, dt):
        """arith.constant tensor<1x..> -> convert -> reshape to a rank-0 tensor (the exporter's idiom)."""
        c = self.const(lit, (1,), src_dt, arith=True)
        if src_dt != dt:
            c = self.convert(c, dt)
        return self.reshape(c, ())

    def splat(self, scalar, shape):
        return self.bcast(scalar, shape, [])


def nanochat_forward_mlir(cfg: NanochatConfig) -> str:
    e = _Emitter()
    B, T, d, V = cfg.batch, cfg.seq_len, cfg.d_model, cfg.vocab
    H, Hkv, hd = cfg.n_head, cfg.n_kv_head, cfg.head_dim
    dkv, F, dt = cfg.d_kv, cfg.mlp_ratio * cfg.d_model, cfg.dtype
    M = B * T
    assert d % H == 0 and H % Hkv == 0 and hd % 2 == 0 and dt in ("f32", "bf16")
    shapes = cfg.param_shapes()
    nP = len(shapes)
    args = [f"%arg{i}: {e.ty(s, dt)}" for i, s in enumerate(shapes)]
    args += [f"%arg{nP}: {e.ty((B, T), 'i64')}", f"%arg{nP + 1}: {e.ty((B, T), 'i64')}"]
    P = [(f"%arg{i}", tuple(s), dt) for i, s in enumerate(shapes)]
    idx = (f"%arg{nP}", (B, T), "i64")
    tgt = (f"%arg{nP + 1}", (B, T), "i64")

    zero_f32 = e.const("0.000000e+00", (), "f32")
    ninf_f32 = e.const("0xFF800000", (), "f32")
    mask_fill = e.const("-6.553600e+04", (), "bf16") if dt == "bf16" else ninf_f32
    cos_t = e.resource("rope_cos", (1, T, 1, hd // 2), "bf16")
    sin_t = e.resource("rope_sin", (1, T, 1, hd // 2), "bf16")
    two_f32 = e.scalar("2", "i64", "f32")
    eps_f32 = e.scalar("1.000000e-05", "f64", "f32")

    def norm(x, width):
        """Parameter-free RMSNorm over the last dimension."""
        shp = x[1]
        xf = e.convert(x, "f32") if dt != "f32" else x
        sq = e.bin("power", xf, e.splat(two_f32, shp))
        s = e.reduce("add", sq, zero_f32, [len(shp) - 1])
        s = e.reshape(s, shp[:-1] + (1,))
        ms = e.bin("divide", s, e.splat(e.scalar(str(width), "i64", "f32"), s[1]))
        r = e.un("rsqrt", e.bin("add", ms, e.splat(eps_f32, s[1])))
        if dt != "f32":
            r = e.convert(r, dt)
        return e.bin("multiply", x, e.bcast(r, shp, list(range(len(shp)))))

    def linear(x2d, w):
        return e.dot(x2d, e.transpose(w, [1, 0]))

    def rope(x):
        nh = x[1][2]
        half = hd // 2
        x1 = e.slice(x, [(0, B), (0, T), (0, nh), (0, half)])
        x2 = e.slice(x, [(0, B), (0, T), (0, nh), (half, hd)])
        if dt == "bf16":
            c = e.bcast(cos_t, x1[1], [0, 1, 2, 3])
            s = e.bcast(sin_t, x1[1], [0, 1, 2, 3])
            ns = e.bcast(e.un("negate", sin_t), x1[1], [0, 1, 2, 3])
        else:
            c = e.bcast(e.convert(cos_t, dt), x1[1], [0, 1, 2, 3])
            s = e.bcast(e.convert(sin_t, dt), x1[1], [0, 1, 2, 3])
            ns = e.bcast(e.convert(e.un("negate", sin_t), dt), x1[1], [0, 1, 2, 3])
        y1 = e.bin("add", e.bin("multiply", x1, c), e.bin("multiply", x2, s))
        y2 = e.bin("add", e.bin("multiply", x1, ns), e.bin("multiply", x2, c))
        return e.concat(y1, y2, 3)

    # causal mask: j - i >= 1
    ar = e.iota((T,), 0)
    col = e.bcast(e.reshape(ar, (1, T)), (T, T), [0, 1])
    row = e.bcast(e.reshape(ar, (T, 1)), (T, T), [0, 1])
    mask2d = e.compare("GE", e.bin("subtract", col, row), e.const("1", (T, T), "i64"))
    mask = e.bcast(e.reshape(mask2d, (1, 1, T, T)), (B, H, T, T), [0, 1, 2, 3])
    fill = e.splat(mask_fill, (B, H, T, T))
    scale = e.scalar(repr(1.0 / math.sqrt(hd)), "f64", dt)

    gat = e.emit(
        f'"stablehlo.gather"({P[0][0]}, {idx[0]}) <{{dimension_numbers = #stablehlo.gather<offset_dims = [2], '
        f'collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = 2>, indices_are_sorted = false, '
        f'slice_sizes = array<i64: 1, {d}>}}>', (B, T, d), dt,
        f"({e.ty((V, d), dt)}, {e.ty((B, T), 'i64')}) -> {e.ty((B, T, d), dt)}")
    x = norm(gat, d)

    for l in range(cfg.n_layer):
        wq, wk, wv, wo, wfc, wpr = P[1 + 6 * l: 7 + 6 * l]
        h = e.reshape(norm(x, d), (M, d))
        q = e.reshape(e.reshape(linear(h, wq), (B, T, d)), (B, T, H, hd))
        k = e.reshape(e.reshape(linear(h, wk), (B, T, dkv)), (B, T, Hkv, hd))
        v = e.reshape(e.reshape(linear(h, wv), (B, T, dkv)), (B, T, Hkv, hd))
        q, k = rope(q), rope(k)
        q, k = norm(q, hd), norm(k, hd)
        q = e.transpose(q, [0, 2, 1, 3])
        k = e.transpose(k, [0, 2, 1, 3])
        v = e.transpose(v, [0, 2, 1, 3])
        if Hkv != H:
            g = H // Hkv
            k = e.reshape(e.bcast(e.reshape(k, (B, Hkv, 1, T, hd)), (B, Hkv, g, T, hd), [0, 1, 2, 3, 4]), (B, H, T, hd))
            v = e.reshape(e.bcast(e.reshape(v, (B, Hkv, 1, T, hd)), (B, Hkv, g, T, hd), [0, 1, 2, 3, 4]), (B, H, T, hd))
        kt = e.transpose(k, [0, 1, 3, 2])
        s = e.dot(e.reshape(q, (B * H, T, hd)), e.reshape(kt, (B * H, hd, T)), batched=True)
        s = e.bin("multiply", e.reshape(s, (B, H, T, T)), e.splat(scale, (B, H, T, T)))
        s = e.select(mask, fill, s)
        sf = e.convert(s, "f32") if dt != "f32" else s
        mx = e.reshape(e.reduce("maximum", sf, ninf_f32, [3]), (B, H, T, 1))
        ex = e.un("exponential", e.bin("subtract", sf, e.bcast(mx, (B, H, T, T), [0, 1, 2, 3])))
        sm = e.reshape(e.reduce("add", ex, zero_f32, [3]), (B, H, T, 1))
        p = e.bin("divide", ex, e.bcast(sm, (B, H, T, T), [0, 1, 2, 3]))
        if dt != "f32":
            p = e.convert(p, dt)
        o = e.dot(e.reshape(p, (B * H, T, T)), e.reshape(v, (B * H, T, hd)), batched=True)
        o = e.reshape(e.transpose(e.reshape(o, (B, H, T, hd)), [0, 2, 1, 3]), (B, T, d))
        x = e.bin("add", x, e.reshape(linear(e.reshape(o, (M, d)), wo), (B, T, d)))
        h = e.reshape(norm(x, d), (M, d))
        u = e.reshape(linear(h, wfc), (B, T, F))
        a = e.bin("maximum", u, e.const("0.000000e+00", (B, T, F), dt))
        a = e.bin("power", a, e.splat(e.scalar("2", "i64", dt), (B, T, F)))
        x = e.bin("add", x, e.reshape(linear(e.reshape(a, (M, F)), wpr), (B, T, d)))

    hf = e.reshape(norm(x, d), (M, d))
    z = e.reshape(linear(hf, P[-1]), (B, T, V))
    if dt != "f32":
        z = e.convert(z, "f32")
    cap = e.splat(e.scalar(str(cfg.softcap), "i64", "f32"), (B, T, V))
    z = e.bin("multiply", e.un("tanh", e.bin("divide", z, cap)), cap)
    z = e.reshape(z, (M, V))
    t1 = e.reshape(tgt, (M,))
    mx = e.bcast(e.reshape(e.reduce("maximum", z, ninf_f32, [1]), (M, 1)), (M, V), [0, 1])
    sh = e.bin("subtract", z, mx)
    se = e.reshape(e.reduce("add", e.un("exponential", sh), zero_f32, [1]), (M, 1))
    logp = e.bin("subtract", sh, e.bcast(e.un("log", se), (M, V), [0, 1]))
    valid = e.compare("NE", t1, e.const("-1", (M,), "i64"))
    safe_t = e.select(valid, t1, e.const("0", (M,), "i64"))
    ij = e.concat(e.iota((M, 1, 1), 0), e.reshape(e.reshape(safe_t, (M, 1)), (M, 1, 1)), 2)
    picked = e.emit(
        f'"stablehlo.gather"({logp[0]}, {ij[0]}) <{{dimension_numbers = #stablehlo.gather<collapsed_slice_dims = [0, 1], '
        f'start_index_map = [0, 1], index_vector_dim = 2>, slice_sizes = array<i64: 1, 1>}}>', (M, 1), "f32",
        f"({e.ty((M, V), 'f32')}, {e.ty((M, 1, 2), 'i64')}) -> {e.ty((M, 1), 'f32')}")
    nll = e.un("negate", e.reshape(picked, (M,)))
    nll = e.select(valid, nll, e.splat(zero_f32, (M,)))
    cnt = e.convert(e.reduce("add", e.convert(valid, "i64"), e.const("0", (), "i64"), [0]), "f32")
    tot = e.reduce("add", nll, zero_f32, [0])
    loss = e.bin("divide", tot, cnt)

    cos_b, sin_b = rope_tables(T, hd, cfg.rope_base)
    hdr = "02000000"
    out = ["module {", f"  func.func @main({', '.join(args)}) -> tensor<f32> {{"]
    out += e.lines
    out += [f"    return {loss[0]} : tensor<f32>", "  }", "}", "", "{-#", "  dialect_resources: {", "    builtin: {",
            f'      rope_sin: "0x{hdr}{sin_b.astype("<u2").tobytes().hex().upper()}",',
            f'      rope_cos: "0x{hdr}{cos_b.astype("<u2").tobytes().hex().upper()}"',
            "    }", "  }", "#-}", ""]
    return "\n".join(out)


# ------------------------------------------------------------------------------------------------
# nanoGPT family (tools/generate_nanogpt_small.py, tools/generate_nanogpt_medium_bf16.py)
# ------------------------------------------------------------------------------------------------
@dataclass
class NanoGPTConfig:
    vocab: int = 65
    d_model: int = 64
    n_layer: int = 2
    n_head: int = 4
    seq_len: int = 32
    batch: int = 64
    dtype: str = "f32"            # "f32" | "bf16"
    mlp_ratio: int = 4
    activation: str = "relu"      # "relu" (the shipped graphs) | "gelu" (tanh approximation; no shipped graph has it)

    @property
    def head_dim(self):
        return self.d_model // self.n_head

    def param_shapes(self):
        d, f = self.d_model, self.mlp_ratio * self.d_model
        s = [(self.vocab, d), (self.seq_len, d)]
        for _ in range(self.n_layer):
            s += [(d,), (d,), (3 * d, d), (d, d), (d,), (d,), (f, d), (d, f)]
        s += [(d,), (d,), (self.vocab, d), (self.vocab,)]
        return s

    def num_params(self):
        return int(sum(int(np.prod(x)) for x in self.param_shapes()))


def nanogpt_forward_mlir(cfg: NanoGPTConfig) -> str:
    """Forward graph of the nanoGPT family with the op sequence and cast points of models/nanogpt_small.mlir (f32)
    and models/nanogpt_medium_bf16.mlir (bf16): learned token + position embeddings, pre-LayerNorm whose variance
    is computed in f64, fused qkv projection split on the last dim, causal softmax (f32), ReLU MLP, final
    LayerNorm, lm_head with bias computed in f32, cross entropy ignoring targets == -100."""
    e = _Emitter()
    B, T, d, V, H, hd = cfg.batch, cfg.seq_len, cfg.d_model, cfg.vocab, cfg.n_head, cfg.head_dim
    F, dt, M = cfg.mlp_ratio * d, cfg.dtype, cfg.batch * cfg.seq_len
    assert d % H == 0 and dt in ("f32", "bf16")
    shapes = cfg.param_shapes()
    nP = len(shapes)
    args = [f"%arg{i}: {e.ty(s, dt)}" for i, s in enumerate(shapes)]
    args += [f"%arg{nP}: {e.ty((B, T), 'i64')}", f"%arg{nP + 1}: {e.ty((B, T), 'i64')}"]
    P = [(f"%arg{i}", tuple(s), dt) for i, s in enumerate(shapes)]
    idx = (f"%arg{nP}", (B, T), "i64")
    tgt = (f"%arg{nP + 1}", (B, T), "i64")

    zero_f32 = e.const("0.000000e+00", (), "f32")
    zero_f64 = e.const("0.000000e+00", (), "f64")
    ninf_f32 = e.const("0xFF800000", (), "f32")
    mask_fill = e.const("-6.553600e+04", (), "bf16") if dt == "bf16" else ninf_f32
    eps_f32 = e.scalar("1.000000e-05", "f64", "f32")
    d_f64 = e.splat(e.scalar(str(d), "i64", "f64"), (B, T, 1))
    d_f32 = e.splat(e.scalar(str(d), "i64", "f32"), (B, T, 1))

    def layernorm(x, w, b):
        xf = e.convert(x, "f32") if dt != "f32" else x
        x64 = e.convert(xf, "f64")
        mean64 = e.bin("divide", e.reshape(e.reduce("add", x64, zero_f64, [2]), (B, T, 1)), d_f64)
        c64 = e.bin("subtract", x64, e.bcast(mean64, (B, T, d), [0, 1, 2]))
        var64 = e.bin("divide", e.reshape(e.reduce("add", e.bin("multiply", c64, c64), zero_f64, [2]), (B, T, 1)), d_f64)
        var = e.convert(var64, "f32")
        mean = e.bin("divide", e.reshape(e.reduce("add", xf, zero_f32, [2]), (B, T, 1)), d_f32)
        r = e.un("rsqrt", e.bin("add", var, e.splat(eps_f32, (B, T, 1))))
        y = e.bin("multiply", e.bin("subtract", xf, e.bcast(mean, (B, T, d), [0, 1, 2])), e.bcast(r, (B, T, d), [0, 1, 2]))
        wf = e.convert(w, "f32") if dt != "f32" else w
        bf = e.convert(b, "f32") if dt != "f32" else b
        y = e.bin("add", e.bin("multiply", y, e.bcast(wf, (B, T, d), [2])), e.bcast(bf, (B, T, d), [2]))
        return e.convert(y, dt) if dt != "f32" else y

    def linear(x2d, w):
        return e.dot(x2d, e.transpose(w, [1, 0]))

    def gather_rows(table, indices, out_shape, offset_dim, ivd):
        rows, width = table[1]
        return e.emit(
            f'"stablehlo.gather"({table[0]}, {indices[0]}) <{{dimension_numbers = #stablehlo.gather<offset_dims = [{offset_dim}], '
            f'collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = {ivd}>, indices_are_sorted = false, '
            f'slice_sizes = array<i64: 1, {width}>}}>', out_shape, table[2],
            f"({e.ty(table[1], table[2])}, {e.ty(indices[1], 'i64')}) -> {e.ty(out_shape, table[2])}")

    tok = gather_rows(P[0], idx, (B, T, d), 2, 2)
    pos = gather_rows(P[1], e.iota((T,), 0), (T, d), 1, 1)
    x = e.bin("add", tok, e.bcast(pos, (B, T, d), [1, 2]))

    # masked_fill(tril == 0, fill): tril[i, j] = 1 where j <= i
    tril = e.select(e.compare("LE", e.iota((T, T), 1), e.iota((T, T), 0)), e.const("1.000000e+00", (T, T), "f32"),
                    e.const("0.000000e+00", (T, T), "f32"))
    m4 = e.compare("EQ", e.reshape(tril, (1, 1, T, T)), e.splat(zero_f32, (1, 1, T, T)), kind="FLOAT")
    mask = e.bcast(m4, (B, H, T, T), [0, 1, 2, 3])
    fill = e.splat(mask_fill, (B, H, T, T))
    scale = e.scalar(repr(1.0 / math.sqrt(hd)), "f64", dt)

    for l in range(cfg.n_layer):
        ln1w, ln1b, wqkv, wo, ln2w, ln2b, wfc, wpr = P[2 + 8 * l: 10 + 8 * l]
        h = e.reshape(layernorm(x, ln1w, ln1b), (M, d))
        qkv = e.reshape(linear(h, wqkv), (B, T, 3 * d))
        q = e.slice(qkv, [(0, B), (0, T), (0, d)])
        k = e.slice(qkv, [(0, B), (0, T), (d, 2 * d)])
        v = e.slice(qkv, [(0, B), (0, T), (2 * d, 3 * d)])
        heads = lambda t: e.transpose(e.reshape(t, (B, T, H, hd)), [0, 2, 1, 3])
        k, q, v = heads(k), heads(q), heads(v)
        kt = e.transpose(k, [0, 1, 3, 2])
        s = e.dot(e.reshape(q, (B * H, T, hd)), e.reshape(kt, (B * H, hd, T)), batched=True)
        s = e.bin("multiply", e.reshape(s, (B, H, T, T)), e.splat(scale, (B, H, T, T)))
        s = e.select(mask, fill, s)
        sf = e.convert(s, "f32") if dt != "f32" else s
        mx = e.reshape(e.reduce("maximum", sf, ninf_f32, [3]), (B, H, T, 1))
        ex = e.un("exponential", e.bin("subtract", sf, e.bcast(mx, (B, H, T, T), [0, 1, 2, 3])))
        sm = e.reshape(e.reduce("add", ex, zero_f32, [3]), (B, H, T, 1))
        p = e.bin("divide", ex, e.bcast(sm, (B, H, T, T), [0, 1, 2, 3]))
        if dt != "f32":
            p = e.convert(p, dt)
        o = e.dot(e.reshape(p, (B * H, T, T)), e.reshape(v, (B * H, T, hd)), batched=True)
        o = e.reshape(e.transpose(e.reshape(o, (B, H, T, hd)), [0, 2, 1, 3]), (B, T, d))
        x = e.bin("add", x, e.reshape(linear(e.reshape(o, (M, d)), wo), (B, T, d)))
        h = e.reshape(layernorm(x, ln2w, ln2b), (M, d))
        u = e.reshape(linear(h, wfc), (B, T, F))
        if cfg.activation == "gelu":
            # 0.5 * u * (1 + tanh(sqrt(2/pi) * (u + 0.044715 * u^3))), the cube as two multiplies; literals are
            # the f32 values of the two constants to nine digits (the recogniser keys on them)
            x3 = e.bin("multiply", e.bin("multiply", u, u), u)
            s_ = e.bin("add", u, e.bin("multiply", e.const("4.47149985e-02", (B, T, F), dt), x3))
            t = e.un("tanh", e.bin("multiply", e.const("7.97884583e-01", (B, T, F), dt), s_))
            p1 = e.bin("add", t, e.const("1.000000e+00", (B, T, F), dt))
            a = e.bin("multiply", e.bin("multiply", e.const("5.000000e-01", (B, T, F), dt), u), p1)
        elif cfg.activation == "relu":
            a = e.bin("maximum", u, e.const("0.000000e+00", (B, T, F), dt))
        else:
            raise ValueError(f"unknown activation {cfg.activation!r}")
        x = e.bin("add", x, e.reshape(linear(e.reshape(a, (M, F)), wpr), (B, T, d)))

    lnfw, lnfb, wh, bh = P[-4:]
    hf = e.reshape(layernorm(x, lnfw, lnfb), (M, d))
    wt = e.transpose(wh, [1, 0])
    if dt != "f32":                                   # the head runs in f32 (addmm on upcast operands), result -> bf16 -> f32
        bhf = e.convert(bh, "f32")
        z = e.dot(e.convert(hf, "f32"), e.convert(wt, "f32"))
    else:
        bhf = bh
        z = e.dot(hf, wt)
    one = e.scalar("1", "i64", "f32")
    z = e.bin("multiply", z, e.splat(one, (M, V)))
    z = e.bin("add", z, e.bcast(e.bin("multiply", bhf, e.splat(one, (V,))), (M, V), [1]))
    if dt != "f32":
        z = e.convert(e.convert(z, dt), "f32")
    t1 = e.reshape(tgt, (M,))
    mx = e.bcast(e.reshape(e.reduce("maximum", z, ninf_f32, [1]), (M, 1)), (M, V), [0, 1])
    sh = e.bin("subtract", z, mx)
    se = e.reshape(e.reduce("add", e.un("exponential", sh), zero_f32, [1]), (M, 1))
    logp = e.bin("subtract", sh, e.bcast(e.un("log", se), (M, V), [0, 1]))
    valid = e.compare("NE", t1, e.const("-100", (M,), "i64"))
    safe_t = e.select(valid, t1, e.const("0", (M,), "i64"))
    ij = e.concat(e.iota((M, 1, 1), 0), e.reshape(e.reshape(safe_t, (M, 1)), (M, 1, 1)), 2)
    picked = e.emit(
        f'"stablehlo.gather"({logp[0]}, {ij[0]}) <{{dimension_numbers = #stablehlo.gather<collapsed_slice_dims = [0, 1], '
        f'start_index_map = [0, 1], index_vector_dim = 2>, slice_sizes = array<i64: 1, 1>}}>', (M, 1), "f32",
        f"({e.ty((M, V), 'f32')}, {e.ty((M, 1, 2), 'i64')}) -> {e.ty((M, 1), 'f32')}")
    nll = e.select(valid, e.un("negate", e.reshape(picked, (M,))), e.splat(zero_f32, (M,)))
    cnt = e.convert(e.reduce("add", e.convert(valid, "i64"), e.const("0", (), "i64"), [0]), "f32")
    loss = e.bin("divide", e.reduce("add", nll, zero_f32, [0]), cnt)
    out = ["module {", f"  func.func @main({', '.join(args)}) -> tensor<f32> {{"]
    out += e.lines
    out += [f"    return {loss[0]} : tensor<f32>", "  }", "}", ""]
    return "\n".join(out)


# ------------------------------------------------------------------------------------------------
# Qwen3-style decoder (the architecture of tools/export_qwen3_generation.py, as a training graph)
# ------------------------------------------------------------------------------------------------
@dataclass
class QwenConfig:
    """A third architecture, neither of the two families the fused kernels cover: RMSNorm with a weight, q / k
    normalised per head with a weight BEFORE RoPE, grouped-query attention, SwiGLU MLP, plain cross entropy with
    ignore index -100.  The reference exports this model for generation only (tools/export_qwen3_generation.py wraps
    Qwen3ForCausalLM for the rollout workers); as a forward graph (params..., ids, targets) -> loss it is what the
    Shepherd would hand to workers to fine-tune that model, and it runs through the general front end."""
    vocab: int = 97
    d_model: int = 64
    n_layer: int = 2
    n_head: int = 4
    n_kv_head: int = 2
    head_dim: int = 16
    d_ff: int = 128
    seq_len: int = 32
    batch: int = 4
    dtype: str = "f32"            # "f32" | "bf16"
    rope_base: float = 10000.0
    eps: float = 1e-6

    def param_shapes(self):
        d, hq, hk, f = self.d_model, self.n_head * self.head_dim, self.n_kv_head * self.head_dim, self.d_ff
        s = [(self.vocab, d)]
        for _ in range(self.n_layer):
            s += [(d,), (hq, d), (hk, d), (hk, d), (self.head_dim,), (self.head_dim,), (d, hq), (d,), (f, d), (f, d), (d, f)]
        s += [(d,), (self.vocab, d)]
        return s

    def num_params(self):
        return int(sum(int(np.prod(x)) for x in self.param_shapes()))


def qwen_forward_mlir(cfg: QwenConfig) -> str:
    """Forward graph: x = embed[ids]; per layer  h = rms(x, ln1); q, k, v = h W^T; q = rope(rms_head(q, q_norm)),
    k = rope(rms_head(k, k_norm)); causal softmax attention (f32 softmax, GQA by broadcasting k / v); x += o W_o^T;
    h = rms(x, ln2); x += (silu(h W_gate^T) * (h W_up^T)) W_down^T;  logits = rms(x, norm) lm_head^T in f32;
    mean NLL over targets != -100.  rms(x, w) = w * (x * rsqrt(mean(x^2) + eps)) with the statistics in f32."""
    e = _Emitter()
    B, T, d, V = cfg.batch, cfg.seq_len, cfg.d_model, cfg.vocab
    H, Hkv, hd, F, dt = cfg.n_head, cfg.n_kv_head, cfg.head_dim, cfg.d_ff, cfg.dtype
    hq, hk, M = H * hd, Hkv * hd, B * T
    assert H % Hkv == 0 and hd % 2 == 0 and dt in ("f32", "bf16")
    shapes = cfg.param_shapes()
    nP = len(shapes)
    args = [f"%arg{i}: {e.ty(s, dt)}" for i, s in enumerate(shapes)]
    args += [f"%arg{nP}: {e.ty((B, T), 'i64')}", f"%arg{nP + 1}: {e.ty((B, T), 'i64')}"]
    P = [(f"%arg{i}", tuple(s), dt) for i, s in enumerate(shapes)]
    idx = (f"%arg{nP}", (B, T), "i64")
    tgt = (f"%arg{nP + 1}", (B, T), "i64")

    zero_f32 = e.const("0.000000e+00", (), "f32")
    ninf_f32 = e.const("0xFF800000", (), "f32")
    mask_fill = e.const("-6.553600e+04", (), "bf16") if dt == "bf16" else ninf_f32
    cos_t = e.resource("rope_cos", (1, T, 1, hd // 2), "bf16")
    sin_t = e.resource("rope_sin", (1, T, 1, hd // 2), "bf16")
    two_f32 = e.scalar("2", "i64", "f32")
    eps_f32 = e.scalar(repr(cfg.eps), "f64", "f32")

    def rms(x, w, width):
        """RMSNorm over the last dimension with the weight w [width]."""
        shp = x[1]
        xf = e.convert(x, "f32") if dt != "f32" else x
        s = e.reduce("add", e.bin("power", xf, e.splat(two_f32, shp)), zero_f32, [len(shp) - 1])
        s = e.reshape(s, shp[:-1] + (1,))
        ms = e.bin("divide", s, e.splat(e.scalar(str(width), "i64", "f32"), s[1]))
        r = e.un("rsqrt", e.bin("add", ms, e.splat(eps_f32, s[1])))
        y = e.bin("multiply", xf, e.bcast(r, shp, list(range(len(shp)))))
        if dt != "f32":
            y = e.convert(y, dt)
        return e.bin("multiply", e.bcast(w, shp, [len(shp) - 1]), y)

    def linear(x2d, w):
        return e.dot(x2d, e.transpose(w, [1, 0]))

    def rope(x):
        nh, half = x[1][2], hd // 2
        x1 = e.slice(x, [(0, B), (0, T), (0, nh), (0, half)])
        x2 = e.slice(x, [(0, B), (0, T), (0, nh), (half, hd)])
        cv = (lambda t: t) if dt == "bf16" else (lambda t: e.convert(t, dt))
        c = e.bcast(cv(cos_t), x1[1], [0, 1, 2, 3])
        s = e.bcast(cv(sin_t), x1[1], [0, 1, 2, 3])
        # rotate_half: (x1, x2) -> (x1 cos - x2 sin, x2 cos + x1 sin)
        y1 = e.bin("subtract", e.bin("multiply", x1, c), e.bin("multiply", x2, s))
        y2 = e.bin("add", e.bin("multiply", x2, c), e.bin("multiply", x1, s))
        return e.concat(y1, y2, 3)

    ar = e.iota((T,), 0)
    col = e.bcast(e.reshape(ar, (1, T)), (T, T), [0, 1])
    row = e.bcast(e.reshape(ar, (T, 1)), (T, T), [0, 1])
    mask2d = e.compare("GT", col, row)
    mask = e.bcast(e.reshape(mask2d, (1, 1, T, T)), (B, H, T, T), [0, 1, 2, 3])
    fill = e.splat(mask_fill, (B, H, T, T))
    scale = e.scalar(repr(1.0 / math.sqrt(hd)), "f64", dt)

    x = e.emit(
        f'"stablehlo.gather"({P[0][0]}, {idx[0]}) <{{dimension_numbers = #stablehlo.gather<offset_dims = [2], '
        f'collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = 2>, indices_are_sorted = false, '
        f'slice_sizes = array<i64: 1, {d}>}}>', (B, T, d), dt,
        f"({e.ty((V, d), dt)}, {e.ty((B, T), 'i64')}) -> {e.ty((B, T, d), dt)}")

    for l in range(cfg.n_layer):
        ln1, wq, wk, wv, qn, kn, wo, ln2, wg, wu, wd = P[1 + 11 * l: 12 + 11 * l]
        h = e.reshape(rms(x, ln1, d), (M, d))
        q = e.reshape(linear(h, wq), (B, T, H, hd))
        k = e.reshape(linear(h, wk), (B, T, Hkv, hd))
        v = e.reshape(linear(h, wv), (B, T, Hkv, hd))
        q, k = rope(rms(q, qn, hd)), rope(rms(k, kn, hd))
        q = e.transpose(q, [0, 2, 1, 3])
        k = e.transpose(k, [0, 2, 1, 3])
        v = e.transpose(v, [0, 2, 1, 3])
        if Hkv != H:
            g = H // Hkv
            k = e.reshape(e.bcast(e.reshape(k, (B, Hkv, 1, T, hd)), (B, Hkv, g, T, hd), [0, 1, 2, 3, 4]), (B, H, T, hd))
            v = e.reshape(e.bcast(e.reshape(v, (B, Hkv, 1, T, hd)), (B, Hkv, g, T, hd), [0, 1, 2, 3, 4]), (B, H, T, hd))
        kt = e.transpose(k, [0, 1, 3, 2])
        s = e.dot(e.reshape(q, (B * H, T, hd)), e.reshape(kt, (B * H, hd, T)), batched=True)
        s = e.bin("multiply", e.reshape(s, (B, H, T, T)), e.splat(scale, (B, H, T, T)))
        s = e.select(mask, fill, s)
        sf = e.convert(s, "f32") if dt != "f32" else s
        mx = e.reshape(e.reduce("maximum", sf, ninf_f32, [3]), (B, H, T, 1))
        ex = e.un("exponential", e.bin("subtract", sf, e.bcast(mx, (B, H, T, T), [0, 1, 2, 3])))
        sm = e.reshape(e.reduce("add", ex, zero_f32, [3]), (B, H, T, 1))
        p = e.bin("divide", ex, e.bcast(sm, (B, H, T, T), [0, 1, 2, 3]))
        if dt != "f32":
            p = e.convert(p, dt)
        o = e.dot(e.reshape(p, (B * H, T, T)), e.reshape(v, (B * H, T, hd)), batched=True)
        o = e.reshape(e.transpose(e.reshape(o, (B, H, T, hd)), [0, 2, 1, 3]), (M, hq))
        x = e.bin("add", x, e.reshape(linear(o, wo), (B, T, d)))
        h = e.reshape(rms(x, ln2, d), (M, d))
        gate, up = linear(h, wg), linear(h, wu)
        act = e.bin("multiply", e.bin("multiply", gate, e.un("logistic", gate)), up)       # silu(gate) * up
        x = e.bin("add", x, e.reshape(linear(act, wd), (B, T, d)))

    hf = e.reshape(rms(x, P[-2], d), (M, d))
    z = linear(hf, P[-1])
    if dt != "f32":
        z = e.convert(z, "f32")
    t1 = e.reshape(tgt, (M,))
    mx = e.bcast(e.reshape(e.reduce("maximum", z, ninf_f32, [1]), (M, 1)), (M, V), [0, 1])
    sh = e.bin("subtract", z, mx)
    se = e.reshape(e.reduce("add", e.un("exponential", sh), zero_f32, [1]), (M, 1))
    logp = e.bin("subtract", sh, e.bcast(e.un("log", se), (M, V), [0, 1]))
    valid = e.compare("NE", t1, e.const("-100", (M,), "i64"))
    safe_t = e.select(valid, t1, e.const("0", (M,), "i64"))
    ij = e.concat(e.iota((M, 1, 1), 0), e.reshape(e.reshape(safe_t, (M, 1)), (M, 1, 1)), 2)
    picked = e.emit(
        f'"stablehlo.gather"({logp[0]}, {ij[0]}) <{{dimension_numbers = #stablehlo.gather<collapsed_slice_dims = [0, 1], '
        f'start_index_map = [0, 1], index_vector_dim = 2>, slice_sizes = array<i64: 1, 1>}}>', (M, 1), "f32",
        f"({e.ty((M, V), 'f32')}, {e.ty((M, 1, 2), 'i64')}) -> {e.ty((M, 1), 'f32')}")
    nll = e.select(valid, e.un("negate", e.reshape(picked, (M,))), e.splat(zero_f32, (M,)))
    cnt = e.convert(e.reduce("add", e.convert(valid, "i64"), e.const("0", (), "i64"), [0]), "f32")
    loss = e.bin("divide", e.reduce("add", nll, zero_f32, [0]), cnt)

    cos_b, sin_b = rope_tables(T, hd, cfg.rope_base)
    hdr = "02000000"
    out = ["module {", f"  func.func @main({', '.join(args)}) -> tensor<f32> {{"]
    out += e.lines
    out += [f"    return {loss[0]} : tensor<f32>", "  }", "}", "", "{-#", "  dialect_resources: {", "    builtin: {",
            f'      rope_sin: "0x{hdr}{sin_b.astype("<u2").tobytes().hex().upper()}",',
            f'      rope_cos: "0x{hdr}{cos_b.astype("<u2").tobytes().hex().upper()}"',
            "    }", "  }", "#-}", ""]
    return "\n".join(out)
