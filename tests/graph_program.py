"""Reads the tensor program the library's general StableHLO front end prints (pcpb_graph_describe) and evaluates it
with torch on the CPU.  Test infrastructure: it lets the CPU suite compare the program — forward ops, stability
patches, gradient rules, adjoint edges — with the oracle's interpretation of the same graph without a GPU."""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from oracle import stablehlo as hlo

DT = {"f32": torch.float32, "f64": torch.float64, "bf16": torch.bfloat16, "i64": torch.int64, "i32": torch.int32,
      "i1": torch.bool}
KINDS = ["const_splat", "const_data", "iota", "unary", "binary", "compare", "select", "convert", "reshape", "transpose",
         "bcast", "slice", "concat", "reduce", "dot", "gather_rows", "gather2", "pad", "scatter_rows", "scatter2",
         "guard_clamp", "seed"]
UNARY = [torch.rsqrt, torch.sqrt, torch.exp, torch.log, torch.tanh, torch.sigmoid, torch.neg, torch.ceil, torch.floor,
         torch.sin, torch.cos, torch.abs]
CMP = [torch.eq, torch.ne, torch.ge, torch.gt, torch.le, torch.lt]


@dataclass
class Val:
    dtype: str
    shape: tuple
    name: str


@dataclass
class Op:
    kind: str
    sub: int
    out: int
    ins: list
    a: list
    b: list
    c: list
    d: list
    f: float
    i: int
    lo: float
    hi: float
    data: bytes = b""


@dataclass
class Program:
    vals: list = field(default_factory=list)
    ops: list = field(default_factory=list)
    args: list = field(default_factory=list)
    grads: list = field(default_factory=list)
    forward_ops: int = 0
    ret: int = -1
    seed: int = -1


def _ints(s):
    return [int(x) for x in s.split(",")] if s else []


def parse(text: str) -> Program:
    if text.startswith("error:"):
        raise ValueError(text)
    p = Program()
    for ln in text.split("\n"):
        t = ln.split(" ")
        if t[0] == "graph":
            kv = dict(x.split("=") for x in t[1:])
            p.forward_ops, p.ret, p.seed = int(kv["forward_ops"]), int(kv["ret"]), int(kv["seed"])
        elif t[0] == "args":
            p.args = [int(x) for x in t[1:]]
        elif t[0] == "grads":
            p.grads = [int(x) for x in t[1:]]
        elif t[0] == "val":
            kv = dict(x.split("=", 1) for x in t[3:])
            p.vals.append(Val(t[2], tuple(_ints(kv["shape"])), kv["name"]))
        elif t[0] == "op":
            kv = dict(x.split("=", 1) for x in t[2:])
            p.ops.append(Op(KINDS[int(kv["kind"])], int(kv["sub"]), int(kv["out"]), _ints(kv["in"]), _ints(kv["a"]),
                            _ints(kv["b"]), _ints(kv["c"]), _ints(kv["d"]), float(kv["f"]), int(kv["i"]), float(kv["lo"]),
                            float(kv["hi"]), bytes.fromhex(kv["data"])))
    return p


def _eval(p: Program, op: Op, x: list):
    v = p.vals[op.out]
    dt = DT[v.dtype]
    k = op.kind
    if k == "const_splat":
        if dt.is_floating_point:
            return torch.full(v.shape, op.f, dtype=torch.float64).to(dt)
        return torch.full(v.shape, bool(op.i) if dt == torch.bool else op.i, dtype=dt)
    if k == "const_data":
        return hlo._bits_to_tensor(op.data, hlo.TType(v.shape, v.dtype))
    if k == "iota":
        d = op.a[0]
        shp = [1] * len(v.shape)
        shp[d] = v.shape[d]
        return torch.arange(v.shape[d], dtype=dt).reshape(shp).expand(v.shape)
    if k == "unary":
        return UNARY[op.sub](x[0])
    if k == "binary":
        a, b = x
        if op.sub == 3 and not dt.is_floating_point:
            return torch.div(a, b, rounding_mode="trunc")
        return [lambda: a + b, lambda: a - b, lambda: a * b, lambda: a / b, lambda: torch.pow(a, b),
                lambda: torch.maximum(a, b), lambda: torch.minimum(a, b), lambda: a & b, lambda: a | b][op.sub]()
    if k == "compare":
        return CMP[op.sub](x[0], x[1])
    if k == "select":
        return torch.where(x[0], x[1], x[2])
    if k == "convert":
        if not dt.is_floating_point and x[0].is_floating_point():
            return torch.trunc(x[0]).to(dt)
        return x[0].to(dt)
    if k == "reshape":
        return x[0].reshape(v.shape)
    if k == "transpose":
        return x[0].permute(op.a)
    if k == "bcast":
        shp = [1] * len(v.shape)
        for src, dst in enumerate(op.a):
            shp[dst] = x[0].shape[src]
        return x[0].reshape(shp).expand(v.shape)
    if k == "slice":
        return x[0][tuple(slice(a, b, c) for a, b, c in zip(op.a, op.b, op.c))]
    if k == "concat":
        return torch.cat(list(x), dim=op.a[0])
    if k == "reduce":
        if op.sub == 0:
            return (x[0].sum(dim=op.a) + x[1]).to(dt)
        return torch.maximum(x[0].amax(dim=op.a), x[1])
    if k == "dot":
        return hlo.dot_general(x[0], x[1], op.a, op.b, op.c, op.d).reshape(v.shape)
    if k == "gather_rows":
        idx = x[1].reshape(-1).clamp(0, x[0].shape[0] - 1)
        return x[0][idx].reshape(v.shape)
    if k == "gather2":
        idx = x[1].reshape(-1, 2)
        return x[0][idx[:, 0].clamp(0, x[0].shape[0] - 1), idx[:, 1].clamp(0, x[0].shape[1] - 1)].reshape(v.shape)
    if k == "pad":
        out = torch.zeros(v.shape, dtype=dt)
        out[tuple(slice(a, b, c) for a, b, c in zip(op.a, op.b, op.c))] = x[0]
        return out
    if k == "scatter_rows":
        out = torch.zeros(v.shape, dtype=dt)
        idx = x[1].reshape(-1).clamp(0, v.shape[0] - 1)
        out.index_add_(0, idx, x[0].reshape((idx.numel(),) + tuple(v.shape[1:])))
        return out
    if k == "scatter2":
        out = torch.zeros(v.shape, dtype=dt).reshape(-1)
        idx = x[1].reshape(-1, 2)
        out.index_add_(0, idx[:, 0] * v.shape[1] + idx[:, 1], x[0].reshape(-1))
        return out.reshape(v.shape)
    if k == "guard_clamp":
        g = x[0]
        g = torch.where((g - g) == 0, g, torch.zeros_like(g))
        if op.sub:
            g = g.to(torch.float32).clamp(op.lo, op.hi).to(dt)
        return g
    raise NotImplementedError(k)


def run(p: Program, inputs: list, seed: float = 1.0, backward: bool = True):
    """-> (loss, [gradient or None per argument])."""
    env = {}
    for a, t in zip(p.args, inputs):
        v = p.vals[a]
        assert tuple(t.shape) == v.shape and t.dtype == DT[v.dtype], (v, t.shape, t.dtype)
        env[a] = t
    n = len(p.ops) if backward else p.forward_ops
    for op in p.ops[:n]:
        if op.kind == "seed":
            env[op.out] = torch.tensor(seed, dtype=DT[p.vals[op.out].dtype]).reshape(p.vals[op.out].shape)
            continue
        r = _eval(p, op, [env[i] for i in op.ins])
        v = p.vals[op.out]
        assert tuple(r.shape) == v.shape and r.dtype == DT[v.dtype], (op, r.shape, r.dtype, v)
        env[op.out] = r
    grads = [env[g] if (backward and g >= 0) else None for g in p.grads]
    return env[p.ret], grads
