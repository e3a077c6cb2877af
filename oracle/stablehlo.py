"""StableHLO text subset: parser and torch-CPU evaluator.  Test infrastructure only.

Covers the op set that appears in the reference's exported forward graphs
(models/*.mlir, produced by tools/generate_*.py through torch_mlir) in the
"pretty" assembly form those files use, including `dense_resource` hex blobs.
Semantics follow the public StableHLO specification; element types are kept
exactly (bf16 ops round per op, f64 stays f64).
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field

import numpy as np
import torch

DTYPES = {
    "f32": torch.float32, "f64": torch.float64, "bf16": torch.bfloat16, "f16": torch.float16,
    "i64": torch.int64, "i32": torch.int32, "i16": torch.int16, "i8": torch.int8, "i1": torch.bool,
}
_NP_OF = {"f32": np.float32, "f64": np.float64, "f16": np.float16, "i64": np.int64, "i32": np.int32,
          "i16": np.int16, "i8": np.int8}


@dataclass(frozen=True)
class TType:
    shape: tuple
    dtype: str

    @property
    def torch_dtype(self):
        return DTYPES[self.dtype]

    @property
    def is_float(self):
        return self.dtype in ("f32", "f64", "bf16", "f16")

    def __str__(self):
        return "tensor<" + "".join(f"{d}x" for d in self.shape) + self.dtype + ">"


def parse_type(s: str) -> TType:
    s = s.strip()
    m = re.fullmatch(r"tensor<(.*)>", s)
    if not m:
        raise ValueError(f"not a tensor type: {s!r}")
    parts = m.group(1).split("x")
    return TType(tuple(int(p) for p in parts[:-1]), parts[-1])


@dataclass
class Op:
    result: str | None          # SSA name without '%', None for return
    name: str                   # e.g. "stablehlo.add", "func.return"
    operands: list
    out_type: TType | None
    in_types: list
    attrs: dict = field(default_factory=dict)


@dataclass
class Func:
    name: str
    args: list                  # [(ssa name, TType)]
    ops: list                   # [Op], the last one is func.return
    result_type: TType
    resources: dict             # name -> bytes (blob, header stripped)

    @property
    def return_value(self):
        return self.ops[-1].operands[0]


_SSA = re.compile(r"%([A-Za-z0-9_.]+)")
_TYPE = re.compile(r"tensor<[^>]*>")


def _int_list(s):
    s = s.strip()
    if not s:
        return []
    return [int(x) for x in s.split(",")]


def _split_types(tail: str):
    """'(T1, T2) -> T3' | 'T' | 'T1, T2'  ->  (in_types, out_type)"""
    types = [parse_type(t) for t in _TYPE.findall(tail)]
    if "->" in tail:
        return types[:-1], types[-1]
    return types, types[-1]


def parse_module(text: str, fn_name: str = "main") -> Func:
    resources = {}
    res_at = text.find("{-#")
    body = text if res_at < 0 else text[:res_at]
    if res_at >= 0:
        for m in re.finditer(r"([A-Za-z0-9_.]+):\s*\"0x([0-9A-Fa-f]*)\"", text[res_at:]):
            raw = bytes.fromhex(m.group(2))
            resources[m.group(1)] = raw[4:]      # 4-byte alignment header precedes the payload

    lines = body.split("\n")
    i = 0
    header = None
    for i, ln in enumerate(lines):
        if re.search(r"func\.func\s+(public\s+|private\s+)?@" + re.escape(fn_name) + r"\(", ln):
            header = ln
            break
    if header is None:
        raise ValueError(f"function @{fn_name} not found")
    sig, ret = header.rsplit("->", 1)
    args = [(m.group(1), parse_type(m.group(2)))
            for m in re.finditer(r"%([A-Za-z0-9_.]+):\s*(tensor<[^>]*>)", sig)]
    result_type = parse_type(_TYPE.search(ret).group(0))

    ops = []
    for ln in lines[i + 1:]:
        s = ln.strip()
        if not s or s.startswith("//"):
            continue
        if s.startswith("return") or s.startswith("func.return"):
            ops.append(Op(None, "func.return", _SSA.findall(s.split(" : ")[0]), None,
                          [parse_type(t) for t in _TYPE.findall(s)]))
            break
        if s == "}":
            break
        ops.append(_parse_op_line(s))
    return Func(fn_name, args, ops, result_type, resources)


def _parse_op_line(s: str) -> Op:
    m = re.match(r"%([A-Za-z0-9_.]+)\s*=\s*(.*)$", s)
    if not m:
        raise ValueError(f"cannot parse op line: {s[:120]!r}")
    res, rest = m.group(1), m.group(2)
    head, tail = rest.rsplit(" : ", 1)
    in_types, out_type = _split_types(tail)
    attrs = {}
    if head.startswith('"'):                                   # generic form: "stablehlo.gather"(...) <{...}>
        name = re.match(r'"([^"]+)"', head).group(1)
        paren = head[head.index("(") + 1: head.index(")")]
        operands = _SSA.findall(paren)
        a = head[head.index(")") + 1:]
        for key in ("offset_dims", "collapsed_slice_dims", "start_index_map", "operand_batching_dims",
                    "start_indices_batching_dims"):
            mm = re.search(key + r"\s*=\s*\[([^\]]*)\]", a)
            attrs[key] = _int_list(mm.group(1)) if mm else []
        mm = re.search(r"index_vector_dim\s*=\s*(\d+)", a)
        attrs["index_vector_dim"] = int(mm.group(1)) if mm else None
        mm = re.search(r"slice_sizes\s*=\s*array<i64:\s*([^>]*)>", a)
        attrs["slice_sizes"] = _int_list(mm.group(1)) if mm else []
        return Op(res, name, operands, out_type, in_types, attrs)

    name = re.match(r"([A-Za-z_.0-9]+)", head).group(1)
    after = head[len(name):]
    if name in ("stablehlo.constant", "arith.constant"):
        attrs["value"] = after.strip()
        return Op(res, "stablehlo.constant", [], out_type, [], attrs)
    operands = _SSA.findall(after)
    if name == "stablehlo.reduce":
        attrs["kind"] = re.search(r"applies\s+stablehlo\.([a-z_]+)", after).group(1)
        attrs["dims"] = _int_list(re.search(r"dimensions\s*=\s*\[([^\]]*)\]", after).group(1))
    elif name in ("stablehlo.broadcast_in_dim", "stablehlo.transpose"):
        attrs["dims"] = _int_list(re.search(r"dims\s*=\s*\[([^\]]*)\]", after).group(1))
    elif name == "stablehlo.dot_general":
        mb = re.search(r"batching_dims\s*=\s*\[([^\]]*)\]\s*x\s*\[([^\]]*)\]", after)
        mc = re.search(r"contracting_dims\s*=\s*\[([^\]]*)\]\s*x\s*\[([^\]]*)\]", after)
        attrs["lb"], attrs["rb"] = (_int_list(mb.group(1)), _int_list(mb.group(2))) if mb else ([], [])
        attrs["lc"], attrs["rc"] = (_int_list(mc.group(1)), _int_list(mc.group(2))) if mc else ([], [])
    elif name == "stablehlo.slice":
        rng = re.search(r"\[([^\]]*)\]", after).group(1)
        sl = []
        for part in rng.split(","):
            p = [int(x) for x in part.strip().split(":")]
            sl.append((p[0], p[1], p[2] if len(p) > 2 else 1))
        attrs["ranges"] = sl
    elif name == "stablehlo.concatenate":
        attrs["dim"] = int(re.search(r"dim\s*=\s*(\d+)", after).group(1))
    elif name in ("stablehlo.iota", "stablehlo.dynamic_iota"):
        attrs["dim"] = int(re.search(r"dim\s*=\s*(\d+)", after).group(1))
    elif name == "stablehlo.compare":
        mm = re.match(r"\s*([A-Z]{2})\s*,", after)
        attrs["dir"] = mm.group(1)
    return Op(res, name, operands, out_type, in_types, attrs)


# ----------------------------------------------------------------------------------------
# evaluation
# ----------------------------------------------------------------------------------------

def _bits_to_tensor(raw: bytes, t: TType) -> torch.Tensor:
    if t.dtype == "bf16":
        u = np.frombuffer(raw, dtype="<u2").astype(np.int32)
        f = (u.astype(np.uint32) << 16).view(np.float32)
        return torch.from_numpy(f.copy()).to(torch.bfloat16).reshape(t.shape)
    if t.dtype == "i1":
        return torch.from_numpy(np.frombuffer(raw, dtype=np.uint8).copy()).bool().reshape(t.shape)
    a = np.frombuffer(raw, dtype=np.dtype(_NP_OF[t.dtype]).newbyteorder("<"))
    return torch.from_numpy(a.astype(_NP_OF[t.dtype]).copy()).reshape(t.shape)


def _scalar_literal(tok: str, t: TType):
    tok = tok.strip()
    if tok in ("true", "false"):
        return tok == "true"
    if tok.startswith("0x") or tok.startswith("-0x"):
        bits = int(tok, 16)
        if t.dtype == "f32":
            return float(np.array([bits], dtype=np.uint32).view(np.float32)[0])
        if t.dtype == "bf16":
            if bits > 0xFFFF:       # a 32-bit pattern given for a bf16 constant: keep the high half
                bits >>= 16
            return float((np.array([bits], dtype=np.uint32) << 16).view(np.float32)[0])
        if t.dtype == "f64":
            return float(np.array([bits], dtype=np.uint64).view(np.float64)[0])
        return bits
    if t.is_float:
        return float(tok)
    return int(float(tok)) if ("e" in tok or "." in tok) else int(tok)


def constant_value(op: Op, resources: dict) -> torch.Tensor:
    v = op.attrs["value"]
    t = op.out_type
    m = re.match(r"dense_resource<([^>]+)>", v)
    if m:
        return _bits_to_tensor(resources[m.group(1)], t)
    m = re.match(r"dense<(.*)>$", v, re.S)
    if not m:
        raise ValueError(f"unsupported constant: {v[:80]}")
    lit = m.group(1).strip()
    if lit.startswith('"0x'):                        # dense<"0x...."> raw payload
        return _bits_to_tensor(bytes.fromhex(lit[3:-1]), t)
    if lit.startswith("["):
        toks = re.findall(r"[-+]?0x[0-9A-Fa-f]+|true|false|[-+]?[0-9.]+(?:[eE][-+]?\d+)?|[-+]?inf|nan", lit)
        vals = [_scalar_literal(x, t) for x in toks]
        return torch.tensor(vals, dtype=torch.float64 if t.is_float else None).to(t.torch_dtype).reshape(t.shape)
    val = _scalar_literal(lit, t)
    if t.is_float:      # constants are exact decimal -> nearest value of the element type
        return torch.full(t.shape, val, dtype=torch.float64).to(t.torch_dtype)
    return torch.full(t.shape, val, dtype=t.torch_dtype)


def dot_general(a, b, lb, rb, lc, rc):
    """StableHLO dot_general: result dims = batch..., lhs free..., rhs free..."""
    letters = "abcdefghijklmnopqrstuvwxyz"
    la = [None] * a.dim()
    lbb = [None] * b.dim()
    nxt = 0
    for i, j in zip(lb, rb):
        la[i] = lbb[j] = letters[nxt]; nxt += 1
    for i, j in zip(lc, rc):
        la[i] = lbb[j] = letters[nxt]; nxt += 1
    out = [la[i] for i in lb]
    for i in range(a.dim()):
        if la[i] is None:
            la[i] = letters[nxt]; nxt += 1
            out.append(la[i])
    for j in range(b.dim()):
        if lbb[j] is None:
            lbb[j] = letters[nxt]; nxt += 1
            out.append(lbb[j])
    return torch.einsum(f"{''.join(la)},{''.join(lbb)}->{''.join(out)}", a, b)


def gather(operand, indices, attrs, out_shape):
    sim = attrs["start_index_map"]
    ivd = attrs["index_vector_dim"]
    if attrs["collapsed_slice_dims"] == [0] and sim == [0]:
        idx = indices
        if ivd is not None and ivd < indices.dim():
            idx = indices.select(ivd, 0)
        idx = idx.clamp(0, operand.shape[0] - 1)
        return operand[idx].reshape(out_shape)
    if attrs["collapsed_slice_dims"] == [0, 1] and sim == [0, 1]:
        i0 = indices.select(ivd, 0).clamp(0, operand.shape[0] - 1)
        i1 = indices.select(ivd, 1).clamp(0, operand.shape[1] - 1)
        return operand[i0, i1].reshape(out_shape)
    raise NotImplementedError(f"gather pattern {attrs}")


_UNARY = {
    "stablehlo.rsqrt": torch.rsqrt, "stablehlo.sqrt": torch.sqrt, "stablehlo.exponential": torch.exp,
    "stablehlo.log": torch.log, "stablehlo.tanh": torch.tanh, "stablehlo.logistic": torch.sigmoid,
    "stablehlo.negate": torch.neg, "stablehlo.ceil": torch.ceil, "stablehlo.sine": torch.sin,
    "stablehlo.cosine": torch.cos, "stablehlo.abs": torch.abs, "stablehlo.floor": torch.floor,
}
_CMP = {"EQ": torch.eq, "NE": torch.ne, "GE": torch.ge, "GT": torch.gt, "LE": torch.le, "LT": torch.lt}


def eval_op(op: Op, x: list, resources: dict) -> torch.Tensor:
    n = op.name
    t = op.out_type
    if n == "stablehlo.constant":
        return constant_value(op, resources)
    if n in _UNARY:
        return _UNARY[n](x[0])
    if n == "stablehlo.add":
        return x[0] + x[1]
    if n == "stablehlo.subtract":
        return x[0] - x[1]
    if n == "stablehlo.multiply":
        return x[0] * x[1]
    if n == "stablehlo.divide":
        if t.is_float:
            return x[0] / x[1]
        return torch.div(x[0], x[1], rounding_mode="trunc")
    if n == "stablehlo.power":
        return torch.pow(x[0], x[1])
    if n == "stablehlo.maximum":
        return torch.maximum(x[0], x[1])
    if n == "stablehlo.minimum":
        return torch.minimum(x[0], x[1])
    if n == "stablehlo.and":
        return x[0] & x[1]
    if n == "stablehlo.or":
        return x[0] | x[1]
    if n == "stablehlo.convert":
        if not t.is_float and x[0].is_floating_point():
            return torch.trunc(x[0]).to(t.torch_dtype)
        return x[0].to(t.torch_dtype)
    if n == "stablehlo.reshape":
        return x[0].reshape(t.shape)
    if n == "stablehlo.transpose":
        return x[0].permute(op.attrs["dims"])
    if n == "stablehlo.broadcast_in_dim":
        dims = op.attrs["dims"]
        shp = [1] * len(t.shape)
        for src, dst in enumerate(dims):
            shp[dst] = x[0].shape[src]
        return x[0].reshape(shp).expand(t.shape)
    if n == "stablehlo.dot_general":
        a = op.attrs
        return dot_general(x[0], x[1], a["lb"], a["rb"], a["lc"], a["rc"])
    if n == "stablehlo.reduce":
        dims = op.attrs["dims"]
        if op.attrs["kind"] == "add":
            r = x[0].sum(dim=dims) if dims else x[0]
            return (r + x[1]).to(t.torch_dtype)
        if op.attrs["kind"] == "maximum":
            r = x[0].amax(dim=dims) if dims else x[0]
            return torch.maximum(r, x[1].to(r.dtype))
        raise NotImplementedError(op.attrs["kind"])
    if n == "stablehlo.slice":
        idx = tuple(slice(a, b, s) for a, b, s in op.attrs["ranges"])
        return x[0][idx]
    if n == "stablehlo.concatenate":
        return torch.cat(list(x), dim=op.attrs["dim"])
    if n == "stablehlo.compare":
        return _CMP[op.attrs["dir"]](x[0], x[1])
    if n == "stablehlo.select":
        return torch.where(x[0], x[1], x[2])
    if n in ("stablehlo.iota", "stablehlo.dynamic_iota"):
        d = op.attrs["dim"]
        shp = [1] * len(t.shape)
        shp[d] = t.shape[d]
        return torch.arange(t.shape[d], dtype=t.torch_dtype).reshape(shp).expand(t.shape)
    if n == "stablehlo.gather":
        return gather(x[0], x[1], op.attrs, t.shape)
    raise NotImplementedError(n)


def evaluate(fn: Func, inputs: list, keep_env: bool = False):
    """Run the function on torch tensors (one per argument, dtypes must match)."""
    if len(inputs) != len(fn.args):
        raise ValueError(f"expected {len(fn.args)} inputs, got {len(inputs)}")
    env = {}
    for (name, t), v in zip(fn.args, inputs):
        if tuple(v.shape) != t.shape or v.dtype != t.torch_dtype:
            raise ValueError(f"argument %{name}: expected {t}, got {tuple(v.shape)} {v.dtype}")
        env[name] = v
    last_use = {}
    if not keep_env:                       # free intermediates after their last use
        for i, op in enumerate(fn.ops):
            for o in op.operands:
                last_use[o] = i
    for i, op in enumerate(fn.ops[:-1]):
        env[op.result] = eval_op(op, [env[o] for o in op.operands], fn.resources)
        if not keep_env:
            for o in set(op.operands):
                if last_use.get(o) == i:
                    del env[o]
    out = env[fn.return_value]
    return (out, env) if keep_env else out
