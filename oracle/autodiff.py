"""Reverse-mode AD over a StableHLO function, restated from the reference.  Test infrastructure only.

The reference builds a gradient *graph* (src/autodiff/engine.zig:196-348) and lets IREE run it;
here the same sweep is applied eagerly to the tensors of one forward evaluation:

  * traversal: use-count reverse Kahn order starting at func.return, FIFO ready queue
    (engine.zig:472-530);
  * per-op rules: src/autodiff/vjp_rules.zig (line of each rule cited below), including the
    deliberately modified ones: divide/log/rsqrt add 1e-4 inside the rule, `maximum` is treated
    as ReLU of operand 0, `power` uses e*(y/x) with 0 where x == 0 and gives the exponent a zero
    gradient;
  * every adjoint edge (engine.zig:604-702): reduce to the operand's shape, finite guard
    ((g-g)==0 ? g : 0), clamp to [clip_min, clip_max] in f32, cast back to the edge's element
    type, then accumulate with an add in that type.

Rematerialisation (engine.zig:25-127) only re-computes values and has no numerical effect; it
is not restated.
"""
from __future__ import annotations

import torch

from . import stablehlo as hlo

EPS = 1e-4      # guard constant hard-coded in vjp_rules.zig:198,1510,1543


def _eps_like(x):
    # ops.constant builds the f32 value and converts it to the element type (src/core/ops.zig:849-854)
    return torch.tensor(EPS, dtype=torch.float32).to(x.dtype)


def reduce_gradient(g, shape):
    """src/core/ops.zig:1074-1129: sum away broadcast dimensions until g has `shape`."""
    shape = tuple(shape)
    if tuple(g.shape) == shape:
        return g
    if g.numel() == 1 and len(shape) == 0:
        return g.reshape(())
    while g.dim() > len(shape):
        g = g.sum(dim=0)
    for i, (gs, s) in enumerate(zip(g.shape, shape)):
        if gs != s and s == 1:
            g = g.sum(dim=i, keepdim=True)
    return g.reshape(shape)


# ---- per-op rules: fn(op, primals, g) -> list of operand gradients (None = no gradient) -------

def _add(op, p, g):            # vjp_rules.zig:29
    return [g, g]


def _subtract(op, p, g):       # :67
    return [g, -g]


def _multiply(op, p, g):       # :106
    return [g * p[1], g * p[0]]


def _divide(op, p, g):         # :154  (denominator b + 1e-4)
    a, b = p
    bs = b + _eps_like(b)
    return [g / bs, -((a * g) / (bs * bs))]


def _power(op, p, g):          # :252
    base, e = p
    y = torch.pow(base, e)
    ydb = torch.where(base == 0, torch.zeros_like(y), y / base)
    return [g * (e * ydb), torch.zeros_like(e)]


def _negate(op, p, g):         # :339
    return [-g]


def _transpose(op, p, g):      # :373
    perm = op.attrs["dims"]
    inv = [0] * len(perm)
    for i, d in enumerate(perm):
        inv[d] = i
    return [g.permute(inv)]


def _dot_general(op, p, g):    # :426  (batch dims are the leading ones)
    a, b = p
    nb = min(a.dim(), b.dim(), g.dim()) - 2
    batch = list(range(nb))
    ga = hlo.dot_general(g, b, batch, batch, [g.dim() - 1], [b.dim() - 1])
    gb = hlo.dot_general(a, g, batch, batch, [a.dim() - 2], [g.dim() - 2])
    return [ga, gb]


def _maximum(op, p, g):        # :499  ReLU rule: operand 0 only, strict x > 0
    x = p[0]
    return [torch.where(x > 0, g, torch.zeros_like(g))]


def _reshape(op, p, g):        # :565
    return [g.reshape(p[0].shape)]


def _reduce(op, p, g):         # sum :599, max :673
    x = p[0]
    dims = op.attrs["dims"]
    kept = [1 if i in dims else s for i, s in enumerate(x.shape)]
    gb = g.reshape(kept).expand(x.shape)
    if op.attrs["kind"] == "maximum":
        mx = x.amax(dim=dims).reshape(kept).expand(x.shape)
        return [torch.where(x == mx, gb, torch.zeros_like(x)), None]
    return [gb.to(x.dtype), None]


def _gather(op, p, g):         # :1115 (row gather -> scatter-add), :779 (2-index gather, linearised)
    operand, idx = p
    a = op.attrs
    out = torch.zeros_like(operand)
    if a["collapsed_slice_dims"] == [0] and a["start_index_map"] == [0]:
        ivd = a["index_vector_dim"]
        if ivd is not None and ivd < idx.dim():
            idx = idx.select(ivd, 0)
        flat = idx.reshape(-1).clamp(0, operand.shape[0] - 1)
        out.index_add_(0, flat, g.reshape(flat.numel(), -1).reshape((flat.numel(),) + tuple(operand.shape[1:])))
        return [out, None]
    if a["collapsed_slice_dims"] == [0, 1]:
        ivd = a["index_vector_dim"]
        lin = idx.select(ivd, 0) * operand.shape[1] + idx.select(ivd, 1)
        flat = out.reshape(-1)
        flat.index_add_(0, lin.reshape(-1), g.reshape(-1))
        return [flat.reshape(operand.shape), None]
    raise NotImplementedError(a)


def _slice(op, p, g):          # :1260 (pad with zeros)
    out = torch.zeros_like(p[0])
    out[tuple(slice(a, b, s) for a, b, s in op.attrs["ranges"])] = g
    return [out]


def _broadcast_in_dim(op, p, g):   # :1336
    x = p[0]
    dims = op.attrs["dims"]
    red = [i for i in range(g.dim()) if i not in dims]
    r = g.sum(dim=red) if red else g
    for i, s in enumerate(x.shape):
        if s == 1 and r.shape[i] != 1:
            r = r.sum(dim=i, keepdim=True)
    return [r.reshape(x.shape).to(x.dtype)]


def _exponential(op, p, g):    # :1436
    return [g * torch.exp(p[0])]


def _log(op, p, g):            # :1476  g / (x + 1e-4)
    return [g / (p[0] + _eps_like(p[0]))]


def _rsqrt(op, p, g):          # :1529  -0.5 * g * rsqrt(x + 1e-4)^3
    r = torch.rsqrt(p[0] + _eps_like(p[0]))
    cub = (r * r) * r
    return [(g * torch.tensor(-0.5, dtype=torch.float32).to(g.dtype)) * cub]


def _convert(op, p, g):        # :1584
    return [g.to(p[0].dtype)]


def _select(op, p, g):         # :1640
    pred = p[0]
    z = torch.zeros_like(g)
    return [None, torch.where(pred, g, z), torch.where(pred, z, g)]


def _tanh(op, p, g):           # :1692
    y = torch.tanh(p[0])
    return [g * (torch.ones_like(y) - y * y)]


def _logistic(op, p, g):       # :1019
    s = torch.sigmoid(p[0])
    return [g * (s * (torch.ones_like(s) - s))]


def _sine(op, p, g):           # :937
    return [g * torch.cos(p[0])]


def _cosine(op, p, g):         # :977
    return [-(g * torch.sin(p[0]))]


def _concatenate(op, p, g):    # :1071
    outs, at = [], 0
    d = op.attrs["dim"]
    for x in p:
        n = x.shape[d]
        outs.append(g.narrow(d, at, n))
        at += n
    return outs


RULES = {
    "stablehlo.add": _add, "stablehlo.subtract": _subtract, "stablehlo.multiply": _multiply,
    "stablehlo.divide": _divide, "stablehlo.power": _power, "stablehlo.negate": _negate,
    "stablehlo.transpose": _transpose, "stablehlo.dot_general": _dot_general,
    "stablehlo.maximum": _maximum, "stablehlo.reshape": _reshape, "stablehlo.reduce": _reduce,
    "stablehlo.gather": _gather, "stablehlo.slice": _slice,
    "stablehlo.broadcast_in_dim": _broadcast_in_dim, "stablehlo.exponential": _exponential,
    "stablehlo.log": _log, "stablehlo.rsqrt": _rsqrt, "stablehlo.convert": _convert,
    "stablehlo.select": _select, "stablehlo.tanh": _tanh, "stablehlo.logistic": _logistic,
    "stablehlo.sine": _sine, "stablehlo.cosine": _cosine, "stablehlo.concatenate": _concatenate,
}
# ops without a rule (iota, dynamic_iota, compare, and, ceil, constant ...) stop the gradient
# (engine.zig:134-193).


def _guard_and_clamp(g, clip_min, clip_max):
    """engine.zig:622-682."""
    finite = (g - g) == 0
    g = torch.where(finite, g, torch.zeros_like(g))
    if clip_min is None:
        return g
    gf = g.to(torch.float32) if g.dtype != torch.float32 else g
    gf = torch.minimum(torch.maximum(gf, torch.tensor(clip_min, dtype=torch.float32)),
                       torch.tensor(clip_max, dtype=torch.float32))
    return gf.to(g.dtype)


def gradients(fn: hlo.Func, env: dict, seed: torch.Tensor, clip_min=-100.0, clip_max=100.0,
              guards=True):
    """Adjoints of every function argument, given env from `stablehlo.evaluate(..., keep_env=True)`.

    guards=False switches the finite guard and the clamp off (used to compare the bare rules with
    torch.autograd); the 1e-4 terms inside the rules stay.
    Returns {arg name: tensor or None}.
    """
    producer = {op.result: op for op in fn.ops if op.result is not None}
    use_counts = {}
    for op in fn.ops:
        for o in op.operands:
            if o in producer:
                use_counts[o] = use_counts.get(o, 0) + 1

    adj = {fn.return_value: seed}
    queue = [fn.ops[-1]]
    while queue:
        op = queue.pop(0)
        if op.name != "func.return" and op.result in adj and op.name in RULES:
            g = adj[op.result]
            if tuple(g.shape) != tuple(op.out_type.shape):
                g = g.reshape(op.out_type.shape)
            primals = [env[o] for o in op.operands]
            grads = RULES[op.name](op, primals, g)
            for o, x, gi in zip(op.operands, primals, grads):
                if gi is None or not x.is_floating_point():
                    continue
                gi = reduce_gradient(gi, x.shape)
                if guards:
                    gi = _guard_and_clamp(gi, clip_min, clip_max)
                if o in adj:
                    adj[o] = adj[o] + gi
                else:
                    adj[o] = gi
        for o in op.operands:
            if o in producer:
                use_counts[o] -= 1
                if use_counts[o] == 0:
                    queue.append(producer[o])
    return {name: adj.get(name) for name, _ in fn.args}
