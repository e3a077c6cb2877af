"""Seeded random forward graphs through the general front end's host side (no GPU): for each graph the library's
tensor program — forward ops, stability patches, gradient rules, adjoint edges, accumulation order — evaluated with
torch must reproduce the oracle's loss and gradients exactly.  The graphs mix element-wise ops, broadcasts, transposes,
reshapes, strided slices, concatenates, reductions over random dimensions, plain and batched dot_generals, compare +
select, row gathers by the integer inputs, iota masks, f64 stretches, integer and f32 <-> bf16 converts over small shapes; values stay finite by construction."""
import random

import pytest
import torch

import graph_program as gp
from oracle.worker import TrainingModule
from pcp_b200.backend import graph_describe
from pcp_b200.export import _Emitter

PARAM_SHAPES = [(4, 6), (6, 5), (5,), (2, 4, 6)]


def _random_graph(seed, dt):
    rng = random.Random(seed)
    e = _Emitter()
    args = [f"%arg{i}: {e.ty(s, dt)}" for i, s in enumerate(PARAM_SHAPES)]
    args += [f"%arg{len(PARAM_SHAPES)}: {e.ty((2, 3), 'i64')}", f"%arg{len(PARAM_SHAPES) + 1}: {e.ty((2, 3), 'i64')}"]
    pool = [(f"%arg{i}", tuple(s), dt) for i, s in enumerate(PARAM_SHAPES)]
    zero = e.const("0.000000e+00", (), dt)
    ninf = e.const("0xFF800000", (), "f32")

    def const_like(x, lit):
        return e.const(lit, x[1], x[2])

    def pick(pred=lambda t: True):
        c = [t for t in pool if pred(t)]
        return rng.choice(c) if c else None

    for _ in range(rng.randint(10, 24)):
        kind = rng.choice(["unary", "binary", "bcast", "transpose", "reshape", "slice", "concat", "reduce", "dot", "bdot",
                           "select", "convert", "safe_div", "rsqrt", "power", "gather", "f64", "iota_mask", "ids"])
        x = pick()
        if kind == "unary":
            y = e.un(rng.choice(["tanh", "logistic", "negate", "sine", "cosine"]), x)
        elif kind == "binary":
            z = pick(lambda t: t[1] == x[1] and t[2] == x[2])
            y = e.bin(rng.choice(["add", "subtract", "multiply", "maximum"]), x, z)
        elif kind == "safe_div":                       # x / (z*z + 1)
            z = pick(lambda t: t[1] == x[1] and t[2] == x[2])
            y = e.bin("divide", x, e.bin("add", e.bin("multiply", z, z), const_like(z, "1.000000e+00")))
        elif kind == "rsqrt":                          # rsqrt(x*x + 1)
            y = e.un("rsqrt", e.bin("add", e.bin("multiply", x, x), const_like(x, "1.000000e+00")))
        elif kind == "power":                          # (x*x + 1) ^ 2 and tanh(x) ^ 3
            if rng.random() < 0.5:
                y = e.bin("power", e.bin("add", e.bin("multiply", x, x), const_like(x, "1.000000e+00")), const_like(x, "2.000000e+00"))
            else:
                y = e.bin("power", e.un("tanh", x), const_like(x, "3.000000e+00"))
        elif kind == "bcast":
            if len(x[1]) >= 3:
                continue
            new = rng.choice([2, 3])
            at = rng.randint(0, len(x[1]))
            shape = x[1][:at] + (new,) + x[1][at:]
            y = e.bcast(x, shape, [i if i < at else i + 1 for i in range(len(x[1]))])
        elif kind == "transpose":
            if len(x[1]) < 2:
                continue
            perm = list(range(len(x[1])))
            rng.shuffle(perm)
            y = e.transpose(x, perm)
        elif kind == "reshape":
            n = 1
            for s in x[1]:
                n *= s
            opts = [(n,)] + [(a, n // a) for a in (2, 3, 4, 5, 6) if n % a == 0]
            y = e.reshape(x, rng.choice(opts))
        elif kind == "slice":
            if not x[1]:
                continue
            rs, shape = [], []
            for s in x[1]:
                a = rng.randint(0, s - 1)
                b = rng.randint(a + 1, s)
                st = rng.choice([1, 1, 2])
                rs.append((a, b, st)); shape.append((b - a + st - 1) // st)
            y = e.emit(f"stablehlo.slice {x[0]} [{', '.join(f'{a}:{b}:{st}' for a, b, st in rs)}]", shape, x[2],
                       f"({e.ty(x[1], x[2])}) -> {e.ty(shape, x[2])}")
        elif kind == "concat":
            if not x[1]:
                continue
            d = rng.randrange(len(x[1]))
            z = pick(lambda t: len(t[1]) == len(x[1]) and t[2] == x[2] and all(a == b for i, (a, b) in enumerate(zip(t[1], x[1])) if i != d))
            y = e.concat(x, z, d)
        elif kind == "reduce":
            if not x[1]:
                continue
            dims = sorted(rng.sample(range(len(x[1])), rng.randint(1, len(x[1]))))
            if rng.random() < 0.3 and x[2] == "f32":
                y = e.reduce("maximum", x, ninf, dims)
            else:
                y = e.reduce("add", x, zero if x[2] == dt else e.const("0.000000e+00", (), x[2]), dims)
        elif kind == "dot":
            a = pick(lambda t: len(t[1]) == 2)
            b = pick(lambda t: a and len(t[1]) == 2 and t[1][0] == a[1][1] and t[2] == a[2])
            if not a or not b:
                continue
            y = e.dot(a, b)
        elif kind == "bdot":
            a = pick(lambda t: len(t[1]) == 3)
            if not a:
                continue
            y = e.dot(a, e.transpose(a, [0, 2, 1]), batched=True)
        elif kind == "select":
            z = pick(lambda t: t[1] == x[1] and t[2] == x[2])
            y = e.select(e.compare(rng.choice(["GT", "LE", "NE"]), x, z, "FLOAT"), x, e.un("negate", z))
        elif kind == "gather":                         # rows of a 2-D value picked by the ids argument (values 0..3)
            t = pick(lambda t: len(t[1]) == 2 and t[1][0] >= 4)
            if not t:
                continue
            y = e.emit(
                f'"stablehlo.gather"({t[0]}, %arg{len(PARAM_SHAPES)}) <{{dimension_numbers = #stablehlo.gather<offset_dims = [2], '
                f'collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = 2>, indices_are_sorted = false, '
                f'slice_sizes = array<i64: 1, {t[1][1]}>}}>', (2, 3, t[1][1]), t[2],
                f"({e.ty(t[1], t[2])}, {e.ty((2, 3), 'i64')}) -> {e.ty((2, 3, t[1][1]), t[2])}")
        elif kind == "f64":                            # a stretch in f64, as the LayerNorm variance of the nanoGPT exports
            if x[2] != "f32":
                continue
            d = e.convert(x, "f64")
            d = e.bin("multiply", d, d)
            if d[1]:
                k = rng.randrange(len(d[1]))
                d = e.reduce("add", d, e.const("0.000000e+00", (), "f64"), [k])
            y = e.convert(d, "f32")
        elif kind == "iota_mask":                      # keep the entries whose index along one dimension is below a bound
            if not x[1]:
                continue
            k = rng.randrange(len(x[1]))
            io = e.iota(x[1], k)
            m = e.compare("LT", io, e.const(str(rng.randint(1, x[1][k])), x[1], "i64"))
            y = e.select(m, x, const_like(x, "0.000000e+00"))
        elif kind == "ids":                            # the integer inputs as numbers: x[0, 0] scaled by (ids + 1) summed
            f = e.convert(e.convert((f"%arg{len(PARAM_SHAPES) + 1}", (2, 3), "i64"), "i32"), x[2])
            one = e.const("1.000000e+00", (2, 3), x[2])
            sc = e.reduce("add", e.bin("add", f, one), e.const("0.000000e+00", (), x[2]), [0, 1])
            y = e.bin("multiply", x, e.bcast(sc, x[1], []))
        else:                                          # convert to the other float type and back
            other = "bf16" if x[2] == "f32" else "f32"
            y = e.convert(x, other)
        pool.append((y[0], tuple(y[1]), y[2]))

    # loss: every parameter and the last values, each tamed by tanh and summed to a scalar
    total = None
    for t in pool[: len(PARAM_SHAPES)] + pool[-6:]:
        v = e.un("tanh", t)
        if v[2] != "f32":
            v = e.convert(v, "f32")
        if v[1]:
            v = e.reduce("add", v, e.const("0.000000e+00", (), "f32"), list(range(len(v[1]))))
        total = v if total is None else e.bin("add", total, v)
    out = ["module {", f"  func.func @main({', '.join(args)}) -> tensor<f32> {{"] + e.lines
    out += [f"    return {total[0]} : tensor<f32>", "  }", "}", ""]
    return "\n".join(out)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_random_graphs_match_the_oracle_exactly(lib_built, dt):
    ids = torch.tensor([[0, 3, 1], [2, 2, 0]], dtype=torch.int64)
    for seed in range(40):
        text = _random_graph(seed, dt)
        mod = TrainingModule(text)
        g = torch.Generator().manual_seed(seed)
        params = mod._model_params([torch.randn(s, generator=g) for s in PARAM_SHAPES])
        prog = gp.parse(graph_describe(text, with_plan=True))            # the plan must exist too (every op has a kernel)
        loss, grads = gp.run(prog, params + [ids, ids], seed=3.0)
        want = mod.model_forward_pass_grad(params, ids, ids, 3.0)
        want_loss = mod.forward([p.to(torch.float32) for p in params], ids, ids)
        assert torch.isfinite(want_loss), seed
        assert float(loss) == float(want_loss), seed
        for i, (a, w) in enumerate(zip(grads, want)):
            a = a if a is not None else torch.zeros_like(w)
            assert a.dtype == w.dtype and torch.equal(a, w), (seed, i)
