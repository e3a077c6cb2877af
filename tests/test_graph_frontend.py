"""General StableHLO front end, host side (no GPU): the tensor program the library derives from a forward graph —
parser, stability patches, gradient rules, adjoint edges — evaluated with torch and compared with the oracle's
interpretation of the same graph (oracle/stablehlo.py + oracle/autodiff.py).  Both apply the same rules to the same
values in the same order, so the comparison is exact."""
import os

import pytest
import torch

import graph_program as gp
import helpers
from helpers import make_model, seeded_params
from oracle.worker import TrainingModule
from pcp_b200 import backend as bk
from pcp_b200.backend import BackendError, graph_describe, inspect_artifact

REF = os.environ.get("PCP_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))


def _batch(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, cfg.vocab, (cfg.batch, cfg.seq_len), generator=g)
    tg = torch.randint(0, cfg.vocab, (cfg.batch, cfg.seq_len), generator=g)
    tg[0, :3] = -1 if hasattr(cfg, "n_kv_head") else -100          # ignored positions
    return ids, tg


def _compare(text, cfg, seed=1.0):
    mod = TrainingModule(text)
    params = seeded_params(cfg, 1)
    ids, tg = _batch(cfg, 3)
    prog = gp.parse(graph_describe(text))
    model_params = mod._model_params(params)
    loss, grads = gp.run(prog, model_params + [ids, tg], seed=seed)
    want = mod.model_forward_pass_grad(model_params, ids, tg, seed)
    want_loss = mod.forward(params, ids, tg)
    assert float(loss) == float(want_loss)
    for g, w in zip(grads, want):
        g = g if g is not None else torch.zeros_like(w)
        assert g.dtype == w.dtype and torch.equal(g, w)
    return prog


@pytest.mark.parametrize("name", ["SMALL_F32", "GPT_SMALL_F32", "GPT_SMALL_BF16", "GPT_GELU_F32"])
def test_program_matches_oracle_exactly(lib_built, name):
    cfg, text = make_model(getattr(helpers, name))
    prog = _compare(text, cfg)
    assert prog.forward_ops < len(prog.ops) and prog.seed >= 0 and all(g >= 0 for g in prog.grads[:-2])


def test_clamp_of_the_adjoint_edges_is_in_the_program(lib_built):
    """d(loss) = 500: the oracle's clamp to +-100 is active on the first edges; the program must clamp the same way."""
    cfg, text = make_model(helpers.SMALL_F32)
    _compare(text, cfg, seed=500.0)


def test_graphs_outside_the_fused_families_take_the_general_path(lib_built):
    cfg, text = make_model(helpers.SMALL_F32)
    assert inspect_artifact(text)["family"] == "fused"
    other = text.replace("stablehlo.tanh ", "stablehlo.logistic ", 1)         # another soft-cap: not nanochat any more
    f = inspect_artifact(other)
    assert f["family"] == "graph" and f["d_model"] == 0 and f["n_layer"] == 0
    assert (f["batch"], f["block"], f["dtype"], f["vocab"]) == (cfg.batch, cfg.seq_len, bk.F32, cfg.vocab)
    assert f["num_tensors"] == len(cfg.param_shapes()) and f["total_params"] == cfg.num_params()
    _compare(other, cfg)


def test_unsupported_graphs_are_refused_with_a_reason(lib_built):
    cfg, text = make_model(helpers.SMALL_F32)
    for bad, what in ((text.replace("stablehlo.tanh ", "stablehlo.erf_inv ", 1), "unsupported op"),
                      (text.replace("func.func @main", "func.func @other"), "@main")):
        with pytest.raises(BackendError) as ei:
            graph_describe(bad)
        assert ei.value.code == bk.E_ARTIFACT and what in str(ei.value)
        with pytest.raises(BackendError):
            inspect_artifact(bad)


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "models")), reason="reference tree not present")
def test_every_shipped_reference_graph_has_a_program(lib_built):
    import glob
    files = sorted(glob.glob(os.path.join(REF, "models", "*.mlir")))
    assert len(files) >= 17
    for fn in files:
        prog = gp.parse(graph_describe(open(fn).read()))
        assert prog.forward_ops > 100 and all(g >= 0 for g in prog.grads[:-2]), fn


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "models")), reason="reference tree not present")
def test_shipped_small_graph_program_matches_oracle(lib_built):
    text = open(os.path.join(REF, "models", "nanochat_smoke_d1_128.mlir")).read()
    mod = TrainingModule(text)
    g = torch.Generator().manual_seed(5)
    params = [torch.randn(s, generator=g) * 0.02 for s in mod.param_shapes]
    B, T = mod.data_types[0].shape
    V = mod.param_shapes[0][0]
    ids = torch.randint(0, V, (B, T), generator=g)
    tg = torch.randint(0, V, (B, T), generator=g)
    prog = gp.parse(graph_describe(text))
    mp = mod._model_params(params)
    loss, grads = gp.run(prog, mp + [ids, tg])
    want = mod.model_forward_pass_grad(mp, ids, tg, 1.0)
    assert float(loss) == float(mod.forward(params, ids, tg))
    for a, w in zip(grads, want):
        assert torch.equal(a, w)


def test_malformed_attributes_are_refused_not_indexed_with(lib_built):
    """Dimension numbers that do not fit their operands (a permutation with a repeated or out-of-range entry, broadcast /
    reduce / concatenate / iota dimensions beyond the rank, a slice past the end, contracting dimensions that do not
    exist) end with PCPB_E_ARTIFACT and a reason."""
    import re
    cfg, text = make_model(helpers.SMALL_F32)

    def first(pattern, repl):
        out, n = re.subn(pattern, repl, text, count=1)
        assert n == 1, pattern
        return out

    bad = {
        "transpose": first(r"(stablehlo\.transpose %\w+, dims = )\[1, 0\]", r"\1[1, 1]"),
        "transpose range": first(r"(stablehlo\.transpose %\w+, dims = )\[0, 2, 1, 3\]", r"\1[0, 2, 1, 7]"),
        "broadcast_in_dim": first(r"(stablehlo\.broadcast_in_dim %\w+, dims = )\[0, 1, 2\]", r"\1[0, 1, 5]"),
        "reduce": first(r"(across dimensions = )\[2\]", r"\1[4]"),
        "slice": first(r"\[0:(\d+), 0:(\d+), 0:(\d+), 0:8\]", r"[0:\1, 0:\2, 0:\3, 0:99]"),
        "concatenate": first(r"(stablehlo\.concatenate %\w+, %\w+, dim = )3", r"\g<1>9"),
        "dot_general": first(r"contracting_dims = \[1\] x \[0\]", "contracting_dims = [3] x [0]"),
        "iota": first(r"stablehlo\.iota dim = 0", "stablehlo.iota dim = 6"),
    }
    for what, t in bad.items():
        with pytest.raises(BackendError) as ei:
            graph_describe(t)
        assert ei.value.code == bk.E_ARTIFACT, what
        assert what.split()[0] in str(ei.value), (what, str(ei.value))


def _plan(text):
    t = graph_describe(text, with_plan=True)
    prog = gp.parse(t)
    head, pv, po = None, {}, {}
    for ln in t.split("\n"):
        f = ln.split(" ")
        if f[0] == "plan":
            head = dict(x.split("=") for x in f[1:])
        elif f[0] == "pv":
            pv[int(f[1])] = {k: int(v) for k, v in (x.split("=") for x in f[2:])}
        elif f[0] == "po":
            d = dict(x.split("=") for x in f[2:])
            po[int(f[1])] = {k: (tuple(int(y) for y in v.split(":")) if ":" in v else int(v)) for k, v in d.items()}
    return prog, {k: int(v) for k, v in head.items()}, pv, po


def _shipped_or_exported(name):
    if name.endswith(".mlir"):
        path = os.path.join(REF, "models", name)
        if not os.path.exists(path):
            pytest.skip("reference tree not present")
        return open(path).read()
    return make_model(getattr(helpers, name))[1]


@pytest.mark.parametrize("name", ["SMALL_F32", "GPT_SMALL_BF16", "GPT_HD64_F32", "nanochat_d4_b4_t2048_bf16.mlir", "nanogpt_medium.mlir"])
def test_executor_plan_invariants(lib_built, name):
    """The executor's plan of a program, checked without a device: every kernel reads values that exist when it runs
    (defined earlier, not yet released), two values whose lifetimes overlap never share arena bytes, results are never
    released, dropped guards and views share storage with their operand, an absorbed broadcast has no storage and its
    one reader takes the source."""
    text = _shipped_or_exported(name)
    prog, head, pv, po = _plan(text)
    INF = 10 ** 9
    root = {v: d["root"] for v, d in pv.items()}
    R = lambda v: pv[root[v]]
    is_view = lambda i, op: op.kind == "reshape" or (op.kind == "convert" and prog.vals[op.ins[0]].dtype == prog.vals[op.out].dtype) or po[i]["skip"]
    producer = {op.out: i for i, op in enumerate(prog.ops)}
    kernels = 0
    for i, op in enumerate(prog.ops):
        f = po[i]
        if not f["need"] or f["const"]:
            continue
        if f["skip"]:
            assert op.kind == "guard_clamp" and root[op.out] == root[op.ins[0]]
            continue
        if f["absorbed"]:
            assert op.kind == "bcast" and root[op.out] == op.out and pv[op.out]["placed_at"] == -1
            readers = [(j, o) for j, o in enumerate(prog.ops) if po[j]["need"] and not is_view(j, o) and any(root[x] == op.out for x in o.ins)]
            assert len(readers) == 1 and readers[0][1].kind == "binary"
            j, o = readers[0]
            k = [root[x] for x in o.ins].index(op.out)
            assert po[j]["oa" if k == 0 else "ob"] == (po[j]["oa" if k == 0 else "ob"][0], op.ins[0]) and po[j]["oa" if k == 0 else "ob"][0] in (1, 2, 3)
            continue
        if is_view(i, op):
            assert root[op.out] == root[op.ins[0]]
            continue
        kernels += 1
        ins = list(op.ins)
        if op.kind in ("binary", "compare", "select"):
            first = 1 if op.kind == "select" else 0         # select: its two value operands
            for k, key in enumerate(("oa", "ob")):
                mode, src = f[key]
                ins[first + k] = None if mode == 4 else (src if mode in (1, 2, 3) else ins[first + k])
        for x in ins:
            if x is None:
                continue
            r = R(x)
            if r["where"] == 2:
                assert 0 <= r["placed_at"] < i and (r["freed_after"] == -1 or r["freed_after"] >= i), (i, op.kind, x, r)
            elif r["where"] == 1:
                assert po[producer[root[x]]]["const"] and po[producer[root[x]]]["need"]      # a constant that is materialised
            else:
                assert root[x] in prog.args
        ro = R(op.out)
        assert ro["where"] == 2 and 0 <= ro["placed_at"] <= i and (ro["freed_after"] == -1 or ro["freed_after"] >= i), (i, op.kind, ro)
        assert ro["off"] + ro["bytes"] <= head["arena"]
    assert kernels > 100
    for v in [prog.ret] + [g for g in prog.grads if g >= 0]:
        assert R(v)["freed_after"] == -1
    live = sorted((d["off"], d["off"] + d["bytes"], d["placed_at"], d["freed_after"] if d["freed_after"] >= 0 else INF, v)
                  for v, d in pv.items() if root[v] == v and d["where"] == 2 and d["placed_at"] >= 0)
    for a in range(len(live)):
        for b in range(a + 1, len(live)):
            if live[b][0] >= live[a][1]:
                break                                        # sorted by offset: no later one overlaps a in memory
            A, B = live[a], live[b]
            assert A[3] < B[2] or B[3] < A[2], (A, B)        # lifetimes apart


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_op_zoo_program_matches_oracle(lib_built, dtype):
    """Ops and op forms outside the model exporters' repertoire (tests/graph_zoo.py), in f32 and with every f32
    replaced by bf16 (the -inf literal then takes the sanitiser's hex rewrite)."""
    from graph_zoo import ZOO_BATCH, ZOO_BLOCK, ZOO_MLIR, ZOO_PARAM_SHAPES, ZOO_VOCAB
    text = ZOO_MLIR.replace("f32", dtype)
    f = inspect_artifact(text)
    assert f["family"] == "graph" and (f["batch"], f["block"], f["num_tensors"], f["total_params"]) == (ZOO_BATCH, ZOO_BLOCK, 3, 90)
    mod = TrainingModule(text)
    g = torch.Generator().manual_seed(0)
    params = mod._model_params([torch.randn(s, generator=g) * 0.5 for s in ZOO_PARAM_SHAPES])
    ids = torch.randint(0, ZOO_VOCAB, (ZOO_BATCH, ZOO_BLOCK), generator=g)
    tg = torch.randint(0, ZOO_VOCAB, (ZOO_BATCH, ZOO_BLOCK), generator=g)
    prog = gp.parse(graph_describe(text))
    loss, grads = gp.run(prog, params + [ids, tg])
    want = mod.model_forward_pass_grad(params, ids, tg, 1.0)
    assert float(loss) == float(mod.forward([p.to(torch.float32) for p in params], ids, tg))
    for a, w in zip(grads, want):
        assert torch.equal(a, w) and float(w.abs().max()) > 0
