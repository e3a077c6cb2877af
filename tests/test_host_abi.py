"""Host-side checks that need no GPU: the shared library loads and exports every function include/pcp_b200.h
declares, the artefact recogniser, and loud failure without a device."""
import os
import re

import pytest

from pcp_b200 import Backend, BackendError, NanochatConfig, nanochat_forward_mlir
from pcp_b200 import backend as bk
from pcp_b200.backend import inspect_artifact, load_library

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("PCP_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))


def declared_functions():
    hdr = open(os.path.join(ROOT, "include", "pcp_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    return sorted(set(re.findall(r"\b(pcpb_[a-z0-9_]+)\s*\(", hdr)))


def test_library_exports_every_declared_symbol(lib_built):
    lib = load_library()
    names = declared_functions()
    assert len(names) >= 30
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    assert sorted(bk.EXPORTS) == names, set(bk.EXPORTS) ^ set(names)


def test_header_cites_reference_interfaces():
    hdr = open(os.path.join(ROOT, "include", "pcp_b200.h")).read()
    for cite in ("src/backends/iree.zig", "src/backends/worker_backend.zig", "src/nodes/workers/worker.zig",
                 "src/algorithms/diloco.zig", "src/optimizers/nesterov.zig", "src/data/loader.zig"):
        assert cite in hdr


def test_inspect_artifact(lib_built):
    cfg = NanochatConfig(vocab=65536, d_model=256, n_layer=3, n_head=8, n_kv_head=4, seq_len=64, batch=2, dtype="bf16")
    f = inspect_artifact(nanochat_forward_mlir(cfg))
    assert (f["vocab"], f["d_model"], f["n_layer"], f["n_head"], f["n_kv_head"], f["head_dim"]) == (65536, 256, 3, 8, 4, 32)
    assert (f["d_ff"], f["batch"], f["block"], f["dtype"], f["num_tensors"]) == (1024, 2, 64, bk.BF16, 20)
    assert f["total_params"] == cfg.num_params()
    for bad in ("", "module {}", "func.func @main(%arg0: tensor<4xf32>) -> tensor<f32> {"):
        with pytest.raises(BackendError) as ei:
            inspect_artifact(bad or " ")
        assert ei.value.code == bk.E_ARTIFACT


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "models")), reason="reference tree not present")
def test_inspect_shipped_reference_graphs(lib_built):
    f = inspect_artifact(open(os.path.join(REF, "models", "nanochat_d8_b8_t2048_bf16.mlir")).read())
    assert (f["d_model"], f["n_layer"], f["n_head"], f["n_kv_head"], f["head_dim"], f["batch"], f["block"]) == (256, 8, 8, 4, 32, 8, 2048)
    assert f["total_params"] == 39321600
    f = inspect_artifact(open(os.path.join(REF, "models", "nanochat_d12_b6_t2048.mlir")).read())
    assert (f["d_model"], f["n_layer"], f["head_dim"], f["dtype"], f["total_params"]) == (768, 12, 128, bk.F32, 185597952)
    f = inspect_artifact(open(os.path.join(REF, "models", "nanogpt_small.mlir")).read())          # nanoGPT family
    assert (f["d_model"], f["n_layer"], f["n_head"], f["head_dim"], f["num_tensors"], f["total_params"]) == (64, 2, 4, 16, 22, 109377)
    f = inspect_artifact(open(os.path.join(REF, "models", "nanogpt_medium_bf16.mlir")).read())
    assert (f["d_model"], f["n_layer"], f["n_head"], f["dtype"], f["total_params"]) == (256, 4, 8, bk.BF16, 3314432)


def test_no_cpu_fallback(lib_built):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(BackendError) as ei:
        Backend(0)
    assert ei.value.code == bk.E_CUDA


def test_d20_parameter_count():
    cfg = NanochatConfig(vocab=65536, d_model=1280, n_layer=20, n_head=10, n_kv_head=10, seq_len=2048, batch=32, dtype="bf16")
    assert cfg.num_params() == 560_988_160 and len(cfg.param_shapes()) == 122
    d8 = NanochatConfig(vocab=65536, d_model=512, n_layer=8, n_head=4, n_kv_head=4, seq_len=2048, batch=8, dtype="bf16")
    assert d8.num_params() == 92_274_688


def test_recogniser_refuses_same_signature_other_body(lib_built, monkeypatch):
    """A graph with the nanochat parameter list but another body (no ReLU^2, a norm dropped, GELU-like ops, another
    ignore index) must not be trained with the built-in nanochat arithmetic: the fused recogniser refuses it
    (PCPB_FRONTEND=fused: no other path), and by default it goes to the general front end, op by op."""
    monkeypatch.setenv("PCPB_FRONTEND", "fused")
    cfg = NanochatConfig(vocab=97, d_model=64, n_layer=2, n_head=4, n_kv_head=2, seq_len=16, batch=2, dtype="f32")
    good = nanochat_forward_mlir(cfg)
    inspect_artifact(good)
    lines = good.split("\n")

    def replace_first(op_from, op_to):
        out, done = [], False
        for ln in lines:
            if not done and f"= stablehlo.{op_from} " in ln:
                ln = ln.replace(f"stablehlo.{op_from} ", f"stablehlo.{op_to} ", 1)
                done = True
            out.append(ln)
        assert done
        return "\n".join(out)

    mutated = {
        "relu -> abs (no ReLU)": replace_first("maximum", "abs"),
        "one rsqrt -> sqrt (a norm changed)": replace_first("rsqrt", "sqrt"),
        "soft-cap tanh -> logistic": replace_first("tanh", "logistic"),
        "softmax exp -> tanh": replace_first("exponential", "tanh"),
        "other ignore index": good.replace("dense<-1>", "dense<-7>"),
    }
    for what, text in mutated.items():
        with pytest.raises(BackendError) as ei:
            inspect_artifact(text)
        assert ei.value.code == bk.E_ARTIFACT, what
    monkeypatch.delenv("PCPB_FRONTEND")
    for what, text in mutated.items():
        if "abs" in what:               # abs with two operands is not StableHLO: refused by both
            with pytest.raises(BackendError):
                inspect_artifact(text)
            continue
        assert inspect_artifact(text)["family"] == "graph", what
    assert inspect_artifact(good)["family"] == "fused"


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "models")), reason="reference tree not present")
def test_every_shipped_reference_graph_is_recognised(lib_built):
    """All forward graphs under the reference's models/ load: both families, f32 and bf16, head widths 16 / 32 / 128."""
    import glob
    files = sorted(glob.glob(os.path.join(REF, "models", "*.mlir")))
    assert len(files) >= 17
    widths = set()
    for fn in files:
        f = inspect_artifact(open(fn).read())
        assert f["n_head"] * f["head_dim"] == f["d_model"] and f["n_head"] % f["n_kv_head"] == 0, fn
        assert f["total_params"] > 0 and f["dtype"] in (bk.F32, bk.BF16), fn
        widths.add(f["head_dim"])
    assert widths == {16, 32, 128}
