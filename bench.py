#!/usr/bin/env python
"""Benchmark of the training hot path: nanochat-d20 bf16 DiLoCo inner steps, one worker per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload d20|d8|tiny]

A step is one inner step of the worker loop on one synthetic FIFO batch per GPU: forward, reverse-AD backward and
the fused AdamW update (src/nodes/workers/worker.zig:1119-1339 done on the device).  The N=1 workload is
BASELINE.json configs[2] at one GPU: nanochat d20 (d_model 1280, 10 heads x 128, 20 layers, vocab 65536, soft-cap
15), B=32, T=2048, Zipf(1.1) u16 tokens from a per-rank seed.

value     tokens/s over all ranks with the round's token chunk already in HBM (device-timed, max over ranks)
e2e       the same through the C ABI from HOST memory: each step copies its token window from pinned host
          memory and reads its loss back; the round's parameter blob upload and delta download are inside the
          timed region and counted in the byte figures
roofline  the tensor-core GEMM kernel (dominant): algorithmic 2*M*N*K FLOPs of its launches / their summed
          CUDA-event durations, against the measured sustained bf16 peak
cpu_baseline  the CPU oracle (restated reference path) on a bounded sample, rank 0 at N=1 only

With --impl reference the oracle itself is timed on the host cores (the reference's IREE llvm-cpu path cannot be
installed offline); only rank 0 works.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # BASELINE.json configs[2] (per GPU)
    "d20": dict(vocab=65536, d_model=1280, n_layer=20, n_head=10, n_kv_head=10, seq_len=2048, batch=32, dtype="bf16"),
    # BASELINE.json configs[1]
    "d8": dict(vocab=65536, d_model=512, n_layer=8, n_head=4, n_kv_head=4, seq_len=2048, batch=8, dtype="bf16"),
    # d8 geometry at a quarter of the batch: small enough for an `ncu --set full` capture
    "d8b2": dict(vocab=65536, d_model=512, n_layer=8, n_head=4, n_kv_head=4, seq_len=2048, batch=2, dtype="bf16"),
    "tiny": dict(vocab=4096, d_model=256, n_layer=2, n_head=2, n_kv_head=2, seq_len=256, batch=4, dtype="bf16"),
    # BASELINE.json configs[0]: nanoGPT-small fp32 (char vocabulary 65, 6 layers, 6 heads, d_model 384, T=256, B=64, GELU)
    "c1": dict(vocab=65, d_model=384, n_layer=6, n_head=6, seq_len=256, batch=64, dtype="f32", activation="gelu"),
    # BASELINE.json configs[3] per GPU: nanoGPT-medium bf16 (head dim 64, tanh-GELU MLP, learned positions, LayerNorm)
    "gptm": dict(vocab=50304, d_model=1024, n_layer=24, n_head=16, seq_len=1024, batch=16, dtype="bf16", activation="gelu"),
    # nanoGPT-medium layer geometry at a profiling size
    "gptml2b8": dict(vocab=50304, d_model=1024, n_layer=2, n_head=16, seq_len=1024, batch=8, dtype="bf16", activation="gelu"),
    # d20 layer geometry at profiling sizes (the kernels and their shapes per token are those of d20)
    "d20l1b8": dict(vocab=4096, d_model=1280, n_layer=1, n_head=10, n_kv_head=10, seq_len=2048, batch=8, dtype="bf16"),
    "d20l2b2": dict(vocab=65536, d_model=1280, n_layer=2, n_head=10, n_kv_head=10, seq_len=2048, batch=2, dtype="bf16"),
    "d20l2b4": dict(vocab=65536, d_model=1280, n_layer=2, n_head=10, n_kv_head=10, seq_len=2048, batch=4, dtype="bf16"),
    "d8ship": dict(vocab=65536, d_model=256, n_layer=8, n_head=8, n_kv_head=4, seq_len=2048, batch=8, dtype="bf16"),
    "d12ship": dict(vocab=65536, d_model=768, n_layer=12, n_head=6, n_kv_head=6, seq_len=2048, batch=6, dtype="f32"),
    "d20l2b16": dict(vocab=65536, d_model=1280, n_layer=2, n_head=10, n_kv_head=10, seq_len=2048, batch=16, dtype="bf16"),
}
DESCR = {
    "d20": "nanochat-d20 bf16 DiLoCo inner step, B=32/GPU, T=2048, AdamW(lr 1e-3, 0.9/0.95, wd 0.1), H=50",
    "d8": "nanochat-d8 (d=512) bf16 inner step, B=8, T=2048, AdamW lr 1e-3",
    "d8b2": "nanochat-d8 (d=512) bf16 inner step, B=2, T=2048 (profiling size)",
    "tiny": "nanochat tiny bf16 inner step (smoke size)",
    "c1": "nanoGPT-small fp32 inner step (6L, d=384, 6 heads x 64, GELU, char vocab 65), B=64, T=256, AdamW(3e-4, 0.9/0.95, wd 0.1)",
    "gptm": "nanoGPT-medium bf16 DiLoCo inner step (24L, d=1024, 16 heads x 64, GELU), B=16/GPU, T=1024, V=50304",
    "gptml2b8": "two nanoGPT-medium layers + its LM head, B=8, T=1024 (attention / LayerNorm profiling size)",
    "d20l1b8": "one d20 layer (d=1280, 10 heads x 128), V=4096, B=8, T=2048 (attention profiling size)",
    "d20l2b2": "two d20 layers + the d20 LM head, B=2, T=2048 (GEMM DRAM-traffic profiling size)",
    "d20l2b4": "two d20 layers + the d20 LM head, B=4, T=2048 (GEMM DRAM-traffic profiling size)",
    "d8ship": "the shipped models/nanochat_d8_b8_t2048_bf16.mlir shape: d=256, 8 query / 4 kv heads x 32, 8 layers, B=8, T=2048",
    "d12ship": "the shipped models/nanochat_d12_b6_t2048.mlir shape: fp32, d=768, 6 heads x 128, 12 layers, B=6, T=2048",
    "d20l2b16": "two d20 layers + the d20 LM head, B=16, T=2048 (LM-head DRAM-traffic profiling size: 128 row tiles)",
}
# BASELINE.json configs[4]: Qwen3-8B-shaped bf16 rollout generation, one replica per GPU
ROLLOUT = dict(vocab=151936, d_model=4096, n_layer=36, n_head=32, n_kv_head=8, head_dim=128, d_ff=12288, batch=16, prompt=512,
               new_tokens=256, page_tokens=16, rope_theta=1e6, rms_eps=1e-6)
ROLLOUT_DESCR = ("Qwen3-8B-shaped bf16 rollout generation (36L, d=4096, 32q/8kv heads x 128, SwiGLU 12288, V=151936, N(0,0.02) weights), "
                 "16 prompts x 512 uniform tokens, greedy decode of 256 tokens, paged KV cache (16-token pages)")
ADAM = {"c1": dict(learning_rate=3e-4, beta1=0.9, beta2=0.95, epsilon=1e-8, weight_decay=0.1, max_grad_norm=1.0)}
ADAM_DEFAULT = dict(learning_rate=1e-3, beta1=0.9, beta2=0.95, epsilon=1e-8, weight_decay=0.1, max_grad_norm=1.0)
H_INNER = 50
# ncu: dram read + write of the LM-head forward launch at the d20 width and vocabulary, per output row (B=16 capture:
# 1.50 GB read + 4.25 GB written for 32768 rows; both grow with the rows: the weights are re-read once per 8192 rows)
LMHEAD_TRAFFIC_BYTES_PER_ROW = 0.1756e6
PEAKS_FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def make_model(cfgd):
    """(config, forward StableHLO text) of a workload: nanochat family when it names n_kv_head, else nanoGPT."""
    from pcp_b200 import NanochatConfig, NanoGPTConfig, nanochat_forward_mlir, nanogpt_forward_mlir
    if "n_kv_head" in cfgd:
        cfg = NanochatConfig(**cfgd)
        return cfg, nanochat_forward_mlir(cfg)
    cfg = NanoGPTConfig(**cfgd)
    return cfg, nanogpt_forward_mlir(cfg)


def flops_per_token(c):
    d, L, T, V = c["d_model"], c["n_layer"], c["seq_len"], c["vocab"]
    dkv = c.get("n_kv_head", c["n_head"]) * (d // c["n_head"])
    n_mm = L * (2 * d * d + 2 * d * dkv + 2 * d * 4 * d) + V * d
    return 6 * n_mm + 6 * L * T * d, 6 * n_mm + 12 * L * T * d


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return d, "measured"
    return dict(PEAKS_FALLBACK), "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples of one GPU while the timed region runs."""

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thr = threading.Thread(target=self._read, daemon=True)
            self.thr.start()
        except OSError:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, val in zip(names, f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def sample_inputs(cfgd, steps, seq, batch):
    """Seeded inputs of the bounded CPU sample: (config, graph text, f32 parameter list, token stream).  The GPU parity
    leg rebuilds exactly these."""
    import torch

    from pcp_b200.synthetic import zipf_tokens
    cfg, text = make_model(dict(cfgd, batch=batch, seq_len=seq))
    g = torch.Generator().manual_seed(0)
    params = [(torch.randn(s, generator=g) * 0.02) for s in cfg.param_shapes()]
    tokens = zipf_tokens((steps + 1) * (batch * seq + 1), cfg.vocab, 1.1, 0)
    return cfg, text, params, tokens


def cpu_oracle_run(cfgd, workload, steps=1, threads=None, seq=256, batch=1):
    """`steps` inner steps (compute_gradients + apply_optimizer) of the CPU oracle on a sample of the workload: the same
    architecture with batch `batch` and T=`seq`.  -> dict(tokens_per_s, seconds, threads, sample, losses)."""
    import torch

    from oracle.loader import FifoU16
    from oracle.optim import AdamConf
    from oracle.worker import TrainingModule
    # all host cores this process may use; a launcher (torchrun) that exports OMP_NUM_THREADS=1 must not turn the
    # reference into a single-threaded run
    torch.set_num_threads(threads or len(os.sched_getaffinity(0)))
    cfg, text, params, tokens = sample_inputs(cfgd, steps, seq, batch)
    mod = TrainingModule(text)
    m = [torch.zeros_like(p) for p in params]
    v = [torch.zeros_like(p) for p in params]
    ds = FifoU16(tokens)
    a = ADAM.get(workload, ADAM_DEFAULT)
    conf = AdamConf(learning_rate=a["learning_rate"], beta1=a["beta1"], beta2=a["beta2"], epsilon=a["epsilon"],
                    weight_decay=a["weight_decay"], max_grad_norm=a["max_grad_norm"])
    losses = []
    t0 = time.perf_counter()
    for s in range(steps):
        x, y = ds.get_batch(batch, seq)
        grads, loss = mod.compute_gradients(params, torch.from_numpy(x), torch.from_numpy(y))
        params, m, v = mod.apply_optimizer(params, grads, m, v, float(s + 1), conf)
        losses.append(float(loss))
    dt = time.perf_counter() - t0
    whole = (batch, seq) == (cfgd["batch"], cfgd["seq_len"])
    sample = (f"{cfgd['n_layer']}L d={cfgd['d_model']} V={cfgd['vocab']} B={batch} T={seq}, {steps} inner step(s) "
              f"(compute_gradients + apply_optimizer) on the torch-CPU oracle")
    if not whole:
        sample += (f"; bounded sample of the B={cfgd['batch']} T={cfgd['seq_len']} workload: every CPU step still runs AdamW "
                   "over all parameters and reads the whole LM head for these few tokens, a fixed cost the full step "
                   "would amortise over many more tokens, so this figure is biased low")
    return {"tokens_per_s": steps * batch * seq / dt, "seconds": dt, "threads": torch.get_num_threads(), "sample": sample,
            "losses": losses, "same_config": whole}


def gpu_losses_on_sample(cfgd, workload, steps, seq, batch, device=0):
    """The same `steps` inner steps as cpu_oracle_run on the same seeded inputs, on the GPU through the C ABI."""
    from pcp_b200 import F32, Backend
    cfg, text, params, tokens = sample_inputs(cfgd, steps, seq, batch)
    blob = np.concatenate([p.numpy().reshape(-1) for p in params]).astype(np.float32)
    with Backend(device) as be:
        be.load_session(text)
        be.set_adam(**ADAM.get(workload, ADAM_DEFAULT))
        be.worker_begin_round(steps, blob, param_dtype=F32)
        be.worker_set_tokens(tokens)
        for _ in range(steps):
            be.worker_step()
        _, losses = be.worker_end_round(steps, param_dtype=F32, want_delta=False)
    return [float(x) for x in losses]


def parity_object(gpu_losses, cpu_losses, dtype):
    tol = 1e-4 if dtype == "f32" else 2e-2
    rel = [abs(a - b) / abs(b) for a, b in zip(gpu_losses, cpu_losses)]
    return {"loss_gpu": gpu_losses, "loss_oracle": cpu_losses, "rel_err": max(rel) if rel else None, "tol": tol,
            "ok": bool(rel) and max(rel) <= tol,
            "what": "per-step loss of the same seeded inner steps on the GPU (C ABI) and on the CPU oracle"}


def run_reference_rollout(args):
    """The restated generation loop (one token per call, dense cache, host arg-max) on the host cores, on a bounded
    sample of the rollout workload: the full width, vocabulary and head geometry, 2 of the 36 layers, one sequence."""
    import torch

    from oracle.rollout import QwenConfig, generate, seeded_params
    c = ROLLOUT
    torch.set_num_threads(len(os.sched_getaffinity(0)))
    prompt_len, new = 32, 8
    cfg = QwenConfig(vocab=c["vocab"], d_model=c["d_model"], n_layer=2, n_head=c["n_head"], n_kv_head=c["n_kv_head"],
                     head_dim=c["head_dim"], d_ff=c["d_ff"], max_seq=prompt_len + new, dtype="bf16")
    params = [p.to(torch.bfloat16) for p in seeded_params(cfg, seed=0, std=0.02)]
    prompt = np.random.default_rng(0).integers(0, cfg.vocab, size=prompt_len).tolist()
    K = max(1, args.steps)
    t0 = time.perf_counter()
    for _ in range(K):
        generate(cfg, params, prompt, new)
    dt = time.perf_counter() - t0
    tps = K * new / dt
    sample = (f"2 of {c['n_layer']} layers at full width (d={c['d_model']}, V={c['vocab']}), 1 sequence, prompt {prompt_len}, {new} new tokens "
              "on the torch-CPU oracle, token by token like the reference's loop; per-token cost of the full model is about "
              f"{c['n_layer']}/2 times the layer part of this")
    line = {"impl": "reference", "metric": "rollout_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": K,
            "warmup": args.warmup, "ms_per_step": 1e3 * dt / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": {"workload": ROLLOUT_DESCR, "reference_arm": "CPU oracle; bounded sample",
                                                             "same_config": False},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)
    return 0


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return 0
    if args.workload == "qwen3_rollout":
        return run_reference_rollout(args)
    cfgd = WORKLOADS[args.workload]
    whole = args.workload == "c1"                       # small enough to time whole on the host cores
    seq, batch = (cfgd["seq_len"], cfgd["batch"]) if whole else (128, 1)
    # warm-up is one short call (imports, allocator); every timed step is one inner step of the sample
    if args.warmup > 0:
        cpu_oracle_run(dict(cfgd, n_layer=1), args.workload, steps=1, seq=min(64, seq), batch=1)
    r = cpu_oracle_run(cfgd, args.workload, steps=max(1, args.steps), seq=seq, batch=batch)
    tps, dt, threads = r["tokens_per_s"], r["seconds"], r["threads"]
    # the reference's CPU worker drives IREE's local-sync device, a single-threaded synchronous executor
    # (src/backends/selection.zig:66): the same sample on one thread, one step
    one = cpu_oracle_run(cfgd, args.workload, steps=1, threads=1, seq=seq, batch=batch)
    line = {
        "impl": "reference", "metric": "train_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": max(1, args.steps), "warmup": args.warmup, "ms_per_step": 1e3 * dt / max(1, args.steps),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": cfgd["dtype"], "data": "synthetic",
        "config": {"workload": DESCR[args.workload], "reference_arm": "CPU oracle (the reference's IREE llvm-cpu path "
                   "is not installable offline)" + ("" if whole else "; bounded sample"), "same_config": r["same_config"]},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": r["sample"],
                         "one_thread": {"value": one["tokens_per_s"], "unit": "tokens/s", "cores": 1, "steps": 1,
                                        "why": "the reference's CPU worker uses IREE local-sync, a single-threaded driver"}},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if not whole and not args.no_other_configs:
        # one configuration timed whole, so that one GPU / CPU ratio is a same-configuration one: BASELINE configs[0]
        c1 = cpu_oracle_run(WORKLOADS["c1"], "c1", steps=2, seq=WORKLOADS["c1"]["seq_len"], batch=WORKLOADS["c1"]["batch"])
        line["other_configs"] = [{"workload": "c1", "descr": DESCR["c1"], "value": c1["tokens_per_s"], "unit": "tokens/s",
                                  "cores": c1["threads"], "same_config": True, "sample": c1["sample"]}]
    print(json.dumps(line), flush=True)
    return 0


def time_workload(name, steps, warmup, device, peaks):
    """A few device-timed inner steps of another BASELINE configuration with its tokens resident in HBM."""
    import torch

    from pcp_b200 import BF16, F32, Backend
    from pcp_b200.synthetic import uniform_tokens, zipf_tokens
    cfgd = WORKLOADS[name]
    cfg, text = make_model(cfgd)
    bf16 = cfgd["dtype"] == "bf16"
    dt = BF16 if bf16 else F32
    BT = cfg.batch * cfg.seq_len
    n_tok = (steps + warmup + 1) * (BT + 1)
    tokens = zipf_tokens(n_tok, cfg.vocab, 1.1, seed=0) if "n_kv_head" in cfgd else uniform_tokens(n_tok, cfg.vocab, seed=0)
    tok_dev = torch.from_numpy(tokens.view(np.int16)).to(f"cuda:{device}")
    with Backend(device) as be:
        be.load_session(text)
        be.set_adam(**ADAM.get(name, ADAM_DEFAULT))
        blob = be.init_master(0, dt)
        if "n_kv_head" not in cfgd:                       # LayerNorm weights at 1 (a N(0, 0.02) scale would zero the block)
            at = 0
            one = np.uint16(0x3F80) if bf16 else np.float32(1.0)
            shapes = cfg.param_shapes()
            for i, s_ in enumerate(shapes):
                n = int(np.prod(s_))
                if len(s_) == 1 and i < len(shapes) - 1 and (i - 2) % 2 == 0:
                    blob[at:at + n] = one
                at += n
        be.worker_begin_round(steps + warmup, blob, param_dtype=dt, tokens_on_device=True)
        be.worker_set_tokens(device_ptr=tok_dev.data_ptr(), n_tokens=n_tok)
        for _ in range(warmup):
            be.worker_step()
        be.synchronize()
        l0 = be.launch_count
        be.timer_start()
        for _ in range(steps):
            be.worker_step()
        ms = be.timer_stop()
        launches = be.launch_count - l0
        _, losses = be.worker_end_round(steps + warmup, param_dtype=dt, want_delta=False)
    fcausal, _ = flops_per_token(cfgd)
    tps = steps * BT / (ms / 1e3)
    peak_burst = peaks.get("bf16_tflops", PEAKS_FALLBACK["bf16_tflops"]) * 1e12
    return {"workload": name, "descr": DESCR[name], "value": tps, "unit": "tokens/s", "ms_per_step": ms / steps, "steps": steps,
            "warmup": warmup, "dtype": cfgd["dtype"], "gpu_launches": int(launches),
            "flops_per_token_causal": fcausal, "achieved_tflops": tps * fcausal / 1e12,
            "mfu_vs_measured_burst_bf16": tps * fcausal / peak_burst,
            "loss_first_last": [float(losses[warmup]), float(losses[-1])]}


def rollout_param_count(c):
    hq, hk = c["n_head"] * c["head_dim"], c["n_kv_head"] * c["head_dim"]
    per = c["d_model"] * (hq + 2 * hk) + hq * c["d_model"] + 2 * c["head_dim"] + 3 * c["d_model"] * c["d_ff"] + 2 * c["d_model"]
    return 2 * c["vocab"] * c["d_model"] + c["n_layer"] * per + c["d_model"]


def time_rollout(device, steps, warmup, peaks, c=None):
    """Rollouts of the Qwen3-8B-shaped configuration: device-timed (prefill + decode) and end to end through the C ABI
    call (host prompts in, host tokens out)."""
    from pcp_b200.backend import Rollout
    c = c or ROLLOUT
    rng = np.random.default_rng(0)
    prompts = rng.integers(0, c["vocab"], size=(c["batch"], c["prompt"])).tolist()
    with Rollout(device, c["vocab"], c["d_model"], c["n_layer"], c["n_head"], c["n_kv_head"], c["head_dim"], c["d_ff"],
                 max_seq=c["prompt"] + c["new_tokens"], max_batch=c["batch"], max_prompt=c["prompt"], page_tokens=c["page_tokens"],
                 rope_theta=c["rope_theta"], rms_eps=c["rms_eps"]) as eng:
        eng.random_weights(0, 0.02)
        for _ in range(warmup):
            eng.generate_rollout(prompts, c["new_tokens"])
        l0 = eng.launch_count
        pre = dec = wall = 0.0
        for _ in range(steps):
            t0 = time.perf_counter()
            toks, _, (p_ms, d_ms) = eng.generate_rollout(prompts, c["new_tokens"])
            wall += time.perf_counter() - t0
            pre += p_ms; dec += d_ms
        launches = eng.launch_count - l0
    n_new = c["batch"] * c["new_tokens"]
    weight_bytes = 2.0 * (rollout_param_count(c) - c["vocab"] * c["d_model"])     # the embedding is gathered, not streamed
    step_ms = dec / steps / max(1, c["new_tokens"] - 1)
    hbm = peaks.get("hbm_gbs", PEAKS_FALLBACK["hbm_gbs"])
    achieved = weight_bytes / (step_ms / 1e3) / 1e9
    return {"value": steps * n_new / ((pre + dec) / 1e3), "e2e": steps * n_new / wall, "prefill_ms": pre / steps, "decode_ms": dec / steps,
            "decode_step_ms": step_ms, "launches": int(launches), "weight_bytes_per_decode_step": weight_bytes,
            "roofline": {"kernel": "k_gemv16w (decode-step weight streaming: every weight byte read once per step for 16 rows)",
                         "bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm, "traffic": None,
                         "how": "algorithmic bytes = bf16 weights of all layers + LM head per decode step, over the mean device time "
                                "of a decode step (CUDA events around the decode loop); the step also reads the KV cache and runs the "
                                "norm / attention / arg-max kernels, so the GEMV kernel alone is above this figure"},
            "h2d_bytes": c["batch"] * c["prompt"] * 8, "d2h_bytes": n_new * 8, "first_tokens": [t[:4] for t in toks[:2]]}


def run_rollout(args):
    rank, world, local = dist_env()
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist_mod.init_process_group("gloo", rank=rank, world_size=world)
        dist = dist_mod
    peaks, peak_src = load_peaks()
    K, W = max(1, args.steps), max(args.warmup, 0)
    sampler = ClockSampler(local)
    if dist:
        dist.barrier()
    sampler.start()
    c = dict(ROLLOUT)
    if args.rollout_layers:                               # profiling sizes: fewer layers / tokens of the same kernels
        c["n_layer"] = args.rollout_layers
    if args.rollout_new:
        c["new_tokens"] = args.rollout_new
    r = time_rollout(local, K, W, peaks, c)
    clocks = sampler.stop()
    n_new = c["batch"] * c["new_tokens"]
    ms = r["prefill_ms"] + r["decode_ms"]
    e2e = r["e2e"]
    if dist:                                              # replicas only: no exchange between ranks; slowest rank sets the time
        import torch
        t = torch.tensor([ms, n_new / e2e], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e = float(t[0]), n_new / float(t[1])
    if rank != 0:
        return 0
    line = {"metric": "rollout_tokens_per_s", "value": world * n_new / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": {"workload": ROLLOUT_DESCR, "model": c, "parallelism": f"{world} independent replicas",
                                            "l2": "inputs larger than L2: every decode step streams 15 GB of weights"},
            "roofline": dict(r["roofline"], peak_source=f"{peak_src} copy bandwidth"),
            "e2e": {"value": world * e2e, "unit": "tokens/s", "h2d_bytes_per_step": r["h2d_bytes"], "d2h_bytes_per_step": r["d2h_bytes"],
                    "how": "wall clock around pcpb_rollout_generate: host prompts in, host tokens out"},
            "gpu_launches": r["launches"], "clocks": clocks, "prefill_ms": r["prefill_ms"], "decode_ms": r["decode_ms"],
            "decode_step_ms": r["decode_step_ms"]}
    print(json.dumps(line), flush=True)
    return 0


def run_ours(args):
    if args.workload == "qwen3_rollout":
        return run_rollout(args)
    import torch

    from pcp_b200 import BF16, F32, Backend
    from pcp_b200.synthetic import zipf_tokens, uniform_tokens

    rank, world, local = dist_env()
    if world != args.gpus and world > 1:
        args.gpus = world
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist_mod.init_process_group("gloo", rank=rank, world_size=world)
        dist = dist_mod
    cfgd = WORKLOADS[args.workload]
    cfg, text = make_model(cfgd)
    bf16 = cfgd["dtype"] == "bf16"
    PDT = BF16 if bf16 else F32
    K, W = args.steps, max(args.warmup, 0)
    BT = cfg.batch * cfg.seq_len
    P = cfg.num_params()
    peaks, peak_src = load_peaks()

    be = Backend(local)
    be.load_session(text)
    be.set_adam(**ADAM.get(args.workload, ADAM_DEFAULT))
    # parameters: 0.02 * N(0,1) from the library's master initialiser (src/algorithms/diloco.zig:513-586), bf16 by
    # truncation like the Shepherd's master copy; LayerNorm weights of the nanoGPT family at 1
    blob = be.init_master(0, PDT)
    if "n_kv_head" not in cfgd:
        at, shapes = 0, cfg.param_shapes()
        for i, s_ in enumerate(shapes):
            n = int(np.prod(s_))
            if len(s_) == 1 and i < len(shapes) - 1 and (i - 2) % 2 == 0:
                blob[at:at + n] = np.uint16(0x3F80) if bf16 else np.float32(1.0)
            at += n
    n_tok = (max(K + W, H_INNER) + 2) * (BT + 1)
    tokens = (zipf_tokens(n_tok, cfg.vocab, 1.1, seed=rank) if "n_kv_head" in cfgd
              else uniform_tokens(n_tok, cfg.vocab, seed=rank))
    pinned = torch.empty(n_tok, dtype=torch.int16).pin_memory() if torch.cuda.is_available() else torch.empty(n_tok, dtype=torch.int16)
    pinned.numpy().view(np.uint16)[:] = tokens
    tok_host = pinned.numpy().view(np.uint16)
    tok_dev = torch.from_numpy(tokens.view(np.int16)).to(f"cuda:{local}")

    def barrier():
        if dist:
            dist.barrier()

    def max_over_ranks(x):
        if not dist:
            return x
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    # ---------------- value: tokens resident in HBM; nothing but the K steps inside the timed region ----------------
    KP = min(K, 4)                                        # extra steps of the same round, profiled, after the timed ones
    be.worker_begin_round(K + W + KP, blob, param_dtype=PDT, tokens_on_device=True)
    be.worker_set_tokens(device_ptr=tok_dev.data_ptr(), n_tokens=n_tok)
    for _ in range(W):
        be.worker_step()
    be.synchronize()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    l0 = be.launch_count
    be.timer_start()
    for _ in range(K):
        be.worker_step()
    ms = be.timer_stop()
    launches = be.launch_count - l0
    clocks = sampler.stop()
    barrier()
    ms = max_over_ranks(ms)
    # roofline pass: the same steps again with every tensor-core GEMM launch bracketed by CUDA events (the events stay
    # out of the timed region above; no synchronisation happens between them)
    be.profile_enable(True)
    be.timer_start()
    for _ in range(KP):
        be.worker_step()
    prof_ms_total = be.timer_stop()
    prof = be.profile_read()
    be.profile_enable(False)
    _, losses = be.worker_end_round(K + W + KP, param_dtype=PDT, want_delta=False)
    tokens_total = world * K * BT
    value = tokens_total / (ms / 1e3)

    # ---------------- outer step (N > 1): reduce-scatter / Nesterov / all-gather over peer memory ----------------
    outer = None
    if world > 1:
        import hashlib
        handles = be.outer_export()
        gathered = [None] * world
        dist.all_gather_object(gathered, handles)
        be.outer_attach_ipc(rank, world, b"".join(gathered))
        barrier()
        times = []
        for _ in range(3):
            be.outer_prepare(param_dtype=PDT)
            barrier()
            t0 = time.perf_counter()
            dev_ms = be.outer_apply(0.7, 0.9, PDT)
            barrier()
            times.append((max_over_ranks(dev_ms), max_over_ranks(1e3 * (time.perf_counter() - t0))))
        dev_ms, wall_ms = min(times)
        # every rank must now hold the same master parameters: compare a checksum of each replica
        digest = hashlib.sha256(np.ascontiguousarray(be.worker_read_state("master")).tobytes()).hexdigest()
        digests = [None] * world
        dist.all_gather_object(digests, digest)
        round_ms = H_INNER * ms / K
        wire = 2 * (world - 1) / world * P * 4
        outer = {"outer_sync_ms": dev_ms, "outer_sync_wall_ms": wall_ms, "pct_of_round": 100.0 * wall_ms / (round_ms + wall_ms),
                 "wire_bytes_per_gpu": wire, "wire_gb_per_s_per_gpu": wire / (dev_ms / 1e3) / 1e9 if dev_ms else None,
                 "nvlink_peak_gb_per_s_per_direction": 770.0, "masters_identical_across_ranks": len(set(digests)) == 1,
                 "collective": "cuda-ipc p2p kernel (no NCCL; host barriers over gloo)",
                 "how": "P2P pull of f32 deltas + fused Nesterov + P2P push of the new master, host barriers on both sides"}

    # ---------------- e2e: host buffers through the C ABI ----------------
    # one DiLoCo round as the worker sees it: blob in, H inner steps from host token windows, delta out.  The default
    # run times a full round of H_INNER steps; short runs (--steps < 8) time K steps and amortise the blobs over those.
    Ke = H_INNER if K >= 8 else max(1, K)
    if n_tok < Ke * BT + 1:
        Ke = max(1, (n_tok - 1) // BT)
    # the round's parameter blob and delta blob live in pinned host memory, like the token windows
    if torch.cuda.is_available():
        blob_t = torch.from_numpy(blob.view(np.int16 if bf16 else np.float32)).pin_memory()
        blob = blob_t.numpy().view(np.uint16 if bf16 else np.float32)
        delta_t = torch.empty(P, dtype=torch.int16 if bf16 else torch.float32).pin_memory()
        delta_buf = delta_t.numpy().view(np.uint16 if bf16 else np.float32)
    else:
        delta_buf = None
    barrier()
    be.timer_start()
    be.worker_begin_round(Ke, blob, param_dtype=PDT, tokens_on_device=False)
    be.worker_set_tokens(device_ptr=tok_host.ctypes.data, n_tokens=n_tok)
    e2e_losses = []
    for _ in range(Ke):
        be.worker_step()
        e2e_losses.append(be.worker_last_loss())
    delta, _ = be.worker_end_round(Ke, param_dtype=PDT, want_delta=True, out=delta_buf)
    e2e_ms = max_over_ranks(be.timer_stop())
    e2e_value = world * Ke * BT / (e2e_ms / 1e3)
    h2d = (BT + 1) * 2 + blob.nbytes / Ke
    d2h = 4 + delta.nbytes / Ke
    be.close()

    if rank != 0:
        return 0

    fcausal, fpalm = flops_per_token(cfgd)
    per_gpu_tps = value / world
    peak_burst = peaks.get("bf16_tflops", PEAKS_FALLBACK["bf16_tflops"]) * 1e12
    peak_sust = peaks.get("bf16_tflops_sustained", PEAKS_FALLBACK["bf16_tflops_sustained"]) * 1e12
    achieved = prof["flops"] / (prof["ms"] / 1e3) / 1e12 if prof["ms"] > 0 else 0.0
    # DRAM traffic of the largest tensor-core GEMM launch of the step, the LM-head forward [B*T x V x d], from ncu
    # captures at B=2 and B=4 of the d20 width and vocabulary; it grows in proportion to the rows.
    traffic, traffic_note = None, None
    if (cfgd["d_model"], cfgd["vocab"]) == (1280, 65536):
        rows = cfgd["batch"] * cfgd["seq_len"]
        traffic = LMHEAD_TRAFFIC_BYTES_PER_ROW * rows
        alg = 2.0 * (rows * cfgd["d_model"] + cfgd["vocab"] * cfgd["d_model"] + rows * cfgd["vocab"])
        traffic_note = (f"bytes of the LM-head forward launch ({rows}x{cfgd['vocab']}x{cfgd['d_model']}), scaled by rows from "
                        f"an ncu capture at B=16; algorithmic bytes of that launch {alg:.4g}")
    line = {
        "metric": "train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": cfgd["dtype"],
        "data": "synthetic",
        "config": {"workload": DESCR[args.workload], "model": cfgd, "tokens_per_step_per_gpu": BT, "params": P,
                   "l2": "inputs larger than L2: every step streams > 10 GB of weights and activations" if P > 5e7 else
                         "small model: parameters and activations of a step may stay in L2 between steps",
                   "parallelism": f"diloco x{world} (one worker per GPU)",
                   "collective": "none inside the timed steps; outer step: cuda-ipc p2p kernel"},
        "mfu": {"per_gpu_tokens_per_s": per_gpu_tps, "flops_per_token_causal": fcausal,
                "mfu_vs_measured_burst": per_gpu_tps * fcausal / peak_burst,
                "mfu_vs_measured_sustained": per_gpu_tps * fcausal / peak_sust,
                "mfu_vs_nominal_2250": per_gpu_tps * fcausal / 2.25e15,
                "mfu_palm_convention_vs_measured_burst": per_gpu_tps * fpalm / peak_burst, "peaks": peak_src},
        "roofline": {"kernel": "k_gemm_tc (tcgen05 bf16 GEMM)", "bound": "tensor", "achieved": achieved,
                     "peak": peak_sust / 1e12, "unit": "TFLOP/s", "frac": achieved / (peak_sust / 1e12) if peak_sust else None,
                     "traffic": traffic, "traffic_note": traffic_note,
                     "launches": prof["launches"], "profiled_steps": KP,
                     "kernel_ms_share_of_step": prof["ms"] / prof_ms_total if prof_ms_total else None,
                     "how": "CUDA events around every launch of the kernel in a separate pass of the same steps, after the timed region",
                     "peak_source": f"{peak_src} sustained bf16"},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": Ke, "how": "pcpb_worker_begin_round(blob in pinned host memory) + per step: pinned host token window -> pcpb_worker_step -> "
                "loss read back; delta blob read back at the end"},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "loss_first_last": [float(losses[W]) if len(losses) > W else None, float(losses[W + K - 1]) if len(losses) >= W + K else None],
    }
    if outer:
        line["outer_step"] = outer
    if world == 1 and not args.no_other_configs and args.workload == "d20":
        # the other BASELINE training configurations, a few device-timed steps each (same method as `value`)
        others = []
        for name, st in (("d8", 8), ("gptm", 6), ("c1", 6)):
            try:
                others.append(time_workload(name, st, 3, local, peaks))
            except Exception as e:
                others.append({"workload": name, "error": str(e)})
        # the general front end (any StableHLO graph: one kernel per op of the derived tensor program, replayed as a CUDA
        # graph) on the nanoGPT-small fp32 configuration: what a graph outside the two fused families costs
        try:
            os.environ["PCPB_FRONTEND"] = "graph"
            o = time_workload("c1", 4, 3, local, peaks)
            o["workload"] = "c1_general_front_end"
            o["descr"] = DESCR["c1"] + "; run op by op by the general StableHLO front end (PCPB_FRONTEND=graph)"
            others.append(o)
        except Exception as e:
            others.append({"workload": "c1_general_front_end", "error": str(e)})
        finally:
            os.environ.pop("PCPB_FRONTEND", None)
        try:                                              # BASELINE configs[4]: rollout generation, two rollouts
            r = time_rollout(local, 2, 1, peaks)
            others.append({"workload": "qwen3_rollout", "descr": ROLLOUT_DESCR, "value": r["value"], "unit": "generated tokens/s",
                           "e2e": r["e2e"], "prefill_ms": r["prefill_ms"], "decode_ms": r["decode_ms"],
                           "decode_step_ms": r["decode_step_ms"], "gpu_launches": r["launches"], "roofline": r["roofline"]})
        except Exception as e:
            others.append({"workload": "qwen3_rollout", "error": str(e)})
        if not args.no_cpu_baseline:
            # the nanoGPT-small fp32 configuration fits the host whole: two seeded inner steps of it on the CPU oracle and on the GPU (its f32
            # GEMMs run on the tensor cores through the three-piece split, its attention on the tiled f32 kernels)
            for o in others:
                if o.get("workload") == "c1" and "error" not in o:
                    try:
                        c1 = WORKLOADS["c1"]
                        rc = cpu_oracle_run(c1, "c1", steps=2, seq=c1["seq_len"], batch=c1["batch"])
                        o["parity"] = parity_object(gpu_losses_on_sample(c1, "c1", 2, c1["seq_len"], c1["batch"], local),
                                                    rc["losses"], "f32")
                        o["cpu_oracle_tokens_per_s_same_config"] = rc["tokens_per_s"]
                    except Exception as e:
                        o["parity"] = {"error": str(e)}
        line["other_configs"] = others
    if world == 1 and not args.no_cpu_baseline:
        try:
            whole = args.workload == "c1"
            seq, batch = (cfgd["seq_len"], cfgd["batch"]) if whole else (128, 1)
            # three inner steps of the sample: 10-15 s of CPU work on the host cores of the GPU boxes of this pool
            r = cpu_oracle_run(cfgd, args.workload, steps=3, seq=seq, batch=batch)
            line["cpu_baseline"] = {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": r["threads"], "kind": "port",
                                    "sample": r["sample"], "seconds": r["seconds"], "same_config": r["same_config"]}
            # the same three seeded steps on the GPU: the oracle's per-step losses are the checker
            line["parity"] = parity_object(gpu_losses_on_sample(cfgd, args.workload, 3, seq, batch, local), r["losses"], cfgd["dtype"])
        except Exception as e:                        # the GPU numbers stand even if the host is too small for the sample
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
    print(json.dumps(line), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="d20", choices=sorted(WORKLOADS) + ["qwen3_rollout"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true")
    ap.add_argument("--rollout-layers", type=int, default=0, help="qwen3_rollout: layers (default: the configuration's 36)")
    ap.add_argument("--rollout-new", type=int, default=0, help="qwen3_rollout: new tokens per sequence (default 256)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
