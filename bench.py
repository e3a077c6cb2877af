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
    # BASELINE.json configs[3] per GPU: nanoGPT-medium bf16 (head dim 64, tanh-GELU MLP, learned positions, LayerNorm)
    "gptm": dict(vocab=50304, d_model=1024, n_layer=24, n_head=16, seq_len=1024, batch=16, dtype="bf16", activation="gelu"),
    # nanoGPT-medium layer geometry at a profiling size
    "gptml2b8": dict(vocab=50304, d_model=1024, n_layer=2, n_head=16, seq_len=1024, batch=8, dtype="bf16", activation="gelu"),
    # d20 layer geometry at profiling sizes (the kernels and their shapes per token are those of d20)
    "d20l1b8": dict(vocab=4096, d_model=1280, n_layer=1, n_head=10, n_kv_head=10, seq_len=2048, batch=8, dtype="bf16"),
    "d20l2b2": dict(vocab=65536, d_model=1280, n_layer=2, n_head=10, n_kv_head=10, seq_len=2048, batch=2, dtype="bf16"),
    "d20l2b4": dict(vocab=65536, d_model=1280, n_layer=2, n_head=10, n_kv_head=10, seq_len=2048, batch=4, dtype="bf16"),
}
DESCR = {
    "d20": "nanochat-d20 bf16 DiLoCo inner step, B=32/GPU, T=2048, AdamW(lr 1e-3, 0.9/0.95, wd 0.1), H=50",
    "d8": "nanochat-d8 (d=512) bf16 inner step, B=8, T=2048, AdamW lr 1e-3",
    "d8b2": "nanochat-d8 (d=512) bf16 inner step, B=2, T=2048 (profiling size)",
    "tiny": "nanochat tiny bf16 inner step (smoke size)",
    "gptm": "nanoGPT-medium bf16 DiLoCo inner step (24L, d=1024, 16 heads x 64, GELU), B=16/GPU, T=1024, V=50304",
    "gptml2b8": "two nanoGPT-medium layers + its LM head, B=8, T=1024 (attention / LayerNorm profiling size)",
    "d20l1b8": "one d20 layer (d=1280, 10 heads x 128), V=4096, B=8, T=2048 (attention profiling size)",
    "d20l2b2": "two d20 layers + the d20 LM head, B=2, T=2048 (GEMM DRAM-traffic profiling size)",
    "d20l2b4": "two d20 layers + the d20 LM head, B=4, T=2048 (GEMM DRAM-traffic profiling size)",
}
H_INNER = 50
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


def cpu_oracle_tokens_per_s(cfgd, steps=1, threads=None, seq=256, batch=1):
    """One inner step (compute_gradients + apply_optimizer) of the CPU oracle on a bounded sample of the
    workload: the same architecture with batch `batch` and T=`seq`."""
    import torch

    from oracle.loader import FifoU16, zipf_tokens
    from oracle.optim import AdamConf
    from oracle.worker import TrainingModule
    # all host cores this process may use; a launcher (torchrun) that exports OMP_NUM_THREADS=1 must not turn the
    # reference into a single-threaded run
    torch.set_num_threads(threads or len(os.sched_getaffinity(0)))
    cfg, text = make_model(dict(cfgd, batch=batch, seq_len=seq))
    mod = TrainingModule(text)
    g = torch.Generator().manual_seed(0)
    params = [(torch.randn(s, generator=g) * 0.02) for s in cfg.param_shapes()]
    m = [torch.zeros_like(p) for p in params]
    v = [torch.zeros_like(p) for p in params]
    ds = FifoU16(zipf_tokens((steps + 1) * (batch * seq + 1), cfg.vocab, 1.1, 0))
    conf = AdamConf(learning_rate=1e-3, beta1=0.9, beta2=0.95, weight_decay=0.1)
    t0 = time.perf_counter()
    for s in range(steps):
        x, y = ds.get_batch(batch, seq)
        grads, loss = mod.compute_gradients(params, torch.from_numpy(x), torch.from_numpy(y))
        params, m, v = mod.apply_optimizer(params, grads, m, v, float(s + 1), conf)
    dt = time.perf_counter() - t0
    return steps * batch * seq / dt, dt, torch.get_num_threads(), f"{cfgd['n_layer']}L d={cfgd['d_model']} V={cfgd['vocab']} " \
        f"B={batch} T={seq}, {steps} inner step(s) (compute_gradients + apply_optimizer) on the torch-CPU oracle"


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return 0
    cfgd = WORKLOADS[args.workload]
    seq, batch = (128, 1)
    # warm-up is one short call (imports, allocator); every timed step is one bounded-sample inner step
    if args.warmup > 0:
        cpu_oracle_tokens_per_s(dict(cfgd, n_layer=1), steps=1, seq=64, batch=1)
    tps, dt, threads, sample = cpu_oracle_tokens_per_s(cfgd, steps=max(1, args.steps), seq=seq, batch=batch)
    fcausal, _ = flops_per_token(dict(cfgd, seq_len=seq))
    line = {
        "impl": "reference", "metric": "train_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": max(1, args.steps), "warmup": args.warmup, "ms_per_step": 1e3 * dt / max(1, args.steps),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": DESCR[args.workload], "reference_arm": "CPU oracle (the reference's IREE llvm-cpu path "
                   "is not installable offline); bounded sample"},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def run_ours(args):
    import torch

    from pcp_b200 import BF16, Backend
    from pcp_b200.synthetic import f32_to_bf16_trunc_bits, zipf_tokens

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
    K, W = args.steps, max(args.warmup, 0)
    BT = cfg.batch * cfg.seq_len
    P = cfg.num_params()
    peaks, peak_src = load_peaks()

    be = Backend(local)
    be.load_session(text)
    be.set_adam(learning_rate=1e-3, beta1=0.9, beta2=0.95, epsilon=1e-8, weight_decay=0.1, max_grad_norm=1.0)
    # parameters: N(0, 0.02) from a seeded generator, truncated to bf16 like the Shepherd's master copy
    g = torch.Generator().manual_seed(0)
    blob32 = torch.empty(P, dtype=torch.float32)
    at = 0
    for s in cfg.param_shapes():
        n = int(np.prod(s))
        blob32[at:at + n] = torch.randn(n, generator=g) * 0.02
        at += n
    blob = f32_to_bf16_trunc_bits(blob32.numpy())
    del blob32
    n_tok = (max(K + W, H_INNER) + 2) * (BT + 1)
    tokens = zipf_tokens(n_tok, cfg.vocab, 1.1, seed=rank)
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

    # ---------------- value: tokens resident in HBM ----------------
    be.worker_begin_round(K + W, blob, param_dtype=BF16, tokens_on_device=True)
    be.worker_set_tokens(device_ptr=tok_dev.data_ptr(), n_tokens=n_tok)
    for _ in range(W):
        be.worker_step()
    be.synchronize()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    l0 = be.launch_count
    be.profile_enable(True)
    be.timer_start()
    for _ in range(K):
        be.worker_step()
    ms = be.timer_stop()
    prof = be.profile_read()
    be.profile_enable(False)
    launches = be.launch_count - l0
    clocks = sampler.stop()
    barrier()
    ms = max_over_ranks(ms)
    _, losses = be.worker_end_round(K + W, param_dtype=BF16, want_delta=False)
    tokens_total = world * K * BT
    value = tokens_total / (ms / 1e3)

    # ---------------- outer step (N > 1): reduce-scatter / Nesterov / all-gather over peer memory ----------------
    outer = None
    if world > 1:
        handles = be.outer_export()
        gathered = [None] * world
        dist.all_gather_object(gathered, handles)
        be.outer_attach_ipc(rank, world, b"".join(gathered))
        barrier()
        times = []
        for _ in range(3):
            be.outer_prepare(param_dtype=BF16)
            barrier()
            t0 = time.perf_counter()
            dev_ms = be.outer_apply(0.7, 0.9, BF16)
            barrier()
            times.append((max_over_ranks(dev_ms), max_over_ranks(1e3 * (time.perf_counter() - t0))))
        dev_ms, wall_ms = min(times)
        round_ms = H_INNER * ms / K
        outer = {"outer_sync_ms": dev_ms, "outer_sync_wall_ms": wall_ms, "pct_of_round": 100.0 * wall_ms / (round_ms + wall_ms),
                 "wire_bytes_per_gpu": 2 * (world - 1) / world * P * 4, "how": "P2P pull of f32 deltas + fused Nesterov + "
                 "P2P push of the new master, host barriers on both sides"}

    # ---------------- e2e: host buffers through the C ABI ----------------
    # one DiLoCo round as the worker sees it: blob in, H inner steps from host token windows, delta out.  The default
    # run times a full round of H_INNER steps; short runs (--steps < 8) time K steps and amortise the blobs over those.
    Ke = H_INNER if K >= 8 else max(1, K)
    if n_tok < Ke * BT + 1:
        Ke = max(1, (n_tok - 1) // BT)
    # the round's parameter blob and delta blob live in pinned host memory, like the token windows
    if torch.cuda.is_available():
        blob_t = torch.from_numpy(blob.view(np.int16)).pin_memory()
        blob = blob_t.numpy().view(np.uint16)
        delta_t = torch.empty(P, dtype=torch.int16).pin_memory()
        delta_buf = delta_t.numpy().view(np.uint16)
    else:
        delta_buf = None
    barrier()
    be.timer_start()
    be.worker_begin_round(Ke, blob, param_dtype=BF16, tokens_on_device=False)
    be.worker_set_tokens(device_ptr=tok_host.ctypes.data, n_tokens=n_tok)
    e2e_losses = []
    for _ in range(Ke):
        be.worker_step()
        e2e_losses.append(be.worker_last_loss())
    delta, _ = be.worker_end_round(Ke, param_dtype=BF16, want_delta=True, out=delta_buf)
    e2e_ms = max_over_ranks(be.timer_stop())
    e2e_value = world * Ke * BT / (e2e_ms / 1e3)
    h2d = (BT + 1) * 2 + blob.nbytes / Ke
    d2h = 4 + delta.nbytes / Ke

    if rank != 0:
        be.close()
        return 0

    fcausal, fpalm = flops_per_token(cfgd)
    per_gpu_tps = value / world
    peak_burst = peaks.get("bf16_tflops", PEAKS_FALLBACK["bf16_tflops"]) * 1e12
    peak_sust = peaks.get("bf16_tflops_sustained", PEAKS_FALLBACK["bf16_tflops_sustained"]) * 1e12
    achieved = prof["flops"] / (prof["ms"] / 1e3) / 1e12 if prof["ms"] > 0 else 0.0
    # DRAM traffic of the largest k_gemm_tc launch of the step, the LM-head forward [B*T x V x d]: ncu measured
    # 1.180 GB (B=2) and 2.398 GB (B=4) of dram read + write for it at the d20 width and vocabulary
    # (profiles/k_gemm_tc_d8b2_ncu_full.md); it grows in proportion to the rows, 0.29 MB per row.
    traffic, traffic_note = None, None
    if (cfgd["d_model"], cfgd["vocab"]) == (1280, 65536):
        rows = cfgd["batch"] * cfgd["seq_len"]
        traffic = 0.29e6 * rows
        alg = 2.0 * (rows * cfgd["d_model"] + cfgd["vocab"] * cfgd["d_model"] + rows * cfgd["vocab"])
        traffic_note = (f"bytes of the LM-head forward launch ({rows}x{cfgd['vocab']}x{cfgd['d_model']}), scaled by rows from "
                        f"ncu captures at B=2 and B=4; algorithmic bytes of that launch {alg:.4g}")
    line = {
        "metric": "train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": DESCR[args.workload], "model": cfgd, "tokens_per_step_per_gpu": BT, "params": P,
                   "l2": "inputs larger than L2: every step streams > 10 GB of weights and activations",
                   "parallelism": f"diloco x{world} (one worker per GPU)"},
        "mfu": {"per_gpu_tokens_per_s": per_gpu_tps, "flops_per_token_causal": fcausal,
                "mfu_vs_measured_burst": per_gpu_tps * fcausal / peak_burst,
                "mfu_vs_measured_sustained": per_gpu_tps * fcausal / peak_sust,
                "mfu_vs_nominal_2250": per_gpu_tps * fcausal / 2.25e15,
                "mfu_palm_convention_vs_measured_burst": per_gpu_tps * fpalm / peak_burst, "peaks": peak_src},
        "roofline": {"kernel": "k_gemm_tc (tcgen05 bf16 GEMM)", "bound": "tensor", "achieved": achieved,
                     "peak": peak_sust / 1e12, "unit": "TFLOP/s", "frac": achieved / (peak_sust / 1e12) if peak_sust else None,
                     "traffic": traffic, "traffic_note": traffic_note,
                     "launches": prof["launches"], "kernel_ms_share_of_step": prof["ms"] / ms if ms else None,
                     "peak_source": f"{peak_src} sustained bf16"},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": Ke, "how": "pcpb_worker_begin_round(blob in pinned host memory) + per step: pinned host token window -> pcpb_worker_step -> "
                "loss read back; delta blob read back at the end"},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "loss_first_last": [float(losses[W]) if len(losses) > W else None, float(losses[-1]) if len(losses) else None],
    }
    if outer:
        line["outer_step"] = outer
    if world == 1 and not args.no_cpu_baseline:
        try:
            seq, batch = (128, 1)
            # three inner steps of the sample: 10-15 s of CPU work on the host cores of the GPU boxes of this pool
            tps, dt, threads, sample = cpu_oracle_tokens_per_s(cfgd, steps=3, seq=seq, batch=batch)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample,
                                    "seconds": dt}
        except Exception as e:                        # the GPU numbers stand even if the host is too small for the sample
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
    be.close()
    print(json.dumps(line), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="d20", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
