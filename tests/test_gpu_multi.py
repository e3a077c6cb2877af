"""Two worker processes on two GPUs (skipped on a one-GPU box): the on-box DiLoCo outer step and streaming DiLoCo with
the fragment's outer step on the side stream, over CUDA IPC peer memory, against the oracle's loops."""
import os
import tempfile

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import SMALL_F32, flat, make_model, seeded_params, tokens_for
from oracle.loader import FifoU16
from oracle.optim import AdamConf, NesterovConf
from oracle.worker import TrainingModule, inner_loop, outer_step, streaming_loop

pytestmark = pytest.mark.gpu

P_FRAG, H, TAU, ALPHA, ROUNDS = 4, 4, 1, 0.5, 2


def _close(got, want, tol):
    diff = np.abs(got.astype(np.float64) - want.astype(np.float64))
    bad = diff > tol + tol * np.abs(want)
    return bad.sum() <= max(1, got.size // 10000) and diff.max() <= 10 * tol


def _rank(rank, world, tmp, port):
    from pcp_b200 import F32, Backend
    from pcp_b200.diloco import DilocoGroup, StreamingGroup, TorchDistTransport, streaming_max_steps
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg, text = make_model(SMALL_F32)
    mod = TrainingModule(text)
    conf = AdamConf(learning_rate=3e-4)
    master = seeded_params(cfg, seed=3, std=0.02)
    ok = True
    with Backend(rank) as be:
        be.load_session(text)
        be.set_adam(conf.learning_rate, conf.beta1, conf.beta2, conf.epsilon, conf.weight_decay, conf.max_grad_norm)
        tr = TorchDistTransport(dist)
        grp = DilocoGroup(be, tr, 0.7, 0.9, F32)
        grp.attach()

        # ---- one DiLoCo round: tau inner steps per worker, outer step over peer memory ----
        tau = 3
        toks = [tokens_for(cfg, tau, seed=70 + w) for w in range(world)]
        ref = [inner_loop(mod, master, FifoU16(toks[w]), tau, cfg.batch, cfg.seq_len, conf) for w in range(world)]
        ref_master, _, _ = outer_step(master, [torch.zeros_like(p) for p in master], [r[0] for r in ref], [r[1] for r in ref],
                                      NesterovConf(0.7, 0.9), cfg.dtype)
        be.worker_begin_round(tau, flat(master), param_dtype=F32)
        be.worker_set_tokens(toks[rank])
        for _ in range(tau):
            be.worker_step()
        delta, losses = be.worker_end_round(tau, param_dtype=F32)
        ok &= _close(delta, flat(ref[rank][0]), 1e-4)
        grp.outer_step(float(losses[-1]))
        ok &= _close(be.worker_read_state("master"), flat(ref_master), 5e-4)
        dist.barrier()                                   # no rank unmaps or frees while a peer may still read

    # ---- streaming DiLoCo, outer steps overlapped with the following training steps ----
    with Backend(rank) as be:
        be.load_session(text)
        be.set_adam(conf.learning_rate, conf.beta1, conf.beta2, conf.epsilon, conf.weight_decay, conf.max_grad_norm)
        tr = TorchDistTransport(dist)
        DilocoGroup(be, tr, 0.7, 0.9, F32).attach()
        steps = streaming_max_steps(P_FRAG, H, TAU, ROUNDS)
        toks = [tokens_for(cfg, steps, seed=50 + w) for w in range(world)]
        ref_params, ref_m, _, ref_losses = streaming_loop(mod, master, [FifoU16(t) for t in toks], P_FRAG, H, TAU, ALPHA, ROUNDS,
                                                          cfg.batch, cfg.seq_len, conf, NesterovConf(0.7, 0.9))
        be.worker_begin_round(steps, flat(master), param_dtype=F32)
        be.worker_set_tokens(toks[rank])
        sg = StreamingGroup(be, tr, P_FRAG, H, TAU, ALPHA, 0.7, 0.9, ROUNDS, overlap=True)
        sg.begin()
        got_losses = []
        for _ in range(sg.max_steps):
            sg.step()
            got_losses.append(be.worker_last_loss())
        dist.barrier()
        ok &= bool(np.allclose(got_losses, ref_losses[rank], rtol=1e-4))
        ok &= _close(be.worker_read_state("params"), flat(ref_params[rank]), 1e-4)
        ok &= _close(be.worker_read_state("master"), flat(ref_m), 1e-4)
        dist.barrier()
    with open(os.path.join(tmp, f"ok{rank}"), "w") as f:
        f.write("1" if ok else "0")
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_two_gpus():
    with tempfile.TemporaryDirectory() as tmp:
        port = 32500 + (os.getpid() % 2000)
        mp.spawn(_rank, args=(2, tmp, port), nprocs=2, join=True)
        for r in range(2):
            assert open(os.path.join(tmp, f"ok{r}")).read() == "1"
