"""Streaming DiLoCo, host side (no GPU): the step schedule against the restated reference schedule, and the
StreamingGroup protocol over two gloo ranks with a numpy stand-in for the device backend (peer memory = file-backed
arrays) against the oracle's streaming loop, bit for bit."""
import os
import tempfile

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle.optim import AdamConf, NesterovConf
from oracle import worker as ow
from pcp_b200.diloco import (StreamingGroup, TorchDistTransport, fragment_phase_start, shard_len, shard_range,
                             streaming_max_steps, streaming_schedule)

SHAPES = [(7,), (3, 5), (11,), (4, 4), (6,), (2, 9), (5,)]            # 7 tensors, 77 elements
SIZES = [int(np.prod(s)) for s in SHAPES]
OFFS = np.concatenate([[0], np.cumsum(SIZES)]).astype(int)
NP = int(OFFS[-1])


def test_schedule_matches_the_restated_reference():
    for P in (1, 2, 3, 4):
        for H in (1, 3, 4, 10):
            for tau in (1, 2, 5):
                for rounds in (1, 3):
                    assert streaming_max_steps(P, H, tau, rounds) == rounds * H + ow.fragment_phase_start(P - 1, H, P) + tau
                    for p in range(P):
                        assert fragment_phase_start(p, H, P) == ow.fragment_phase_start(p, H, P)
                    for t in range(1, streaming_max_steps(P, H, tau, rounds) + 1):
                        assert streaming_schedule(t, P, H, tau, rounds) == ow.streaming_schedule(t, P, H, tau, rounds)


def test_every_sent_fragment_round_is_merged_tau_steps_later():
    P, H, tau, rounds = 4, 6, 2, 3
    sent, merged = {}, {}
    for t in range(1, streaming_max_steps(P, H, tau, rounds) + 1):
        recv, send = streaming_schedule(t, P, H, tau, rounds)
        for key in recv:
            merged[key] = t
        for key in send:
            sent[key] = t
    assert set(sent) == set(merged) == {(p, r) for p in range(P) for r in range(rounds)}
    assert all(merged[k] == sent[k] + tau for k in sent)


class QuadraticModule:
    """Stand-in for TrainingModule: loss = 0.5 * sum((theta - x)^2) with x drawn per step; plain SGD as the
    'optimizer' (the streaming logic does not care what the inner step is)."""

    @staticmethod
    def compute_gradients(params, x, y):
        target = x.to(torch.float32).reshape(-1)[0]
        grads = [p - target for p in params]
        return grads, sum(((p - target) ** 2).sum() for p in params) * 0.5

    @staticmethod
    def apply_optimizer(params, grads, m, v, t, conf):
        lr = torch.tensor(conf.learning_rate, dtype=torch.float32)
        return [p - lr * g for p, g in zip(params, grads)], m, v


class TargetStream:
    def __init__(self, seed):
        self.rng = np.random.default_rng(seed)

    def get_batch(self, batch, block):
        x = np.full((batch, block), np.float32(self.rng.standard_normal()), np.float32)
        return x, x


class FakeStreamBackend:
    """theta / snapshot private; delta and the master replica of every rank in np.memmap files."""

    def __init__(self, tmp, rank, world, master0, stream, lr_inner):
        self.tmp, self.rank, self.world = tmp, rank, world
        self.delta = np.memmap(os.path.join(tmp, f"delta{rank}"), np.float32, "w+", shape=(NP,))
        self.master = np.memmap(os.path.join(tmp, f"master{rank}"), np.float32, "w+", shape=(NP,))
        self.master[:] = master0; self.master.flush()
        self.theta = master0.copy()
        self.vel = np.zeros(shard_len(NP, world), np.float32)
        self.stream, self.lr_inner = stream, np.float32(lr_inner)

    def _ranges(self, fragment):
        return [(int(OFFS[i]), int(OFFS[i + 1])) for i in range(len(SHAPES)) if i % self.P == fragment]

    def stream_begin(self, P, alpha, lr, mu):
        self.P, self.alpha, self.lr, self.mu = P, np.float32(alpha), np.float32(lr), np.float32(mu)
        self.snap = self.theta.copy()

    def worker_step(self):
        x, _ = self.stream.get_batch(1, 1)
        self.theta = self.theta - self.lr_inner * (self.theta - x.reshape(-1)[0])

    def stream_send(self, fragment):
        for lo, hi in self._ranges(fragment):
            self.delta[lo:hi] = self.snap[lo:hi] - self.theta[lo:hi]
            self.snap[lo:hi] = self.theta[lo:hi]
        self.delta.flush()

    def stream_outer(self, fragment):
        s_lo, s_hi = shard_range(NP, self.world, self.rank)
        for t_lo, t_hi in self._ranges(fragment):
            lo, hi = max(t_lo, s_lo), min(t_hi, s_hi)
            if hi <= lo:
                continue
            acc = np.zeros(hi - lo, np.float32)
            for w in range(self.world):
                acc = acc + np.memmap(os.path.join(self.tmp, f"delta{w}"), np.float32, "r", shape=(NP,))[lo:hi]
            acc = acc / np.float32(self.world)
            v = self.mu * self.vel[lo - s_lo:hi - s_lo] + acc
            self.vel[lo - s_lo:hi - s_lo] = v
            new = np.array(self.master[lo:hi]) - self.lr * (acc + self.mu * v)
            for w in range(self.world):
                m = np.memmap(os.path.join(self.tmp, f"master{w}"), np.float32, "r+", shape=(NP,))
                m[lo:hi] = new
                m.flush()
        return 0.0

    def stream_outer_start(self, fragment):            # the stand-in has no side stream: do it now
        self.stream_outer(fragment)

    def stream_outer_wait(self, fragment):
        return 0.0

    def stream_merge(self, fragment):
        glob = np.array(np.memmap(os.path.join(self.tmp, f"master{self.rank}"), np.float32, "r", shape=(NP,)))
        for lo, hi in self._ranges(fragment):
            v = self.alpha * self.theta[lo:hi] + (np.float32(1.0) - self.alpha) * glob[lo:hi]
            self.theta[lo:hi] = v
            self.snap[lo:hi] = v


CFG = dict(P=3, H=4, tau=2, alpha=0.5, rounds=2, lr_inner=0.05)


def _oracle(world):
    rng = np.random.default_rng(0)
    master0 = rng.standard_normal(NP).astype(np.float32)
    split = lambda a: [torch.from_numpy(a[OFFS[i]:OFFS[i + 1]].copy()).reshape(SHAPES[i]) for i in range(len(SHAPES))]
    params, master, vel, _ = ow.streaming_loop(QuadraticModule(), split(master0), [TargetStream(100 + w) for w in range(world)],
                                               CFG["P"], CFG["H"], CFG["tau"], CFG["alpha"], CFG["rounds"], 1, 1,
                                               AdamConf(learning_rate=CFG["lr_inner"]), NesterovConf(0.7, 0.9))
    cat = lambda ts: np.concatenate([t.numpy().reshape(-1) for t in ts])
    return master0, [cat(p) for p in params], cat(master), cat(vel)


def _rank(rank, world, tmp, port, overlap):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    master0, ref_params, ref_master, ref_vel = _oracle(world)
    be = FakeStreamBackend(tmp, rank, world, master0, TargetStream(100 + rank), CFG["lr_inner"])
    dist.barrier()                                             # every rank's files exist
    grp = StreamingGroup(be, TorchDistTransport(dist), CFG["P"], CFG["H"], CFG["tau"], CFG["alpha"], 0.7, 0.9, CFG["rounds"],
                         overlap=overlap)
    grp.begin()
    for _ in range(grp.max_steps):
        grp.step()
    dist.barrier()
    lo, hi = shard_range(NP, world, rank)
    ok = (np.array_equal(be.theta, ref_params[rank]) and np.array_equal(np.array(be.master), ref_master)
          and np.array_equal(be.vel[:hi - lo], ref_vel[lo:hi]))
    with open(os.path.join(tmp, f"ok{rank}"), "w") as f:
        f.write("1" if ok else "0")
    dist.destroy_process_group()


@pytest.mark.parametrize("world,overlap", [(2, False), (2, True)])
def test_streaming_protocol_over_gloo(world, overlap):
    with tempfile.TemporaryDirectory() as tmp:
        port = 31500 + (os.getpid() % 2000) + world + 7 * int(overlap)
        mp.spawn(_rank, args=(world, tmp, port, overlap), nprocs=world, join=True)
        for r in range(world):
            assert open(os.path.join(tmp, f"ok{r}")).read() == "1"
