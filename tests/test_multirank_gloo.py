"""World-size-2 (and 3) CPU test of the N > 1 host protocol: two gloo ranks run the DilocoGroup sequence
(handle exchange, barrier, shard update, barrier, loss mean) with a numpy stand-in for the device backend whose
"peer memory" is a file-backed shared array; the result must equal the oracle's outer step bit for bit."""
import os
import sys
import tempfile

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle.optim import NesterovConf
from oracle.worker import outer_step
from pcp_b200.diloco import DilocoGroup, TorchDistTransport, shard_len, shard_range

P = 1000


class FakeBackend:
    """Keeps delta / master of every rank in np.memmap files so that ranks can read and write each other's."""

    def __init__(self, tmp, rank, world, master0, delta):
        self.tmp, self.rank, self.world = tmp, rank, world
        self.delta = np.memmap(os.path.join(tmp, f"delta{rank}"), np.float32, "w+", shape=(P,))
        self.master = np.memmap(os.path.join(tmp, f"master{rank}"), np.float32, "w+", shape=(P,))
        self.delta[:] = delta; self.master[:] = master0
        self.delta.flush(); self.master.flush()
        self.vel = np.zeros(shard_len(P, world), np.float32)

    def outer_export(self):
        return f"{self.rank}".encode().ljust(128, b"\0")

    def outer_attach_ipc(self, rank, world, handles):
        assert len(handles) == world * 128 and rank == self.rank
        self.peers = [int(handles[w * 128:(w + 1) * 128].rstrip(b"\0")) for w in range(world)]

    def outer_prepare(self, lr, mu, dt):
        self.delta.flush()

    def outer_apply(self, lr, mu, dt, contributors=None):
        lo, hi = shard_range(P, self.world, self.rank)
        ranks = contributors if contributors is not None else list(range(self.world))
        acc = np.zeros(hi - lo, np.float32)
        for w in ranks:
            acc = acc + np.memmap(os.path.join(self.tmp, f"delta{w}"), np.float32, "r", shape=(P,))[lo:hi]
        acc = acc / np.float32(len(ranks))
        acc[~np.isfinite(acc)] = 0
        lr, mu = np.float32(lr), np.float32(mu)
        v = mu * self.vel[:hi - lo] + acc
        self.vel[:hi - lo] = v
        new = self.master[lo:hi] - lr * (acc + mu * v)
        for w in range(self.world):
            m = np.memmap(os.path.join(self.tmp, f"master{w}"), np.float32, "r+", shape=(P,))
            m[lo:hi] = new
            m.flush()
        return 0.0


def _worker(rank, world, tmp, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)
    master0 = rng.standard_normal(P).astype(np.float32)
    deltas = [rng.standard_normal(P).astype(np.float32) * 0.01 for _ in range(world)]
    deltas[0][5] = np.nan                                        # NaN -> 0 guard of the averaged delta
    be = FakeBackend(tmp, rank, world, master0, deltas[rank])
    grp = DilocoGroup(be, TorchDistTransport(dist))
    loss, _ = grp.outer_step(float(rank + 1))
    ref_m, ref_v, ref_loss = outer_step([torch.from_numpy(master0)], [torch.zeros(P)],
                                        [[torch.from_numpy(d)] for d in deltas], [float(r + 1) for r in range(world)],
                                        NesterovConf(0.7, 0.9), "f32")
    got = np.array(np.memmap(os.path.join(tmp, f"master{rank}"), np.float32, "r", shape=(P,)))
    ok = np.array_equal(got, ref_m[0].numpy()) and abs(loss - ref_loss) < 1e-12
    lo, hi = shard_range(P, world, rank)
    ok = ok and np.array_equal(be.vel[:hi - lo], ref_v[0].numpy()[lo:hi])
    with open(os.path.join(tmp, f"ok{rank}"), "w") as f:
        f.write("1" if ok else "0")
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_outer_step_protocol_over_gloo(world):
    with tempfile.TemporaryDirectory() as tmp:
        port = 29500 + (os.getpid() % 2000) + world
        mp.spawn(_worker, args=(world, tmp, port), nprocs=world, join=True)
        for r in range(world):
            assert open(os.path.join(tmp, f"ok{r}")).read() == "1"


def test_shard_ranges_cover_exactly():
    for total in (1, 255, 256, 1000, 560_988_160):
        for world in (1, 2, 3, 4, 8):
            s = shard_len(total, world)
            assert s % 256 == 0 and s * world >= total
            at = 0
            for r in range(world):
                lo, hi = shard_range(total, world, r)
                assert lo == min(at, total) and lo <= hi <= total
                at = max(at, hi)
            assert at == total


# ---------------------------------------------------------------------------------------------------------
# a rank leaves between rounds: the velocity shards are handed over and cut again for the smaller group
# ---------------------------------------------------------------------------------------------------------
class ElasticFakeBackend(FakeBackend):
    def worker_read_state(self, which):
        if which == "master":
            return np.array(np.memmap(os.path.join(self.tmp, f"master{self.file_id}"), np.float32, "r", shape=(P,)))
        assert which == "velocity"
        return self.vel.copy()

    def worker_write_state(self, which, values):
        assert which == "velocity" and len(values) == shard_len(P, self.world)
        self.vel = np.array(values, np.float32)

    def outer_attach_ipc(self, rank, world, handles):
        # like the library: the same (rank, world) keeps the shard, another membership starts it at zero
        if (rank, world) != (self.rank, self.world) or not hasattr(self, "peers"):
            self.vel = np.zeros(shard_len(P, world), np.float32)
        self.rank, self.world = rank, world
        self.peers = [int(handles[w * 128:(w + 1) * 128].rstrip(b"\0")) for w in range(world)]

    def outer_export(self):
        return f"{self.file_id}".encode().ljust(128, b"\0")

    def outer_apply(self, lr, mu, dt, contributors=None):
        lo, hi = shard_range(P, self.world, self.rank)
        acc = np.zeros(hi - lo, np.float32)
        for fid in self.peers:
            acc = acc + np.memmap(os.path.join(self.tmp, f"delta{fid}"), np.float32, "r", shape=(P,))[lo:hi]
        acc = acc / np.float32(len(self.peers))
        acc[~np.isfinite(acc)] = 0
        lr, mu = np.float32(lr), np.float32(mu)
        v = mu * self.vel[:hi - lo] + acc
        self.vel[:hi - lo] = v
        new = self.master[lo:hi] - lr * (acc + mu * v)
        for fid in self.peers:
            m = np.memmap(os.path.join(self.tmp, f"master{fid}"), np.float32, "r+", shape=(P,))
            m[lo:hi] = new
            m.flush()
        return 0.0


def _elastic_worker(rank, world, tmp, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)
    master0 = rng.standard_normal(P).astype(np.float32)
    deltas1 = [rng.standard_normal(P).astype(np.float32) * 0.01 for _ in range(world)]
    deltas2 = [rng.standard_normal(P).astype(np.float32) * 0.01 for _ in range(world)]
    be = ElasticFakeBackend(tmp, rank, world, master0, deltas1[rank])
    be.file_id = rank
    grp = DilocoGroup(be, TorchDistTransport(dist))
    grp.outer_step(0.0)                                           # round 1: all three workers
    stay = [0, 2]
    shards = grp.hand_over()                                      # every rank of the old group, the leaver included
    sub = dist.new_group(stay)                                    # collective over all processes
    ok = True
    if rank in stay:
        be.delta[:] = deltas2[rank]; be.delta.flush()
        grp.regroup(TorchDistTransport(dist, sub), shards, P)
        grp.outer_step(0.0)                                       # round 2: two workers, momentum carried
        m1, v1, _ = outer_step([torch.from_numpy(master0)], [torch.zeros(P)], [[torch.from_numpy(d)] for d in deltas1],
                               [0.0] * world, NesterovConf(0.7, 0.9), "f32")
        m2, v2, _ = outer_step(m1, v1, [[torch.from_numpy(deltas2[r])] for r in stay], [0.0] * 2, NesterovConf(0.7, 0.9), "f32")
        got = np.array(np.memmap(os.path.join(tmp, f"master{rank}"), np.float32, "r", shape=(P,)))
        lo, hi = shard_range(P, 2, stay.index(rank))
        ok = np.array_equal(got, m2[0].numpy()) and np.array_equal(be.vel[:hi - lo], v2[0].numpy()[lo:hi])
        ok = ok and grp.master_checksum_agrees()
    with open(os.path.join(tmp, f"ok{rank}"), "w") as f:
        f.write("1" if ok else "0")
    dist.barrier()
    dist.destroy_process_group()


def test_rank_leaves_between_rounds_velocity_survives():
    """Three workers do a round, worker 1 leaves, workers 0 and 2 regroup and do another round: master and velocity
    equal the restated Shepherd's, which keeps the Nesterov velocities across membership changes
    (src/algorithms/diloco.zig:418-444, src/optimizers/nesterov.zig:70-98)."""
    with tempfile.TemporaryDirectory() as tmp:
        port = 29500 + (os.getpid() % 2000) + 7
        mp.spawn(_elastic_worker, args=(3, tmp, port), nprocs=3, join=True)
        for r in range(3):
            assert open(os.path.join(tmp, f"ok{r}")).read() == "1"


def test_reshard_velocity_round_trips_and_lost_shard():
    from pcp_b200.diloco import reshard_velocity
    full = np.arange(P, dtype=np.float32) + 1
    old = []
    for r in range(3):
        lo, hi = shard_range(P, 3, r)
        sh = np.zeros(shard_len(P, 3), np.float32); sh[:hi - lo] = full[lo:hi]
        old.append(sh)
    for new_world in (1, 2, 4):
        got = np.concatenate([reshard_velocity(old, P, new_world, r)[: shard_range(P, new_world, r)[1] - shard_range(P, new_world, r)[0]]
                              for r in range(new_world)])
        assert np.array_equal(got, full)
    old[1] = None                                                 # a rank that died without handing its shard over
    got = np.concatenate([reshard_velocity(old, P, 2, r)[: shard_range(P, 2, r)[1] - shard_range(P, 2, r)[0]] for r in range(2)])
    lo, hi = shard_range(P, 3, 1)
    want = full.copy(); want[lo:hi] = 0
    assert np.array_equal(got, want)
