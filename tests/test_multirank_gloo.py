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
