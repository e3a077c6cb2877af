"""Host-side protocol of the on-box DiLoCo outer step (one worker per GPU, one process per worker).

Mirrors the round structure of DiLoCo.run (src/algorithms/diloco.zig:415-499) with the Shepherd's
accumulate-and-apply replaced by a reduce-scatter / Nesterov / all-gather over peer memory:

    every rank:  inner loop -> delta in its own device buffer
    barrier                                    (all deltas complete and visible)
    rank r:      shard r of  mean(delta_w) -> Nesterov -> new master, written into every rank's parameter buffer
    barrier                                    (all shards written)

Shard r covers elements [r*S, min((r+1)*S, P)) of the flat parameter vector (argument order), with
S = ceil(P / W) rounded up to a multiple of 256 — the same rule the library applies (pcpb_outer_attach_*).
The group object only needs `barrier()` and `all_gather_bytes()` from the transport, so it runs on
torch.distributed (gloo or nccl) or in a single process.
"""
from __future__ import annotations


def shard_len(total_params: int, world: int) -> int:
    s = (total_params + world - 1) // world
    return (s + 255) // 256 * 256


def shard_range(total_params: int, world: int, rank: int):
    s = shard_len(total_params, world)
    lo = min(rank * s, total_params)
    return lo, min(lo + s, total_params)


class TorchDistTransport:
    def __init__(self, dist):
        self.dist = dist
        self.rank = dist.get_rank()
        self.world = dist.get_world_size()

    def barrier(self):
        self.dist.barrier()

    def all_gather_bytes(self, payload: bytes):
        out = [None] * self.world
        self.dist.all_gather_object(out, payload)
        return out

    def all_reduce_mean(self, x: float) -> float:
        import torch
        t = torch.tensor([x], dtype=torch.float64)
        self.dist.all_reduce(t)
        return float(t[0]) / self.world


class DilocoGroup:
    """One rank's view of the worker group.  `backend` needs outer_export / outer_attach_ipc / outer_prepare /
    outer_apply (pcp_b200.Backend, or a stand-in in tests)."""

    def __init__(self, backend, transport, learning_rate=0.7, momentum=0.9, param_dtype=0):
        self.be, self.tr = backend, transport
        self.lr, self.mu, self.dt = learning_rate, momentum, param_dtype
        self.attached = False

    def attach(self):
        handles = self.tr.all_gather_bytes(self.be.outer_export())
        self.be.outer_attach_ipc(self.tr.rank, self.tr.world, b"".join(handles))
        self.tr.barrier()
        self.attached = True

    def outer_step(self, final_loss: float, contributors=None):
        """-> (mean loss over contributors' ranks, device ms of the shard kernel)."""
        if not self.attached:
            self.attach()
        self.be.outer_prepare(self.lr, self.mu, self.dt)
        self.tr.barrier()
        ms = self.be.outer_apply(self.lr, self.mu, self.dt, contributors)
        self.tr.barrier()
        return self.tr.all_reduce_mean(final_loss), ms
