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


def reshard_velocity(old_shards, total_params: int, new_world: int, new_rank: int):
    """The velocity shard of `new_rank` in a group of `new_world` ranks, cut from the shards of the previous group.

    old_shards: one float32 array per previous rank (its shard as the backend returns it, padding included), or
    None for a rank whose state was lost (it died without handing its shard over): that slice restarts at zero, the
    rest of the momentum survives.  The reference keeps all velocities on the Shepherd, so a worker that leaves never
    costs it any (src/algorithms/diloco.zig:418-444, src/optimizers/nesterov.zig:70-98); here they are spread over
    the workers and have to be cut again when the membership changes."""
    import numpy as np
    old_world = len(old_shards)
    full = np.zeros(total_params, np.float32)
    for r, sh in enumerate(old_shards):
        lo, hi = shard_range(total_params, old_world, r)
        if sh is not None and hi > lo:
            full[lo:hi] = np.asarray(sh, np.float32)[: hi - lo]
    out = np.zeros(shard_len(total_params, new_world), np.float32)
    lo, hi = shard_range(total_params, new_world, new_rank)
    out[: hi - lo] = full[lo:hi]
    return out


class TorchDistTransport:
    """torch.distributed as the transport; `group` restricts it to a sub-group (ranks are then group ranks)."""

    def __init__(self, dist, group=None):
        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def barrier(self):
        self.dist.barrier(group=self.group)

    def all_gather_bytes(self, payload: bytes):
        out = [None] * self.world
        self.dist.all_gather_object(out, payload, group=self.group)
        return out

    def all_reduce_mean(self, x: float) -> float:
        import torch
        t = torch.tensor([x], dtype=torch.float64)
        self.dist.all_reduce(t, group=self.group)
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

    def hand_over(self):
        """What a rank publishes before the membership changes: the velocity shards of every rank of the current
        group, gathered through the transport.  Every rank of the current group calls it, the ones that are about to
        leave included (a rank leaves only between rounds, src/algorithms/diloco.zig:418-427)."""
        import numpy as np
        mine = np.ascontiguousarray(self.be.worker_read_state("velocity"), np.float32)
        return [np.frombuffer(b, np.float32) for b in self.tr.all_gather_bytes(mine.tobytes())]

    def regroup(self, new_transport, old_shards, total_params: int):
        """Continue with another membership: attach over `new_transport` (the ranks that stay, renumbered) and restore
        this rank's new velocity shard from the previous group's shards (`hand_over`; None entries = lost)."""
        self.tr = new_transport
        self.attach()
        self.be.worker_write_state("velocity", reshard_velocity(old_shards, total_params, self.tr.world, self.tr.rank))
        self.tr.barrier()

    def master_checksum_agrees(self) -> bool:
        """After an outer step every rank must hold the same master parameters: compares a checksum of each rank's
        replica over the transport."""
        import hashlib
        import numpy as np
        digest = hashlib.sha256(np.ascontiguousarray(self.be.worker_read_state("master")).tobytes()).digest()
        return len(set(self.tr.all_gather_bytes(digest))) == 1

    def outer_step(self, final_loss: float, contributors=None):
        """-> (mean loss over contributors' ranks, device ms of the shard kernel)."""
        if not self.attached:
            self.attach()
        self.be.outer_prepare(self.lr, self.mu, self.dt)
        self.tr.barrier()
        ms = self.be.outer_apply(self.lr, self.mu, self.dt, contributors)
        self.tr.barrier()
        return self.tr.all_reduce_mean(final_loss), ms


# ---------------------------------------------------------------------------------------------------------
# Streaming DiLoCo: the worker's step schedule (src/nodes/workers/worker.zig:2207-2240, 2367-2383)
# ---------------------------------------------------------------------------------------------------------
def fragment_phase_start(fragment: int, inner_steps: int, num_fragments: int) -> int:
    """floor(p * H / P): the step offset of fragment p's cycle."""
    return (fragment * inner_steps) // num_fragments


def streaming_max_steps(num_fragments: int, inner_steps: int, overlap_tau: int, max_rounds: int) -> int:
    """Steps of the loop: max_rounds * H plus the time for the last fragment's last merge (worker.zig:2202-2203)."""
    return max_rounds * inner_steps + fragment_phase_start(num_fragments - 1, inner_steps, num_fragments) + overlap_tau


def streaming_schedule(t: int, num_fragments: int, inner_steps: int, overlap_tau: int, max_rounds: int):
    """(fragments to merge before step t, fragments to send after step t), t counted from 1, each entry a
    (fragment, fragment_round) pair."""
    recv, send = [], []
    for p in range(num_fragments):
        tp = fragment_phase_start(p, inner_steps, num_fragments)
        if t > tp + overlap_tau and (t - tp - overlap_tau) % inner_steps == 0:
            r = (t - tp - overlap_tau) // inner_steps - 1
            if r < max_rounds:
                recv.append((p, r))
        if t > tp and (t - tp) % inner_steps == 0:
            r = (t - tp) // inner_steps - 1
            if r < max_rounds:
                send.append((p, r))
    return recv, send


class StreamingGroup:
    """One rank's view of a streaming-DiLoCo run.  `backend` needs worker_step / stream_begin / stream_send /
    stream_outer / stream_merge and the outer-step attachment (pcp_b200.Backend, or a stand-in in tests).

    A fragment's outer step follows its send (every rank sends, barrier, every rank updates its shard of the fragment
    and writes it into all replicas of the master); the merge into the working parameters happens overlap_tau steps
    later, as in the reference, where that time hides the network round trip.  With overlap=True (backends that have
    stream_outer_start / stream_outer_wait) the outer step runs on a side stream under those overlap_tau training
    steps and is waited for, with a barrier, just before the merge; otherwise it runs to completion after the send."""

    def __init__(self, backend, transport, num_fragments=4, inner_steps=50, overlap_tau=1, alpha=0.5,
                 learning_rate=0.7, momentum=0.9, max_rounds=1, overlap=False):
        if overlap_tau < 1:
            raise ValueError("overlap_tau must be at least 1: a fragment cannot be merged in the step it was sent")
        self.be, self.tr = backend, transport
        self.P, self.H, self.tau, self.alpha = num_fragments, inner_steps, overlap_tau, alpha
        self.lr, self.mu, self.max_rounds = learning_rate, momentum, max_rounds
        self.overlap = bool(overlap)
        self.t = 0
        self.outer_ms = 0.0

    @property
    def max_steps(self) -> int:
        return streaming_max_steps(self.P, self.H, self.tau, self.max_rounds)

    def begin(self):
        """After the backend's round has been opened (worker_begin_round with tau = max_steps)."""
        self.be.stream_begin(self.P, self.alpha, self.lr, self.mu)
        self.tr.barrier()
        self.t = 0

    def step(self):
        """Merges due, one training step, sends (+ their outer steps) due.  Returns (merged, sent) fragment lists."""
        self.t += 1
        recv, send = streaming_schedule(self.t, self.P, self.H, self.tau, self.max_rounds)
        if self.overlap and recv:
            for p, _ in recv:
                self.outer_ms += self.be.stream_outer_wait(p)
            self.tr.barrier()                              # every rank's writes into this replica have landed
        for p, _ in recv:
            self.be.stream_merge(p)
        self.be.worker_step()
        for p, _ in send:
            self.be.stream_send(p)
            self.tr.barrier()
            if self.overlap:
                self.be.stream_outer_start(p)
            else:
                self.outer_ms += self.be.stream_outer(p)
                self.tr.barrier()
        return [p for p, _ in recv], [p for p, _ in send]
