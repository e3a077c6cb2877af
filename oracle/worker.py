"""Training module, worker inner loop and DiLoCo outer step, restated.  Test infrastructure only.

TrainingModule   the functions src/compiler/graph_builder.zig:56-278 emits around the forward graph
                 (compute_gradients / apply_optimizer / accumulate_gradients), evaluated eagerly.
inner_loop       src/nodes/workers/worker.zig:855-1412 (Adam state reset every round, tau steps,
                 host-side accumulation scaling, NaN heal of m/v, delta = initial - final, bf16
                 delta by truncation, reports the LAST step's loss).
outer_step       src/algorithms/diloco.zig:828-1060 (f32 sum of deltas, / collected count,
                 NaN/Inf -> 0, Nesterov per tensor, bf16 master by truncation, mean of losses).
"""
from __future__ import annotations

import math

import torch

from . import autodiff, sanitizer, stablehlo as hlo
from .optim import AdamConf, NesterovConf, adamw_update, bf16_truncate, nesterov_update


class TrainingModule:
    def __init__(self, forward_mlir: str, sanitize: bool = True, clip=(-100.0, 100.0), guards=True):
        self.dtype = sanitizer.model_dtype_of(forward_mlir)
        text = sanitizer.sanitize(forward_mlir) if sanitize else forward_mlir
        self.fn = hlo.parse_module(text, "main")
        # parameters = all @main arguments except the last two (src/mlir/model_introspection.zig:251-312)
        self.num_params = len(self.fn.args) - 2
        self.param_types = [t for _, t in self.fn.args[: self.num_params]]
        self.data_types = [t for _, t in self.fn.args[self.num_params:]]
        self.clip = clip
        self.guards = guards

    @property
    def param_shapes(self):
        return [t.shape for t in self.param_types]

    def _model_params(self, params_f32):
        return [p.to(t.torch_dtype) for p, t in zip(params_f32, self.param_types)]   # RNE convert

    def forward(self, params_f32, ids, targets):
        return hlo.evaluate(self.fn, self._model_params(params_f32) + [ids, targets])

    def compute_gradients(self, params_f32, ids, targets):
        """-> (grads_f32 list, loss).  graph_builder.zig:98-164: params converted to the model dtype,
        gradient function seeded with 1.0, gradients converted back to f32."""
        ins = self._model_params(params_f32) + [ids, targets]
        loss, env = hlo.evaluate(self.fn, ins, keep_env=True)
        seed = torch.ones((), dtype=loss.dtype)
        adj = autodiff.gradients(self.fn, env, seed, self.clip[0], self.clip[1], self.guards)
        grads = []
        for (name, t) in self.fn.args[: self.num_params]:
            g = adj[name]
            if g is None:
                g = torch.zeros(t.shape, dtype=t.torch_dtype)
            grads.append(g.to(torch.float32))
        return grads, loss

    def model_forward_pass_grad(self, params_model, ids, targets, seed: float):
        """The gradient function the AD engine emits next to the forward function (src/autodiff/engine.zig:196-330):
        parameters in the model dtype, d(loss) = seed given by the caller, gradients in the model dtype.  The seed
        passes through the guard and clamp of every edge like any other adjoint."""
        ins = [p.to(t.torch_dtype) for p, t in zip(params_model, self.param_types)] + [ids, targets]
        loss, env = hlo.evaluate(self.fn, ins, keep_env=True)
        adj = autodiff.gradients(self.fn, env, torch.tensor(seed, dtype=loss.dtype), self.clip[0], self.clip[1], self.guards)
        out = []
        for (name, t) in self.fn.args[: self.num_params]:
            g = adj[name]
            out.append(g if g is not None else torch.zeros(t.shape, dtype=t.torch_dtype))
        return out

    @staticmethod
    def apply_optimizer(params, grads, m, v, t, conf: AdamConf):
        out = [adamw_update(p, g, mi, vi, t, conf) for p, g, mi, vi in zip(params, grads, m, v)]
        return [o[0] for o in out], [o[1] for o in out], [o[2] for o in out]


def inner_loop(mod: TrainingModule, initial_params_f32, dataset, tau: int, batch: int, block: int,
               conf: AdamConf, accumulation_steps: int = 1, param_dtype: str | None = None,
               adam_state=None, record=None):
    """One START_INNER_LOOP.  Returns (delta list as f32 tensors [already truncated for bf16],
    final loss, final params f32, (m, v, t)).

    adam_state=None reproduces the reference (m = v = 0, t = 1 at the start of every round,
    worker.zig:864-866); passing the previous round's (m, v, t) gives the persistent variant the
    reference's older parity test assumed.
    """
    param_dtype = param_dtype or mod.dtype
    params = [p.clone().to(torch.float32) for p in initial_params_f32]
    if adam_state is None:
        m = [torch.zeros_like(p) for p in params]
        v = [torch.zeros_like(p) for p in params]
        t = 1.0
    else:
        m, v, t = adam_state
    final_loss = 0.0
    for _ in range(tau):
        acc = [torch.zeros_like(p) for p in params]
        avg_loss = 0.0
        for _a in range(accumulation_steps):
            x, y = dataset.get_batch(batch, block)
            grads, loss = mod.compute_gradients(params, torch.from_numpy(x), torch.from_numpy(y))
            acc = [a + g for a, g in zip(acc, grads)]            # accumulate_gradients
            avg_loss += float(loss.to(torch.float32))
        if accumulation_steps > 1:
            avg_loss /= accumulation_steps
            scale = torch.tensor(1.0 / accumulation_steps, dtype=torch.float32)
            acc = [a * scale for a in acc]
        params, m, v = mod.apply_optimizer(params, acc, m, v, t, conf)
        if record is not None:
            record.append((avg_loss, [p.clone() for p in params]))
        final_loss = avg_loss
        t += 1.0
    healed = False
    for i in range(len(m)):                                        # worker.zig:1346-1369
        if not (torch.isfinite(m[i]).all() and torch.isfinite(v[i]).all()):
            m[i].zero_(); v[i].zero_(); healed = True
    if healed:
        t = 1.0
    deltas = []
    for p0, p1 in zip(initial_params_f32, params):
        d = p0.to(torch.float32) - p1
        deltas.append(bf16_truncate(d) if param_dtype == "bf16" else d)
    return deltas, final_loss, params, (m, v, t)


def outer_step(master, velocities, worker_deltas, worker_losses, conf: NesterovConf, dtype: str):
    """master: list of f32 tensors (for bf16: values already representable in bf16).
    worker_deltas: one list of tensors per contributing worker.  Returns (master', velocities', loss)."""
    n = len(worker_deltas)
    divisor = torch.tensor(float(n), dtype=torch.float32)
    new_master, new_vel = [], []
    for i, (theta, vel) in enumerate(zip(master, velocities)):
        acc = torch.zeros_like(theta, dtype=torch.float32)
        for w in range(n):
            acc = acc + worker_deltas[w][i].to(torch.float32)
        acc = acc / divisor
        acc = torch.where(torch.isfinite(acc), acc, torch.zeros_like(acc))
        th, ve = nesterov_update(theta.to(torch.float32), vel, acc, conf)
        new_master.append(bf16_truncate(th) if dtype == "bf16" else th)
        new_vel.append(ve)
    loss = float(sum(worker_losses) / n) if n else 0.0
    return new_master, new_vel, loss


# ---------------------------------------------------------------------------------------------------------
# Streaming DiLoCo (src/nodes/workers/worker.zig:2207-2610, src/algorithms/streaming_diloco.zig:425-466)
# ---------------------------------------------------------------------------------------------------------
def fragment_phase_start(p: int, inner_steps: int, num_fragments: int) -> int:
    """First step of fragment p's cycle: floor(p * H / P) (worker.zig:2367-2373)."""
    return int(math.floor(float(p) * float(inner_steps) / float(num_fragments)))


def streaming_schedule(t: int, num_fragments: int, inner_steps: int, overlap_tau: int, max_rounds: int):
    """(receives, sends) of step t (1-based), each a list of (fragment, fragment_round) in fragment order.
    Receives happen before the step's compute, sends after it (worker.zig:2213-2239); rounds past max_rounds are
    skipped (:2219, :2235)."""
    recv, send = [], []
    for p in range(num_fragments):
        tp = fragment_phase_start(p, inner_steps, num_fragments)
        if t > tp + overlap_tau and (t - tp - overlap_tau) % inner_steps == 0:
            r = (t - tp - overlap_tau) // inner_steps - 1                 # fragmentReceiveRound, :2380-2383
            if r < max_rounds:
                recv.append((p, r))
        if t > tp and (t - tp) % inner_steps == 0:
            r = (t - tp) // inner_steps - 1                               # fragmentSendRound, :2375-2378
            if r < max_rounds:
                send.append((p, r))
    return recv, send


def streaming_loop(mod: TrainingModule, master, datasets, num_fragments: int, inner_steps: int, overlap_tau: int,
                   alpha: float, max_rounds: int, batch: int, block: int, conf: AdamConf, nconf: NesterovConf,
                   record=None):
    """W workers (one dataset each) and the Shepherd's fragment state, stepped in lock-step.

    Worker: tensor i belongs to fragment i % P (worker.zig:2417).  Every step: merge the fragments due
    (blend = alpha*current + (1-alpha)*global, snapshot <- blend, :2583-2600), one compute_gradients +
    apply_optimizer with persistent m, v and an increasing timestep (:2249-2345), then send the fragments due
    (delta = snapshot - current, snapshot <- current, :2433-2437).  Shepherd: per fragment, deltas summed in
    arrival order, divided by the worker count, Nesterov on the master tensors, the new master tensors broadcast
    (streaming_diloco.zig:425-466); no non-finite filter and no truncation on this path.  All f32.
    Returns (final params per worker, master, velocities, per-step losses per worker)."""
    W = len(datasets)
    P = num_fragments
    a = torch.tensor(alpha, dtype=torch.float32)
    one_minus_a = torch.tensor(1.0, dtype=torch.float32) - a
    master = [p.clone().to(torch.float32) for p in master]
    vel = [torch.zeros_like(p) for p in master]
    params = [[p.clone() for p in master] for _ in range(W)]
    snap = [[p.clone() for p in master] for _ in range(W)]
    m = [[torch.zeros_like(p) for p in master] for _ in range(W)]
    v = [[torch.zeros_like(p) for p in master] for _ in range(W)]
    tstep = [1.0] * W
    merged = {}                                                            # (fragment, round) -> {tensor index: tensor}
    losses = [[] for _ in range(W)]
    max_steps = max_rounds * inner_steps + fragment_phase_start(P - 1, inner_steps, P) + overlap_tau   # :2202-2203
    divisor = torch.tensor(float(W), dtype=torch.float32)
    for t in range(1, max_steps + 1):
        recv, send = streaming_schedule(t, P, inner_steps, overlap_tau, max_rounds)
        for w in range(W):
            for (p, r) in recv:
                for i, g in merged[(p, r)].items():
                    blended = a * params[w][i] + one_minus_a * g
                    params[w][i] = blended
                    snap[w][i] = blended.clone()
            x, y = datasets[w].get_batch(batch, block)
            grads, loss = mod.compute_gradients(params[w], torch.from_numpy(x), torch.from_numpy(y))
            params[w], m[w], v[w] = mod.apply_optimizer(params[w], grads, m[w], v[w], tstep[w], conf)
            tstep[w] += 1.0
            losses[w].append(float(loss.to(torch.float32)))
        for (p, r) in send:
            out = {}
            for i in range(len(master)):
                if i % P != p:
                    continue
                acc = torch.zeros_like(master[i])
                for w in range(W):
                    acc = acc + (snap[w][i] - params[w][i])
                    snap[w][i] = params[w][i].clone()
                acc = acc / divisor
                master[i], vel[i] = nesterov_update(master[i], vel[i], acc, nconf)
                out[i] = master[i].clone()
            merged[(p, r)] = out
        if record is not None:
            record.append([[q.clone() for q in params[w]] for w in range(W)])
    return params, master, vel, losses
