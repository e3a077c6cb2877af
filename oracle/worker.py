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
