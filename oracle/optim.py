"""AdamW inner update and Nesterov outer update, restated.  Test infrastructure only.

adamw_update   follows src/optimizers/adam_mlir.zig:50-149 op by op, in f32.
nesterov_update follows src/optimizers/nesterov.zig:70-98.
Default constants are the ones the reference hard-codes for a DiLoCo run
(src/algorithms/diloco.zig:205-211 and :218-221).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class AdamConf:
    learning_rate: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    epsilon: float = 1e-8
    weight_decay: float = 0.01
    max_grad_norm: float = 1.0


def _f(x):
    return torch.tensor(x, dtype=torch.float64).to(torch.float32)


def adamw_update(p, g, m, v, t: float, conf: AdamConf):
    """One tensor.  p, g, m, v: f32 tensors of one shape; t: the f32 timestep (1.0 at the first step).

    Returns (p', m', v').
    """
    p = p.to(torch.float32)
    g = g.to(torch.float32)
    beta1, beta2, one = _f(conf.beta1), _f(conf.beta2), _f(1.0)
    lr, eps, decay = _f(conf.learning_rate), _f(conf.epsilon), _f(conf.weight_decay)
    max_norm = _f(conf.max_grad_norm)

    g_for_norm = torch.minimum(torch.maximum(g, _f(-1000.0)), _f(1000.0))
    sum_sq = g_for_norm * g_for_norm
    for _ in range(p.dim()):                       # one dimension at a time (adam_mlir.zig:89-94)
        sum_sq = sum_sq.sum(dim=0)
    norm = torch.sqrt(sum_sq) + eps
    clip_scale = max_norm / torch.maximum(norm, max_norm)
    gc = g * clip_scale                            # scale applied to the ORIGINAL gradient

    new_m = beta1 * m + (one - beta1) * gc
    new_v = beta2 * v + (one - beta2) * (gc * gc)

    tt = torch.tensor(t, dtype=torch.float32)
    m_corr = torch.maximum(one - torch.pow(beta1, tt), eps)
    v_corr = torch.maximum(one - torch.pow(beta2, tt), eps)
    m_hat = new_m / m_corr
    v_hat = new_v / v_corr
    ratio = m_hat / (torch.sqrt(v_hat) + eps)
    new_p = p - lr * (ratio + decay * p)
    return new_p, new_m, new_v


@dataclass
class NesterovConf:
    learning_rate: float = 0.7
    momentum: float = 0.9


def nesterov_update(master, velocity, outer_grad, conf: NesterovConf):
    """v <- mu*v + g ; theta <- theta - lr*(g + mu*v).  All f32.  Returns (theta', v')."""
    lr = _f(conf.learning_rate)
    mu = _f(conf.momentum)
    v_new = mu * velocity + outer_grad
    return master - lr * (outer_grad + mu * v_new), v_new


def bf16_truncate(x: torch.Tensor) -> torch.Tensor:
    """f32 -> bf16 by dropping the low 16 bits (src/nodes/workers/worker.zig:1384,
    src/algorithms/diloco.zig:1038), returned as f32 holding the truncated value."""
    bits = x.to(torch.float32).contiguous().view(torch.int32)
    return (bits & -65536).view(torch.float32)
