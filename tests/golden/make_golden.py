"""Generates tests/golden/*.npz from the reference's shipped forward graphs.

Run where the reference tree is available (PCP_REFERENCE, default: the directory `reference` next to this
repository); the fixtures are committed so that machines without the tree can check against them.

  nanochat_small.npz   models/nanochat_small.mlir (f32, V=65 d=64 L=2 H=4 T=32 B=64):
                       seeded parameters and one FIFO batch -> loss and all gradients of
                       compute_gradients, then 2 inner AdamW steps with the reference's constants
                       (src/algorithms/diloco.zig:205-211) -> delta = initial - final parameters and the two losses.
  kats.npz             nothing to generate: the closed-form KATs live in tests/test_oracle_kats.py.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.loader import FifoU16, uniform_tokens            # noqa: E402
from oracle.optim import AdamConf                            # noqa: E402
from oracle.worker import TrainingModule, inner_loop         # noqa: E402

REF = os.environ.get("PCP_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))


def main():
    text = open(os.path.join(REF, "models", "nanochat_small.mlir")).read()
    mod = TrainingModule(text)
    g = torch.Generator().manual_seed(0)
    params = [torch.randn(s, generator=g) * 0.02 for s in mod.param_shapes]
    B, T = mod.data_types[0].shape
    tokens = uniform_tokens(4 * (B * T + 1), 65, seed=1)
    ds = FifoU16(tokens)
    x, y = ds.get_batch(B, T)
    grads, loss = mod.compute_gradients(params, torch.from_numpy(x), torch.from_numpy(y))
    rec = []
    ds2 = FifoU16(tokens)
    deltas, final_loss, p2, (m2, v2, t2) = inner_loop(mod, params, ds2, tau=2, batch=B, block=T,
                                                      conf=AdamConf(learning_rate=1e-3), record=rec)
    flat = lambda ts: np.concatenate([t.reshape(-1).numpy() for t in ts]).astype(np.float32)
    np.savez_compressed(
        os.path.join(os.path.dirname(os.path.abspath(__file__)), "nanochat_small.npz"),
        params=flat(params), tokens=tokens, ids=x, targets=y, loss=np.float32(loss), grads=flat(grads),
        step_losses=np.array([r[0] for r in rec], np.float32), delta_after_2=flat(deltas))
    print("loss", float(loss), "step losses", [r[0] for r in rec])


if __name__ == "__main__":
    main()
