"""pcpb_adamw_step_noalloc: the AdamW step for callers that cannot allocate device memory (hosts that own the
whole device arena, step loops with a no-allocation rule).  Called through the C ABI on caller-owned tensors and
compared with the regular apply_optimizer entry point on the same data, twice in a row: the second call finds the
first call's contents in the shared fixed scratch and must not be affected by them.  The restated optimizer of the
oracle is the second checker, including for the scalar tail path, in-place updates and the empty tensor.

The file name keeps this test last in collection order, so a run that stops at the first failure has already run
every other test."""
import numpy as np
import pytest
import torch

from helpers import SMALL_F32
from oracle.optim import AdamConf as OracleAdamConf
from oracle.optim import adamw_update
from pcp_b200 import F32, Backend, BackendError, NanochatConfig, nanochat_forward_mlir
from pcp_b200 import backend as bk

pytestmark = pytest.mark.gpu


def _reference_update(be, shapes, p, g, m, v, t):
    ins = [be.move_to_device(a, a.shape, F32) for grp in (p, g, m, v) for a in grp]
    ins.append(be.move_to_device(np.float32(t), (), F32))
    outs = be.execute_with_device_buffers(None, "apply_optimizer", ins)
    N = len(shapes)
    res = [[be.read_to_host(outs[k * N + i], F32, shapes[i]) for i in range(N)] for k in range(3)]
    for b in ins + outs:
        b.release()
    return res


def test_noalloc_adamw_matches_apply_optimizer_twice_in_a_row():
    cfg = NanochatConfig(**SMALL_F32)
    shapes = cfg.param_shapes()
    rng = np.random.default_rng(123)
    mk = lambda scale: [(rng.standard_normal(s) * scale).astype(np.float32) for s in shapes]
    p, g, m = mk(0.1), mk(3.0), mk(0.01)
    v = [np.abs(x) for x in mk(0.01)]
    conf = bk.AdamConf(3e-4, 0.9, 0.95, 1e-8, 0.1, 1.0)
    dev = torch.device("cuda:0")
    with Backend(0) as be:
        be.load_session(nanochat_forward_mlir(cfg))
        be.set_adam(conf.learning_rate, conf.beta1, conf.beta2, conf.epsilon, conf.weight_decay, conf.max_grad_norm)
        ref = {t: _reference_update(be, shapes, p, g, m, v, t) for t in (1.0, 4.0)}
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    # first call: the largest tensor; second call: a smaller one, so that stale partial sums lie beyond its chunks
    order = [int(np.argmax([a.size for a in p])), int(np.argmin([a.size for a in p]))]
    for t in (1.0, 4.0):
        for i in order:
            tp, tg, tm, tv = (torch.from_numpy(x[i]).to(dev) for x in (p, g, m, v))
            op, om, ov = torch.empty_like(tp), torch.empty_like(tp), torch.empty_like(tp)
            bk.adamw_step_noalloc(tp.data_ptr(), tg.data_ptr(), tm.data_ptr(), tv.data_ptr(), op.data_ptr(),
                                  om.data_ptr(), ov.data_ptr(), tp.numel(), conf, t, stream)
            torch.cuda.synchronize(dev)
            np.testing.assert_allclose(op.cpu().numpy(), ref[t][0][i], rtol=2e-6, atol=1e-9)
            np.testing.assert_allclose(om.cpu().numpy(), ref[t][1][i], rtol=2e-6, atol=1e-12)
            np.testing.assert_allclose(ov.cpu().numpy(), ref[t][2][i], rtol=2e-6, atol=1e-12)
            # ... and against the restated reference optimizer directly
            rp, rm, rv = adamw_update(torch.from_numpy(p[i]), torch.from_numpy(g[i]), torch.from_numpy(m[i]),
                                      torch.from_numpy(v[i]), t, OracleAdamConf(3e-4, 0.9, 0.95, 1e-8, 0.1, 1.0))
            np.testing.assert_allclose(op.cpu().numpy(), rp.numpy(), rtol=2e-6, atol=1e-9)
            np.testing.assert_allclose(om.cpu().numpy(), rm.numpy(), rtol=2e-6, atol=1e-12)
            np.testing.assert_allclose(ov.cpu().numpy(), rv.numpy(), rtol=2e-6, atol=1e-12)


def test_noalloc_tail_misaligned_in_place_and_empty():
    """Three chunks and five elements on pointers one float off the 16-byte grid (the scalar path), out of place and
    then in place (p_out == p, m_out == m, v_out == v, which the interface allows), against the oracle; n == 0 returns
    without touching anything."""
    n = 8192 * 3 + 5
    rng = np.random.default_rng(9)
    conf = bk.AdamConf(1e-3, 0.9, 0.999, 1e-8, 0.01, 1.0)
    oconf = OracleAdamConf(1e-3, 0.9, 0.999, 1e-8, 0.01, 1.0)
    dev = torch.device("cuda:0")
    host = [(rng.standard_normal(n) * s).astype(np.float32) for s in (0.1, 2.0, 0.01, 0.01)]
    host[3] = np.abs(host[3])
    rp, rm, rv = adamw_update(*[torch.from_numpy(x) for x in host], 3.0, oconf)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def off_by_one(x):                       # a view that starts 4 bytes past a 16-byte boundary
        buf = torch.zeros(n + 8, device=dev)
        view = buf[1:n + 1]
        view.copy_(torch.from_numpy(x))
        assert view.data_ptr() % 16 == 4
        return buf, view

    bufs = [off_by_one(x) for x in host]
    tp, tg, tm, tv = [b[1] for b in bufs]
    outs = [off_by_one(np.zeros(n, np.float32)) for _ in range(3)]
    op, om, ov = [o[1] for o in outs]
    bk.adamw_step_noalloc(tp.data_ptr(), tg.data_ptr(), tm.data_ptr(), tv.data_ptr(), op.data_ptr(), om.data_ptr(),
                          ov.data_ptr(), n, conf, 3.0, stream)
    torch.cuda.synchronize(dev)
    for got, want, atol in ((op, rp, 1e-9), (om, rm, 1e-12), (ov, rv, 1e-12)):
        np.testing.assert_allclose(got.cpu().numpy(), want.numpy(), rtol=2e-6, atol=atol)
    for o in outs:                            # nothing written outside [0, n)
        assert float(o[0][0]) == 0.0 and not o[0][n + 1:].any()
    # in place
    bk.adamw_step_noalloc(tp.data_ptr(), tg.data_ptr(), tm.data_ptr(), tv.data_ptr(), tp.data_ptr(), tm.data_ptr(),
                          tv.data_ptr(), n, conf, 3.0, stream)
    torch.cuda.synchronize(dev)
    assert torch.equal(tp, op) and torch.equal(tm, om) and torch.equal(tv, ov)
    # empty tensor: success, no launch, nothing touched
    before = tp.clone()
    bk.adamw_step_noalloc(tp.data_ptr(), tg.data_ptr(), tm.data_ptr(), tv.data_ptr(), tp.data_ptr(), tm.data_ptr(),
                          tv.data_ptr(), 0, conf, 4.0, stream)
    torch.cuda.synchronize(dev)
    assert torch.equal(tp, before)


def test_noalloc_rejects_oversized_and_null():
    conf = bk.AdamConf(1e-3, 0.9, 0.999, 1e-8, 0.01, 1.0)
    x = torch.zeros(16, device="cuda:0")
    a = x.data_ptr()
    with pytest.raises(BackendError) as ei:
        bk.adamw_step_noalloc(a, a, a, a, a, a, a, bk.NOALLOC_MAX_ELEMS + 1, conf, 1.0)
    assert ei.value.code == bk.E_TOO_LARGE and "exceeds" in str(ei.value)
    with pytest.raises(BackendError) as ei:
        bk.adamw_step_noalloc(None, a, a, a, a, a, a, 16, conf, 1.0)
    assert ei.value.code == bk.E_INVALID
