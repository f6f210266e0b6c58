"""The steps either side of a projection in a decode layer, through the C ABI against the oracle: the gated feed-forward's
silu(gate x) * (up x) as one launch, RMS norm, residual add, logit soft-cap. GPU only (-m gpu)."""
import numpy as np
import pytest

from tests import oracle_lib as ol
from tests.test_gpu_parity import rel_err, torch_cuda

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("t,rows,cols", [(ol.Q4_K, 300, 1024), (ol.Q6_K, 130, 768), (ol.Q8_0, 64, 512), (ol.Q4_0, 96, 2048), (ol.Q4_K, 1000, 4096)])
@pytest.mark.parametrize("mode,tokens", [("float", 1), ("int8", 1), ("float", 3), ("int8", 5)])
def test_gated_feed_forward_in_one_launch(rq_ctx, oracle, t, rows, cols, mode, tokens):
    import recipe_dev_b200 as rq

    gate = oracle.quantize(t, oracle.normal(101, t, rows * cols, 0.02))
    up = oracle.quantize(t, oracle.normal(101, 50 + t, rows * cols, 0.02))
    x = oracle.normal(101, 99, tokens * cols, 1.0).reshape(tokens, cols)
    wg, wu = rq_ctx.weight_from_host(t, gate, rows, cols), rq_ctx.weight_from_host(t, up, rows, cols)
    act, omode = (rq.ACT_FLOAT, ol.FLOAT_RUN) if mode == "float" else (rq.ACT_INT8, ol.INT8)
    xd = torch_cuda(x if tokens > 1 else x[0])
    y = rq_ctx.matvec_glu(wg, wu, xd, act_mode=act, step=32).cpu().numpy().reshape(tokens, rows)
    g = oracle.matvec(t, gate, rows, cols, x, omode, 32)
    u = oracle.matvec(t, up, rows, cols, x, omode, 32)
    want = oracle.glu(g, u).reshape(tokens, rows)
    assert rel_err(y, want) <= 1e-3
    # the same numbers as the two projections followed by the elementwise product, to fp32 rounding
    gd = rq_ctx.matvec(wg, xd, act_mode=act, step=32).cpu().numpy().reshape(tokens, rows)
    ud = rq_ctx.matvec(wu, xd, act_mode=act, step=32).cpu().numpy().reshape(tokens, rows)
    assert rel_err(y, oracle.glu(gd, ud).reshape(tokens, rows)) <= 1e-4
    rq_ctx.check()


def test_glu_argument_validation(rq_ctx, oracle):
    import recipe_dev_b200 as rq

    a = rq_ctx.weight_from_host(ol.Q4_K, oracle.quantize(ol.Q4_K, oracle.normal(102, 0, 8 * 256, 0.02)), 8, 256)
    b = rq_ctx.weight_from_host(ol.Q4_K, oracle.quantize(ol.Q4_K, oracle.normal(102, 1, 4 * 256, 0.02)), 4, 256)
    with pytest.raises(rq.RqError, match="one format and one shape"):
        rq_ctx.matvec_glu(a, b, torch_cuda(np.zeros(256, np.float32)))
    c = rq_ctx.weight_from_host(ol.Q8_0, oracle.quantize(ol.Q8_0, oracle.normal(102, 2, 8 * 96, 0.02)), 8, 96)
    with pytest.raises(rq.RqError, match="whole 256-value units"):
        rq_ctx.matvec_glu(c, c, torch_cuda(np.zeros(96, np.float32)))


@pytest.mark.parametrize("n,tokens", [(4096, 1), (2560, 4), (100, 3), (14336, 2)])
def test_rmsnorm_add_softcap(rq_ctx, oracle, n, tokens):
    import recipe_dev_b200 as rq

    x = oracle.normal(103, n, tokens * n, 1.7).reshape(tokens, n)
    gain = oracle.normal(103, 1, n, 0.3) + 1.0
    for g in (gain, None):
        y = rq_ctx.rmsnorm(torch_cuda(x), None if g is None else torch_cuda(g), 1e-6).cpu().numpy()
        want = oracle.rmsnorm(x, g, 1e-6)
        # the sum of squares is added by a tree here and in index order by the oracle: fp32 rounding of a sum of n positive terms
        assert np.max(np.abs(y - want)) <= 2e-6 * np.max(np.abs(want))
    # channel-major planes (the reference's layout): x[k * tokens + t]
    import torch

    xc = torch_cuda(np.ascontiguousarray(x.T))
    yc = torch.empty_like(xc)
    assert rq_ctx.lib.rq_rmsnorm(rq_ctx.handle, xc.data_ptr(), tokens, 1, n, tokens, None, 1e-6, yc.data_ptr(), tokens, 1, None) == 0
    assert np.array_equal(yc.cpu().numpy().T, rq_ctx.rmsnorm(torch_cuda(x), None, 1e-6).cpu().numpy())
    a, b = torch_cuda(x), torch_cuda(x[::-1].copy())
    assert np.array_equal(rq_ctx.add(a, b).cpu().numpy(), x + x[::-1])
    logits = oracle.normal(103, 2, tokens * n, 25.0)
    got = rq_ctx.softcap(torch_cuda(logits), 30.0).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), oracle.softcap(logits, 30.0).view(np.uint32))
    with pytest.raises(rq.RqError, match="finite and positive"):
        rq_ctx.softcap(torch_cuda(logits), 0.0)
    rq_ctx.check()
