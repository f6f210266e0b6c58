"""Stream ordering of the context's work areas, the bounded-wait give-up path, explicit reservation.
GPU only (-m gpu). Nothing here faults, traps or hangs a GPU: the one wait that runs out is a
millisecond-limited wait in a kernel that then returns by itself."""
import numpy as np
import pytest

from tests import oracle_lib as ol
from tests.test_gpu_parity import rel_err, torch_cuda

pytestmark = pytest.mark.gpu


def test_calls_on_two_streams_do_not_share_records(rq_ctx, oracle):
    """Two INT8 calls on different streams, back to back: the second call's records must not overwrite
    the first's while its kernel still reads them (a wrong-value race, not a fault)."""
    import torch

    import recipe_dev_b200 as rq

    rows, cols = 20000, 14336  # wide: the quantiser is a launch of its own and the records live in the scratch
    t = ol.Q4_K
    blocks = oracle.quantize(t, oracle.normal(61, t, rows * cols, 0.02))
    w = rq_ctx.weight_from_host(t, blocks, rows, cols)
    xa, xb = oracle.normal(61, 1, cols, 1.0), oracle.normal(61, 2, cols, 1.0)
    da, db = torch_cuda(xa), torch_cuda(xb)
    ref_a = rq_ctx.matvec(w, da, act_mode=rq.ACT_INT8).cpu().numpy()
    ref_b = rq_ctx.matvec(w, db, act_mode=rq.ACT_INT8).cpu().numpy()
    sa, sb = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    for _ in range(5):
        ya = rq_ctx.matvec(w, da, act_mode=rq.ACT_INT8, stream=sa)
        yb = rq_ctx.matvec(w, db, act_mode=rq.ACT_INT8, stream=sb)
        torch.cuda.synchronize()
        assert np.array_equal(ya.cpu().numpy(), ref_a) and np.array_equal(yb.cpu().numpy(), ref_b)
    # sampled rows against the oracle too
    pick = np.arange(0, rows, 997)
    sub = blocks.reshape(rows, -1)[pick].reshape(-1)
    assert rel_err(ref_a[pick], oracle.matvec(t, sub, pick.size, cols, xa, ol.INT8, 32)) <= 5e-5
    rq_ctx.check()
    del sa, sb


def test_a_wait_that_runs_out_is_reported_and_nothing_hangs(oracle):
    import torch

    import recipe_dev_b200 as rq

    ctx = rq.Context(0)
    try:
        # refused at the default two-second limit: the self-test is for millisecond limits only
        assert ctx.lib.rq_wait_selftest(ctx.handle, None) == -1
        ctx.set_wait_limit(2_000_000)  # 2 ms
        ctx.wait_selftest()
        with pytest.raises(rq.RqError) as err:
            ctx.check()
        assert err.value.status == -6 and "code 21" in str(err.value)
        ctx.check()  # the flag was cleared by the failing check
        # the context is still usable, and kernels run with the short limit without tripping it
        blocks = oracle.quantize(ol.Q4_K, oracle.normal(62, 0, 64 * 1024, 0.02))
        w = ctx.weight_from_host(ol.Q4_K, blocks, 64, 1024)
        x = oracle.normal(62, 1, 1024, 1.0)
        y = ctx.matvec(w, torch_cuda(x), act_mode=rq.ACT_INT8).cpu().numpy()
        assert rel_err(y, oracle.matvec(ol.Q4_K, blocks, 64, 1024, x, ol.INT8, 32)) <= 5e-5
        ctx.check()
        assert ctx.lib.rq_set_wait_limit(ctx.handle, 10) == -1
    finally:
        ctx.close()
    torch.cuda.synchronize()


def test_reserve_makes_later_calls_allocation_free(oracle):
    import torch

    import recipe_dev_b200 as rq

    ctx = rq.Context(0)
    try:
        rows, cols, tokens = 256, 2048, 8
        ctx.reserve(rows, cols, tokens)
        blocks = oracle.quantize(ol.Q6_K, oracle.normal(63, 0, rows * cols, 0.02))
        w = ctx.weight_from_host(ol.Q6_K, blocks, rows, cols)
        x = torch_cuda(oracle.normal(63, 1, tokens * cols, 1.0).reshape(tokens, cols))
        ctx.matvec(w, x, act_mode=rq.ACT_INT8)   # warm-up: module load
        ctx.matmul(w, x, act_mode=rq.ACT_FLOAT)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        y1 = ctx.matvec(w, x, act_mode=rq.ACT_INT8)
        y2 = ctx.matmul(w, x, act_mode=rq.ACT_FLOAT)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before - 0 or torch.cuda.mem_get_info()[0] <= free_before
        # torch allocated y1 / y2 from its own cache; the library itself took nothing new:
        ctx2_free = torch.cuda.mem_get_info()[0]
        ctx.matvec(w, x, y=y1, act_mode=rq.ACT_INT8)
        ctx.matmul(w, x, y=y2, act_mode=rq.ACT_FLOAT)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == ctx2_free
        assert ctx.lib.rq_reserve(ctx.handle, 0, cols, tokens) == -1
    finally:
        ctx.close()
