"""The entry point that allocates nothing (rq_matvec_int8_static), through the C ABI.

Some hosts cannot let a library call cudaMalloc: they have already given all device memory to
their own arenas, or they run a decode loop that must not stall on an allocation's device-wide
synchronisation. For them the INT8 product keeps its activation scratch in a fixed array inside
the library. This file checks that entry point against the ordinary one on two calls in a row
(the array is shared and keeps the last call's contents), and that it refuses a column wider
than the array. It is named to be collected last, so a run that stops at the first failure has
already run every other test; it also passes alone in a fresh process.
"""
import ctypes

import numpy as np
import pytest

from tests import oracle_lib as ol

pytestmark = pytest.mark.gpu

TOL = 1e-3  # the same band the other parity tests use (max relative error, fp32 accumulate)


def rel_err(y, ref):
    y, ref = np.asarray(y, np.float64), np.asarray(ref, np.float64)
    floor = 1e-3 * np.max(np.abs(ref))
    return float(np.max(np.abs(y - ref) / np.maximum(np.abs(ref), floor)))


def cuda(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("t,rows,cols,step", [(ol.Q4_K, 70, 1024, 32), (ol.Q6_K, 33, 768, 256), (ol.Q8_0, 9, 96, 32)])
def test_static_scratch_matches_allocating_entry_point_twice(rq_ctx, oracle, t, rows, cols, step):
    blocks = oracle.quantize(t, oracle.normal(21, t, rows * cols, 0.02))
    w = rq_ctx.weight_from_host(t, blocks, rows, cols)
    # two calls in a row on different columns: the second must not see anything of the first
    for call, stream_id in enumerate((300, 301)):
        x = oracle.normal(21, stream_id + t, cols, 1.0)
        if call == 1:
            x[: cols // 2] = 0.0  # zero groups: their steps and codes must be rewritten, not inherited
        xd = cuda(x)
        got = rq_ctx.matvec_int8_static(w, xd, step=step).cpu().numpy()
        want = rq_ctx.matvec(w, xd, act_mode=1, step=step).cpu().numpy()
        assert rel_err(got, want) <= TOL, (call, rel_err(got, want))
        assert rel_err(got, oracle.matvec(t, blocks, rows, cols, x, ol.INT8, step)) <= TOL
    rq_ctx.check()


def test_static_scratch_refuses_columns_beyond_its_size(rq_ctx, oracle):
    cols = 32768 + 256
    blocks = oracle.quantize(ol.Q8_0, oracle.normal(22, 0, cols, 0.02))
    w = rq_ctx.weight_from_host(ol.Q8_0, blocks, 1, cols)
    x, y = cuda(np.zeros(cols, np.float32)), cuda(np.zeros(1, np.float32))
    rc = rq_ctx.lib.rq_matvec_int8_static(rq_ctx.handle, w.handle, x.data_ptr(), y.data_ptr(), 32, None)
    assert rc == -5 and b"32768" in rq_ctx.lib.rq_last_error()
    # the widest column it serves does work
    cols = 32768
    blocks = oracle.quantize(ol.Q8_0, oracle.normal(22, 1, 2 * cols, 0.02))
    w = rq_ctx.weight_from_host(ol.Q8_0, blocks, 2, cols)
    xh = oracle.normal(22, 2, cols, 1.0)
    got = rq_ctx.matvec_int8_static(w, cuda(xh)).cpu().numpy()
    assert rel_err(got, oracle.matvec(ol.Q8_0, blocks, 2, cols, xh, ol.INT8, 32)) <= TOL
    assert rq_ctx.lib.rq_matvec_int8_static(rq_ctx.handle, w.handle, None, y.data_ptr(), 32, None) == -1


def test_static_call_allocates_nothing_and_leaves_the_context_scratch_alone(oracle):
    """The property the entry point exists for: on a fresh context, at a width the context has never
    seen, the second static call leaves free device memory unchanged, and the context holds no int8
    records afterwards (an INT8_CACHED call of that width still fails)."""
    import torch

    import recipe_dev_b200 as rq

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    ctx = rq.Context(0)
    try:
        rows, cols = 48, 5 * 256
        blocks = oracle.quantize(ol.Q4_K, oracle.normal(23, 0, rows * cols, 0.02))
        w = ctx.weight_from_host(ol.Q4_K, blocks, rows, cols)
        xh = oracle.normal(23, 1, cols, 1.0)
        x, y = cuda(xh), cuda(np.zeros(rows, np.float32))
        ctx.matvec_int8_static(w, x, y)  # the warm-up call: symbol address, module load
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        ctx.matvec_int8_static(w, x, y)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, (free_before, free_after)
        assert rel_err(y.cpu().numpy(), oracle.matvec(ol.Q4_K, blocks, rows, cols, xh, ol.INT8, 32)) <= TOL
        # the context's scratch was never written: nothing is cached for this width
        rc = ctx.matvec_raw(w, x.data_ptr(), 1, cols, 1, y.data_ptr(), 1, rows, 2, 32)
        assert rc == -1 and b"no cached int8 records" in ctx.lib.rq_last_error()
        ctx.check()
    finally:
        ctx.close()
