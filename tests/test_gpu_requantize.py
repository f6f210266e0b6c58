"""The load-time re-encode `.int(8)` applies to a lone Q6_K / Q4_0 tensor (finish_int_sums,
recipe.rs:22345-22369; requantize_bound :22373-22431; load kernel emit_requantize :8016-8127):
the device kernel against the oracle, byte for byte, and the int8 matvec over the re-encoded
weight against the oracle doing the same. GPU only (-m gpu)."""
import numpy as np
import pytest

from tests import oracle_lib as ol
from tests.test_gpu_parity import rel_err, torch_cuda

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("t", [ol.Q6_K, ol.Q4_0, ol.Q4_K, ol.Q8_0])
@pytest.mark.parametrize("cols", [768, 96 * 32 + 32])
def test_requantize_byte_exact(rq_ctx, oracle, t, cols):
    import recipe_dev_b200 as rq

    per, stride = ol.GEOMETRY[t]
    if cols % per:
        pytest.skip("width is not a whole number of blocks of this format")
    rows = 29
    blocks = oracle.quantize(t, oracle.normal(41, t, rows * cols, 0.02))
    w = rq_ctx.weight_from_host(t, blocks, rows, cols)
    q = rq_ctx.requantize(w, rq.Q8_0)
    assert (q.type, q.rows, q.cols) == (rq.Q8_0, rows, cols)
    got = rq_ctx.export(q)
    want = oracle.requantize_q8_0(t, blocks)
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, f"{bad.size} bytes differ, first in block {bad[0] // 34}"
    # arbitrary bytes: every code / scale pattern of the source format (finite scales)
    rng = np.random.default_rng(t + cols)
    raw = rng.integers(0, 256, size=(rows * cols // per, stride), dtype=np.uint8)
    for off in ([0, 2] if t == ol.Q4_K else [208] if t == ol.Q6_K else [0]):
        raw[:, off + 1] &= 0x3F  # |d| < 2: products stay far inside fp16's range
    w2 = rq_ctx.weight_from_host(t, raw.reshape(-1), rows, cols)
    got = rq_ctx.export(rq_ctx.requantize(w2, rq.Q8_0))
    want = oracle.requantize_q8_0(t, raw.reshape(-1))
    assert np.array_equal(got, want)


@pytest.mark.parametrize("t", [ol.Q6_K, ol.Q4_0])
@pytest.mark.parametrize("step", [32, 256])
def test_int8_over_reencoded_weight_is_recipes_int8(rq_ctx, oracle, t, step):
    """What recipe computes for `.int(8)` over a lone Q6_K / Q4_0 tensor: int8 records x the Q8_0 re-encode."""
    import recipe_dev_b200 as rq

    rows, cols = 160, 2048
    blocks = oracle.quantize(t, oracle.normal(42, t, rows * cols, 0.02))
    x = oracle.normal(42, 100 + t, cols, 1.0)
    w = rq_ctx.weight_from_host(t, blocks, rows, cols)
    assert rq_ctx.lib.rq_int8_keeps(t) == 0
    w8 = rq_ctx.int8_weight(w)
    assert w8.type == rq.Q8_0
    y = rq_ctx.matvec(w8, torch_cuda(x), act_mode=rq.ACT_INT8, step=step).cpu().numpy()
    t8, b8 = oracle.int8_blocks(t, blocks)
    ref = oracle.matvec(t8, b8, rows, cols, x, ol.INT8, step)
    assert rel_err(y, ref) <= (5e-5 if step == 32 else 2e-4)  # the integer parts are exact; fp32 summation order differs
    # the direct dot over the stored blocks is a different rounding of the weights: close, not the same path
    direct = rq_ctx.matvec(w, torch_cuda(x), act_mode=rq.ACT_INT8, step=step).cpu().numpy()
    gap = float(np.max(np.abs(direct - ref)) / np.max(np.abs(ref)))
    assert 0.0 < gap <= 2e-2, gap
    rq_ctx.check()


def test_kept_formats_are_not_reencoded(rq_ctx, oracle):
    for t in (ol.Q8_0, ol.Q4_K):
        assert rq_ctx.lib.rq_int8_keeps(t) == 1
        blocks = oracle.quantize(t, oracle.normal(43, t, 8 * 256, 0.02))
        w = rq_ctx.weight_from_host(t, blocks, 8, 256)
        assert rq_ctx.int8_weight(w) is w
        assert oracle.int8_blocks(t, blocks)[0] == t
