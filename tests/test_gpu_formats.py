"""The other stored formats (Q4_1, Q5_0, Q5_1, Q5_K, IQ4_NL, Q8_1, Q2_K, Q3_K, Q8_K, IQ4_XS; recipe.rs:15812-15824) on the device: decode bit for
bit with the oracle, export gives back the bytes, embedding gather, the run-decoder product within 1e-3, the Q8_0
re-encode byte for byte (what `.int(8)` does to them at load, recipe.rs:22345-22369), int8 over the re-encoded
weight against the oracle doing the same, and the refusals. GPU only (-m gpu)."""
import numpy as np
import pytest

from tests import oracle_lib as ol
from tests.test_gpu_parity import TOL, rel_err, torch_cuda

pytestmark = pytest.mark.gpu

TYPES = [ol.Q4_1, ol.Q5_0, ol.Q5_1, ol.Q5_K, ol.IQ4_NL, ol.Q8_1, ol.Q2_K, ol.Q3_K, ol.Q8_K, ol.IQ4_XS]


def _weight(rq_ctx, t, rows, cols, seed, arbitrary=False):
    values, stride = ol.GEOMETRY[t]
    rng = np.random.default_rng(seed)
    if arbitrary:
        blocks = ol.arbitrary_blocks(t, rows * cols // values, rng)
    else:
        blocks = ol.random_blocks(t, rows * cols // values, rng)
    return blocks, rq_ctx.weight_from_host(t, blocks, rows, cols)


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("arbitrary", [False, True])
def test_decode_export_gather(rq_ctx, oracle, t, arbitrary):
    import torch

    rows, cols = 37, 1280
    blocks, w = _weight(rq_ctx, t, rows, cols, 500 + t, arbitrary)
    assert (w.type, w.rows, w.cols) == (t, rows, cols)
    got = rq_ctx.dequant(w).cpu().numpy().reshape(-1)
    want = oracle.dequantize(t, blocks)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(rq_ctx.export(w), blocks)
    ids = torch.tensor([36, 0, 5, 5, 17], dtype=torch.int32, device="cuda")
    rowsets = rq_ctx.gather_rows(w, ids).cpu().numpy()
    assert np.array_equal(rowsets.view(np.uint32), want.reshape(rows, cols)[[36, 0, 5, 5, 17]].view(np.uint32))
    # a row range of the tensor, as a row-split placement binds it
    part = rq_ctx.weight_from_host(t, blocks, rows, cols, row_first=9, row_count=20)
    assert np.array_equal(rq_ctx.dequant(part).cpu().numpy().reshape(-1).view(np.uint32), want.reshape(rows, cols)[9:29].reshape(-1).view(np.uint32))


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("shape", [(64, 1024, 1), (301, 2560, 3), (16, 256, 2)])
def test_float_product_against_oracle(rq_ctx, oracle, t, shape):
    import recipe_dev_b200 as rq

    rows, cols, tokens = shape
    blocks, w = _weight(rq_ctx, t, rows, cols, 600 + t)
    x = oracle.normal(43, t, tokens * cols, 1.0).reshape(tokens, cols)
    ref = oracle.matvec(t, blocks, rows, cols, x, ol.FLOAT_RUN)
    y = rq_ctx.matvec(w, torch_cuda(x), act_mode=rq.ACT_FLOAT).cpu().numpy()
    assert rel_err(y, ref) <= TOL
    y2 = rq_ctx.matmul(w, torch_cuda(x), act_mode=rq.ACT_FLOAT).cpu().numpy()
    assert np.array_equal(y, y2)  # the batched entry serves these formats through the same kernel
    if tokens == 1:
        yh = rq_ctx.matvec_host(w, x[0], act_mode=rq.ACT_FLOAT)
        assert np.array_equal(yh, y.reshape(-1))
    ys = [rq_ctx.matvec(w, torch_cuda(x)) * 0 for _ in range(2)]
    rq_ctx.matvec_multi([w, w], torch_cuda(x), ys, act_mode=rq.ACT_FLOAT)
    assert np.array_equal(ys[0].cpu().numpy(), y) and np.array_equal(ys[1].cpu().numpy(), y)


@pytest.mark.parametrize("t", TYPES)
def test_int8_is_the_q8_0_reencode(rq_ctx, oracle, t):
    import recipe_dev_b200 as rq

    rows, cols = 96, 2048
    blocks, w = _weight(rq_ctx, t, rows, cols, 700 + t)
    assert rq_ctx.lib.rq_int8_keeps(t) == 0
    w8 = rq_ctx.int8_weight(w)
    assert w8.type == rq.Q8_0
    assert np.array_equal(rq_ctx.export(w8), oracle.requantize_q8_0(t, blocks))
    x = oracle.normal(44, t, cols, 1.0)
    for step in (32, 256):
        y = rq_ctx.matvec(w8, torch_cuda(x), act_mode=rq.ACT_INT8, step=step).cpu().numpy()
        t8, b8 = oracle.int8_blocks(t, blocks)
        assert t8 == ol.Q8_0
        assert rel_err(y, oracle.matvec(t8, b8, rows, cols, x, ol.INT8, step)) <= (5e-5 if step == 32 else 2e-4)
    # the stored blocks themselves have no int8 dot: the call says what to do instead
    if t != ol.Q4_1:  # Q4_1 is `.int(4)`'s storage and has an int8 dot (test_int4_is_the_q4_1_reencode)
        with pytest.raises(rq.RqError, match="rq_weight_requantize"):
            rq_ctx.matvec(w, torch_cuda(x), act_mode=rq.ACT_INT8)
    with pytest.raises(rq.RqError):
        rq_ctx.matvec_int8_static(w, torch_cuda(x))
    with pytest.raises(rq.RqError):
        rq_ctx.matvec_glu(w, w, torch_cuda(x))
    with pytest.raises(rq.RqError):
        rq_ctx.quantize(t, torch_cuda(np.zeros(cols, np.float32)))


def test_expert_banks_refuse_them(rq_ctx):
    import recipe_dev_b200 as rq

    blocks = np.zeros(2 * 256 * 256 // 32 * 20, np.uint8)
    with pytest.raises(rq.RqError, match="expert banks"):
        rq_ctx.moe_prepare(rq.Q4_1, blocks, blocks, blocks, experts=2, hidden=256, ffn=256)


def test_bound_from_a_gguf_file(rq_ctx, oracle, tmp_path):
    import recipe_dev_b200 as rq
    from tests import gguf_writer as gw

    rng = np.random.default_rng(800)
    shapes = {f"blk.{i}.w": (t, 40, 512) for i, t in enumerate(TYPES)}
    blocks = {name: ol.random_blocks(t, rows * cols // ol.GEOMETRY[t][0], rng) for name, (t, rows, cols) in shapes.items()}
    path = tmp_path / "formats.gguf"
    gw.write_gguf(path, [], [(name, [cols, rows], t, blocks[name]) for name, (t, rows, cols) in shapes.items()])
    g = rq.Gguf(path)
    for name, (t, rows, cols) in shapes.items():
        w = g.bind(rq_ctx, name, row_first=8, row_count=24)
        want = oracle.dequantize(t, blocks[name]).reshape(rows, cols)[8:32]
        assert np.array_equal(rq_ctx.dequant(w).cpu().numpy().view(np.uint32), want.view(np.uint32))
    rq_ctx.check()


@pytest.mark.parametrize("t", [ol.Q4_K, ol.Q6_K, ol.Q8_0, ol.Q4_0, ol.Q4_1, ol.Q5_K, ol.IQ4_NL, ol.Q3_K, ol.Q8_K])
@pytest.mark.parametrize("cols", [2048, 96 * 32 + 32])
def test_int4_is_the_q4_1_reencode(rq_ctx, oracle, t, cols):
    """`.int(4)` (recipe.rs:22348): storage Q4_1 by the load kernel's encoder, byte for byte; int8 records against its codes."""
    import recipe_dev_b200 as rq

    values, _ = ol.GEOMETRY[t]
    if cols % values:
        pytest.skip("width is not a whole number of blocks of this format")
    rows = 48
    if t in (ol.Q4_K, ol.Q6_K, ol.Q8_0, ol.Q4_0):
        blocks = oracle.quantize(t, oracle.normal(45, t, rows * cols, 0.02))
        w = rq_ctx.weight_from_host(t, blocks, rows, cols)
    else:
        blocks, w = _weight(rq_ctx, t, rows, cols, 900 + t)
    assert rq_ctx.lib.rq_int4_keeps(t) == (1 if t == ol.Q4_1 else 0)
    w4 = rq_ctx.int4_weight(w)
    assert w4.type == rq.Q4_1
    t4, b4 = oracle.int4_blocks(t, blocks)
    got = rq_ctx.export(w4)
    bad = np.nonzero(got != b4)[0]
    assert bad.size == 0, f"{bad.size} bytes differ, first in block {bad[0] // 20}"
    if t != ol.Q4_1:
        # an explicit re-encode of a Q4_1 tensor is the encoder applied to its decoded values (not the identity in general)
        again = rq_ctx.export(rq_ctx.requantize(w4, rq.Q4_1))
        assert np.array_equal(again, oracle.requantize_q4_1(ol.Q4_1, b4))
    for tokens in (1, 3):
        x = oracle.normal(46, t, tokens * cols, 1.0).reshape(tokens, cols)
        for step in (32, 256):
            y = rq_ctx.matvec(w4, torch_cuda(x), act_mode=rq.ACT_INT8, step=step).cpu().numpy()
            ref = oracle.matvec(ol.Q4_1, b4, rows, cols, x, ol.INT8, step)
            # every slice value is the oracle's bits; the slices (whose minimum terms are large and cancel) are added in another order
            assert rel_err(y, ref) <= 5e-4
            assert np.array_equal(rq_ctx.matmul(w4, torch_cuda(x), act_mode=rq.ACT_INT8, step=step).cpu().numpy(), y)
    rq_ctx.check()
