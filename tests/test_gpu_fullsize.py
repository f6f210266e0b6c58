"""BASELINE's full sizes through properties that do not need the whole CPU answer. GPU only (-m gpu).

The decode-layer matrices (Q4_K 14336 x 4096, Q6_K 4096 x 14336) and the LM head (Q6_K 262144 x 2560) are quantised
on the device from seeded noise; their blocks come back through rq_weight_export, and the CPU oracle is run on a
sample of rows only. Beside that sample:
  * scaling x by two scales an int8 result by two, bit for bit (the codes do not change, the steps double exactly);
  * a row range uploaded on its own (a die's share of a row split) gives the bits the whole matrix gives for those rows;
  * the dequantised matrix is the oracle's on the sampled rows, bit for bit;
  * the batched product equals the matvec within the fp32 noise of either, at every token count of the batched config.
"""
import numpy as np
import pytest

from tests import oracle_lib as ol

pytestmark = pytest.mark.gpu
TOL = 1e-3

SHAPES = [(ol.Q4_K, 14336, 4096), (ol.Q6_K, 4096, 14336), (ol.Q6_K, 262144, 2560)]


def rel_err(y, ref):
    y, ref = np.asarray(y, np.float64), np.asarray(ref, np.float64)
    floor = 1e-3 * np.max(np.abs(ref))
    return float(np.max(np.abs(y - ref) / np.maximum(np.abs(ref), floor)))


def device_weight(rq_ctx, t, rows, cols, seed):
    import torch

    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    w32 = torch.randn(rows * cols, generator=gen, device="cuda") * 0.02
    blocks = rq_ctx.quantize(t, w32)
    del w32
    return rq_ctx.weight_from_device(t, blocks, rows, cols), gen


@pytest.mark.parametrize("t,rows,cols", SHAPES)
def test_full_size_matvec_properties(rq_ctx, oracle, t, rows, cols):
    import torch

    w, gen = device_weight(rq_ctx, t, rows, cols, 1000 + rows)
    x = torch.randn(cols, generator=gen, device="cuda")
    per, stride = ol.GEOMETRY[t]
    row_bytes = cols // per * stride
    host_blocks = rq_ctx.export(w)
    rng = np.random.default_rng(rows)
    sample = np.sort(rng.choice(rows, size=48, replace=False))
    sample_blocks = np.concatenate([host_blocks[r * row_bytes:(r + 1) * row_bytes] for r in sample])
    xh = x.cpu().numpy()
    for mode, omode in ((1, ol.INT8), (0, ol.FLOAT_RUN)):
        y = rq_ctx.matvec(w, x, act_mode=mode, step=32)
        ref = oracle.matvec(t, sample_blocks, len(sample), cols, xh, omode, 32)
        got = y.cpu().numpy()[sample]
        # the floor of the metric is taken over the sampled rows only: the same band as the small-shape tests
        assert rel_err(got, ref) <= TOL, mode
        if mode == 1:
            y2 = rq_ctx.matvec(w, 2.0 * x, act_mode=1, step=32)
            assert torch.equal(y2, 2.0 * y)
    # the dequantised weights of the sampled rows, bit for bit
    deq = rq_ctx.dequant(w)
    want = oracle.dequantize(t, sample_blocks).reshape(len(sample), cols)
    assert np.array_equal(deq[torch.from_numpy(sample).cuda()].cpu().numpy().view(np.uint32), want.view(np.uint32))
    del deq
    # a row range on its own: the same bits as the whole matrix's rows
    first, count = rows // 3 + 5, 777 if rows > 2000 else 77
    part = rq_ctx.weight_from_host(t, host_blocks, rows, cols, row_first=first, row_count=count)
    y = rq_ctx.matvec(w, x, act_mode=1, step=32)
    yp = rq_ctx.matvec(part, x, act_mode=1, step=32)
    assert torch.equal(yp, y[first:first + count])
    rq_ctx.check()
    part.free()
    w.free()


@pytest.mark.parametrize("t,rows,cols", SHAPES[:2])
@pytest.mark.parametrize("tokens", [16, 64, 512])
def test_full_size_batched_product_matches_matvec(rq_ctx, t, rows, cols, tokens):
    import torch

    w, gen = device_weight(rq_ctx, t, rows, cols, 2000 + rows)
    x = torch.randn(tokens, cols, generator=gen, device="cuda")
    y = rq_ctx.matmul(w, x)
    # the fp32 matvec of a few positions; both are within a few 1e-7 of the exact product
    for pos in (0, tokens // 2, tokens - 1):
        one = rq_ctx.matvec(w, x[pos], act_mode=0)
        assert rel_err(y[pos].cpu().numpy(), one.cpu().numpy()) <= TOL
    # linearity in the tokens: the product of a sum of two positions is the sum of their products (fp32 noise)
    both = rq_ctx.matmul(w, (x[0] + x[1]).unsqueeze(0).contiguous())
    assert rel_err(both[0].cpu().numpy(), (y[0] + y[1]).cpu().numpy()) <= TOL
    rq_ctx.check()
    w.free()


def test_full_size_expert_bank_split_adds_up(rq_ctx, oracle):
    """BASELINE's expert bank (256 experts, top-8, hidden 2048, ffn 512, gated shared expert) at 16 tokens: the outputs of
    eight expert-parallel shares (shared expert on share 0) add up to the whole bank's, and the token the oracle is run
    on agrees with it."""
    import torch

    t, experts, top, hidden, ffn, tokens = ol.Q4_K, 256, 8, 2048, 512, 16
    gen = torch.Generator(device="cuda")
    gen.manual_seed(77)

    def host_blocks(n_rows, n_cols):
        w32 = torch.randn(n_rows * n_cols, generator=gen, device="cuda") * 0.02
        b = rq_ctx.quantize(t, w32).cpu().numpy()
        del w32
        return b

    gate, up, down = host_blocks(experts * ffn, hidden), host_blocks(experts * ffn, hidden), host_blocks(experts * hidden, ffn)
    shared = (host_blocks(ffn, hidden), host_blocks(ffn, hidden), host_blocks(hidden, ffn), (torch.randn(hidden, generator=gen, device="cuda") * 0.02).cpu().numpy())
    scores = torch.randn(experts, tokens, generator=gen, device="cuda")
    x = torch.randn(hidden, tokens, generator=gen, device="cuda")
    routing = rq_ctx.moe_route(scores, top)
    assert np.array_equal(routing.cpu().numpy().view(np.uint32), oracle.topk(scores.cpu().numpy(), top, 0, True).view(np.uint32))
    whole = rq_ctx.moe_prepare(t, gate, up, down, experts, hidden, ffn, shared=shared)
    want = rq_ctx.moe_forward(whole, x, routing, top).double()
    whole.free()
    total = torch.zeros_like(want)
    shares = 8
    for r in range(shares):
        first, count = r * experts // shares, experts // shares
        bank = rq_ctx.moe_prepare(t, gate, up, down, experts, hidden, ffn, expert_first=first, expert_count=count, shared=shared if r == 0 else None)
        total += rq_ctx.moe_forward(bank, x, routing, top, include_shared=(r == 0)).double()  # the whole plane: a share reads its experts' rows
        bank.free()
    rq_ctx.check()
    assert rel_err(total.cpu().numpy(), want.cpu().numpy()) <= TOL
    # one token through the CPU oracle
    xo = x[:, :1].contiguous().cpu().numpy()
    ro = routing[:, :1].contiguous().cpu().numpy()
    ref = oracle.moe_forward(t, gate, up, down, experts, top, hidden, ffn, xo, ro, shared=shared)
    assert rel_err(want[:, :1].cpu().numpy(), ref) <= TOL
