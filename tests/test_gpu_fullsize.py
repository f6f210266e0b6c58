"""BASELINE's full sizes through properties that do not need the whole CPU answer. GPU only (-m gpu).

The decode-layer matrices (Q4_K 14336 x 4096, Q6_K 4096 x 14336) and the LM head (Q6_K 262144 x 2560) are quantised
on the device from seeded noise; their blocks come back through rq_weight_export, and the CPU oracle is run on a
sample of rows only. Beside that sample:
  * scaling x by two scales an int8 result by two, bit for bit (the codes do not change, the steps double exactly);
  * a row range uploaded on its own (a die's share of a row split) gives the bits the whole matrix gives for those rows;
  * the dequantised matrix is the oracle's on the sampled rows, bit for bit;
  * the batched product, the Q8_0 and Q4_0 configs, the LM head at four tokens and every token of the expert bank meet
    the oracle on sampled rows as well; `.int(8)` over a lone Q6_K / Q4_0 tensor is checked both as recipe computes it
    (Q8_0 re-encode at load) and as the direct dot over the stored blocks.
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


def sampled_rows(rq_ctx, w, t, rows, cols, count, seed):
    """`count` rows of a device weight as host GGUF blocks (through rq_weight_export), with their indices."""
    per, stride = ol.GEOMETRY[t]
    row_bytes = cols // per * stride
    host_blocks = rq_ctx.export(w)
    sample = np.sort(np.random.default_rng(seed).choice(rows, size=min(count, rows), replace=False))
    return sample, np.concatenate([host_blocks[r * row_bytes:(r + 1) * row_bytes] for r in sample]), host_blocks


@pytest.mark.parametrize("t,rows,cols", SHAPES[:2])
@pytest.mark.parametrize("tokens", [16, 64, 512])
def test_full_size_batched_product_against_oracle(rq_ctx, oracle, t, rows, cols, tokens):
    """BASELINE's batched config (Q4_K 14336 x 4096, Q6_K 4096 x 14336 at 16 / 64 / 512 tokens): every token of a sample
    of rows against the CPU oracle, fp32 activations and int8 activations (the tensor-core kernel serves both)."""
    import torch

    w, gen = device_weight(rq_ctx, t, rows, cols, 2000 + rows)
    x = torch.randn(tokens, cols, generator=gen, device="cuda")
    sample, sample_blocks, _ = sampled_rows(rq_ctx, w, t, rows, cols, 24, rows + tokens)
    xh = x.cpu().numpy()
    pick = torch.from_numpy(sample).cuda()
    y = rq_ctx.matmul(w, x)
    got = y[:, pick].cpu().numpy()
    # fp32 activations: against the exact product of the oracle's dequantised rows (bit-exact weights), and against the oracle's
    # own fp32 sums. At thousands of inputs per row two fp32 summation orders differ by about 1e-6 of the largest output, which
    # is the whole width of the band for outputs that cancel to nearly zero: the oracle comparison gets twice the band, the
    # comparison with the exact product the band itself.
    exact = xh.astype(np.float64) @ oracle.dequantize(t, sample_blocks).astype(np.float64).reshape(len(sample), cols).T
    assert rel_err(got, exact) <= TOL
    ref = oracle.matvec(t, sample_blocks, len(sample), cols, xh, ol.FLOAT_RUN)
    assert rel_err(got, ref) <= 2 * TOL
    y8 = rq_ctx.matmul(w, x, act_mode=1, step=32)
    ref8 = oracle.matvec(t, sample_blocks, len(sample), cols, xh, ol.INT8, 32)
    assert rel_err(y8[:, pick].cpu().numpy(), ref8) <= TOL
    # linearity in the tokens: the product of a sum of two positions is the sum of their products (fp32 noise)
    both = rq_ctx.matmul(w, (x[0] + x[1]).unsqueeze(0).contiguous())
    assert rel_err(both[0].cpu().numpy(), (y[0] + y[1]).cpu().numpy()) <= TOL
    rq_ctx.check()
    w.free()


def test_full_size_q8_0_first_config(rq_ctx, oracle):
    """BASELINE's first config: Q8_0 4096 x 4096, batch 1, both activation modes, against the oracle on sampled rows."""
    import torch

    t, rows, cols = ol.Q8_0, 4096, 4096
    w, gen = device_weight(rq_ctx, t, rows, cols, 3000)
    x = torch.randn(cols, generator=gen, device="cuda")
    sample, sample_blocks, _ = sampled_rows(rq_ctx, w, t, rows, cols, 96, 3000)
    xh = x.cpu().numpy()
    for mode, omode, step in ((1, ol.INT8, 32), (1, ol.INT8, 256), (0, ol.FLOAT_RUN, 32)):
        y = rq_ctx.matvec(w, x, act_mode=mode, step=step).cpu().numpy()
        assert rel_err(y[sample], oracle.matvec(t, sample_blocks, len(sample), cols, xh, omode, step)) <= TOL, (mode, step)
    rq_ctx.check()
    w.free()


@pytest.mark.parametrize("rows,cols", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
def test_full_size_q4_0_layer_both_int8_readings(rq_ctx, oracle, rows, cols):
    """The Q4_0 variant of the decode layer (q/o, k/v, gate/up, down shapes). Under `.int(8)` recipe re-encodes a lone
    Q4_0 tensor to Q8_0 at load and dots that ("recipe's .int(8)"); the direct dot over the stored nibbles is this
    library's opt-in. Each is checked against the oracle doing the same thing."""
    import torch

    import recipe_dev_b200 as rq

    t = ol.Q4_0
    w, gen = device_weight(rq_ctx, t, rows, cols, 4000 + rows + cols)
    x = torch.randn(cols, generator=gen, device="cuda")
    sample, sample_blocks, _ = sampled_rows(rq_ctx, w, t, rows, cols, 48, rows + cols)
    xh = x.cpu().numpy()
    # recipe's .int(8): the Q8_0 re-encode, byte for byte on the sampled rows, then the int8 dot
    w8 = rq_ctx.int8_weight(w)
    assert w8.type == rq.Q8_0
    t8, b8 = oracle.int8_blocks(t, sample_blocks)
    got8 = rq_ctx.export(w8).reshape(rows, cols // 32 * 34)[sample].reshape(-1)
    assert np.array_equal(got8, b8)
    y = rq_ctx.matvec(w8, x, act_mode=1, step=32).cpu().numpy()
    assert rel_err(y[sample], oracle.matvec(t8, b8, len(sample), cols, xh, ol.INT8, 32)) <= TOL
    # the direct dot and the fp32 handling over the stored blocks
    for mode, omode in ((1, ol.INT8), (0, ol.FLOAT_RUN)):
        y = rq_ctx.matvec(w, x, act_mode=mode, step=32).cpu().numpy()
        assert rel_err(y[sample], oracle.matvec(t, sample_blocks, len(sample), cols, xh, omode, 32)) <= TOL, mode
    rq_ctx.check()
    w8.free()
    w.free()


@pytest.mark.parametrize("rows,cols", [(4096, 14336), (262144, 2560)])
def test_full_size_q6k_recipes_int8(rq_ctx, oracle, rows, cols):
    """`down` and the LM head are lone Q6_K tensors: recipe's `.int(8)` dots their Q8_0 re-encode."""
    import torch

    import recipe_dev_b200 as rq

    t = ol.Q6_K
    w, gen = device_weight(rq_ctx, t, rows, cols, 5000 + rows)
    x = torch.randn(cols, generator=gen, device="cuda")
    sample, sample_blocks, _ = sampled_rows(rq_ctx, w, t, rows, cols, 48, rows)
    w8 = rq_ctx.int8_weight(w)
    t8, b8 = oracle.int8_blocks(t, sample_blocks)
    y = rq_ctx.matvec(w8, x, act_mode=1, step=32).cpu().numpy()
    assert rel_err(y[sample], oracle.matvec(t8, b8, len(sample), cols, x.cpu().numpy(), ol.INT8, 32)) <= TOL
    rq_ctx.check()
    w8.free()
    w.free()


def test_full_size_lm_head_four_tokens(rq_ctx, oracle):
    """The LM head at batch 4: the four-token pass of the matvec kernel and the tensor-core route of rq_matmul, every
    token of a sample of rows against the oracle's int8 answer, steps 32 and 256."""
    import torch

    t, rows, cols = ol.Q6_K, 262144, 2560
    w, gen = device_weight(rq_ctx, t, rows, cols, 6000)
    x = torch.randn(4, cols, generator=gen, device="cuda")
    sample, sample_blocks, _ = sampled_rows(rq_ctx, w, t, rows, cols, 64, 6000)
    pick = torch.from_numpy(sample).cuda()
    xh = x.cpu().numpy()
    for step in (32, 256):
        ref = oracle.matvec(t, sample_blocks, len(sample), cols, xh, ol.INT8, step)
        y = rq_ctx.matvec(w, x, act_mode=1, step=step)
        assert rel_err(y[:, pick].cpu().numpy(), ref) <= TOL, step
        y = rq_ctx.matmul(w, x, act_mode=1, step=step)
        assert rel_err(y[:, pick].cpu().numpy(), ref) <= TOL, step
    yf = rq_ctx.matmul(w, x, act_mode=0)
    assert rel_err(yf[:, pick].cpu().numpy(), oracle.matvec(t, sample_blocks, len(sample), cols, xh, ol.FLOAT_RUN)) <= TOL
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
    # every token through the CPU oracle
    ref = oracle.moe_forward(t, gate, up, down, experts, top, hidden, ffn, x.cpu().numpy(), routing.cpu().numpy(), shared=shared)
    assert rel_err(want.cpu().numpy(), ref) <= TOL
