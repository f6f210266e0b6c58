"""gguf_moe on the GPU against the CPU oracle: routing weights bit for bit, the expert bank forward
within 1e-3, and the expert-parallel split adding up to the whole. GPU only."""
import numpy as np
import pytest

from tests import oracle_lib as ol

pytestmark = pytest.mark.gpu
TOL = 1e-3


def rel_err(y, ref):
    y, ref = np.asarray(y, np.float64), np.asarray(ref, np.float64)
    floor = 1e-3 * np.max(np.abs(ref))
    return float(np.max(np.abs(y - ref) / np.maximum(np.abs(ref), floor)))


def cuda(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("scoring,renorm", [(0, True), (0, False), (1, True), (1, False)])
@pytest.mark.parametrize("experts,top,tokens", [(256, 8, 16), (64, 6, 3), (8, 2, 1), (5, 5, 2)])
def test_routing_bit_exact(rq_ctx, oracle, experts, top, tokens, scoring, renorm):
    scores = oracle.normal(31, experts + tokens, experts * tokens, 1.0).reshape(experts, tokens)
    scores[1, 0] = scores[0, 0]  # a tie: the lower index wins
    want = oracle.topk(scores, top, scoring, renorm)
    got = rq_ctx.moe_route(cuda(scores), top, scoring, renorm).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.all((got != 0).sum(axis=0) == top)


@pytest.mark.parametrize("experts,top", [(256, 8), (512, 6), (96, 8), (1024, 8)])
def test_routing_with_many_equal_scores(rq_ctx, oracle, experts, top):
    """Scores drawn from a handful of values, zeros of both signs and infinities: the kept experts are the first of each
    run of equal keys, whichever way the kernel orders them (counting for up to 512 experts, repeated maxima beyond)."""
    rng = np.random.default_rng(experts)
    levels = np.float32([-2.0, -0.0, 0.0, 0.5, 0.5, 1.25, 3.0])
    scores = levels[rng.integers(0, levels.size, size=(experts, 6))]
    scores[:, 4] = 1.0                               # all equal: the first `top` experts
    scores[:, 5] = -np.inf
    scores[experts // 2:experts // 2 + 3, 5] = np.inf
    bias = levels[rng.integers(0, levels.size, size=experts)]
    for scoring in (0, 1):
        for renorm in (True, False):
            want = oracle.topk(scores[:, :5], top, scoring, renorm)
            got = rq_ctx.moe_route(cuda(scores[:, :5]), top, scoring, renorm).cpu().numpy()
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (scoring, renorm)
        want = oracle.topk(scores[:, :5], top, scoring, True, bias)
        got = rq_ctx.moe_route(cuda(scores[:, :5]), top, scoring, True, bias=cuda(bias)).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), ("bias", scoring)
    # infinities among the scores (sigmoid scoring keeps them finite)
    want = oracle.topk(scores[:, 5:6], top, 1, True)
    got = rq_ctx.moe_route(cuda(scores[:, 5:6]), top, 1, True).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    rq_ctx.check()


def test_routing_with_selection_bias(rq_ctx, oracle):
    scores = oracle.normal(32, 0, 64 * 4, 1.0).reshape(64, 4)
    bias = oracle.normal(32, 1, 64, 0.5)
    for scoring in (0, 1):
        want = oracle.topk(scores, 8, scoring, True, bias)
        got = rq_ctx.moe_route(cuda(scores), 8, scoring, True, bias=cuda(bias)).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def make_bank(oracle, t, experts, hidden, ffn, seed):
    gate = oracle.quantize(t, oracle.normal(seed, 1, experts * ffn * hidden, 0.05))
    up = oracle.quantize(t, oracle.normal(seed, 2, experts * ffn * hidden, 0.05))
    down = oracle.quantize(t, oracle.normal(seed, 3, experts * hidden * ffn, 0.05))
    shared = (oracle.quantize(t, oracle.normal(seed, 4, ffn * hidden, 0.05)), oracle.quantize(t, oracle.normal(seed, 5, ffn * hidden, 0.05)),
              oracle.quantize(t, oracle.normal(seed, 6, hidden * ffn, 0.05)), oracle.normal(seed, 7, hidden, 0.05))
    return gate, up, down, shared


@pytest.mark.parametrize("t,experts,top,hidden,ffn,tokens", [(ol.Q4_K, 16, 4, 512, 256, 3), (ol.Q4_K, 32, 8, 2048, 512, 2), (ol.Q6_K, 8, 2, 256, 256, 1),
                                                               (ol.Q8_0, 8, 3, 256, 512, 2)])
def test_moe_forward_parity(rq_ctx, oracle, t, experts, top, hidden, ffn, tokens):
    gate, up, down, shared = make_bank(oracle, t, experts, hidden, ffn, 41)
    x = oracle.normal(41, 8, hidden * tokens, 1.0).reshape(hidden, tokens)
    scores = oracle.normal(41, 9, experts * tokens, 1.0).reshape(experts, tokens)
    routing = oracle.topk(scores, top, 0, True)
    want = oracle.moe_forward(t, gate, up, down, experts, top, hidden, ffn, x, routing, shared=shared)
    bank = rq_ctx.moe_prepare(t, gate, up, down, experts, hidden, ffn, shared=shared)
    routing_d = rq_ctx.moe_route(cuda(scores), top)
    got = rq_ctx.moe_forward(bank, cuda(x), routing_d, top).cpu().numpy()
    rq_ctx.check()
    assert rel_err(got, want) <= TOL
    # without the shared expert
    want_r = oracle.moe_forward(t, gate, up, down, experts, top, hidden, ffn, x, routing, shared=None)
    got_r = rq_ctx.moe_forward(bank, cuda(x), routing_d, top, include_shared=False).cpu().numpy()
    assert rel_err(got_r, want_r) <= TOL
    # routing and the bank as one call: the same weights plane and the same output bits as the two calls
    for scoring, renorm in ((0, True), (1, False)):
        routing_2 = rq_ctx.moe_route(cuda(scores), top, scoring, renorm)
        two = rq_ctx.moe_forward(bank, cuda(x), routing_2, top).cpu().numpy()
        one, weights = rq_ctx.moe_route_forward(bank, cuda(scores), cuda(x), top, scoring, renorm)
        assert np.array_equal(weights.cpu().numpy().view(np.uint32), routing_2.cpu().numpy().view(np.uint32))
        assert np.array_equal(one.cpu().numpy().view(np.uint32), two.view(np.uint32))
    rq_ctx.check()


def test_moe_expert_parallel_split_adds_up(rq_ctx, oracle):
    """Experts dealt to four ranks: the ranks' outputs (shared expert on rank 0 only) sum to the block's."""
    t, experts, top, hidden, ffn, tokens = ol.Q4_K, 16, 4, 512, 256, 4
    gate, up, down, shared = make_bank(oracle, t, experts, hidden, ffn, 43)
    x = oracle.normal(43, 8, hidden * tokens, 1.0).reshape(hidden, tokens)
    routing = oracle.topk(oracle.normal(43, 9, experts * tokens, 1.0).reshape(experts, tokens), top, 0, True)
    want = oracle.moe_forward(t, gate, up, down, experts, top, hidden, ffn, x, routing, shared=shared)
    total = np.zeros_like(want, dtype=np.float64)
    ranks = 4
    for r in range(ranks):
        bank = rq_ctx.moe_prepare(t, gate, up, down, experts, hidden, ffn, expert_first=r * experts // ranks, expert_count=experts // ranks,
                                  shared=shared if r == 0 else None)
        part = rq_ctx.moe_forward(bank, cuda(x), cuda(routing), top, include_shared=(r == 0)).cpu().numpy()
        total += part
    rq_ctx.check()
    assert rel_err(total, want) <= TOL
    # a rank no token routes to returns exact zeros
    lonely = np.zeros_like(routing)
    lonely[0, :] = 1.0
    bank = rq_ctx.moe_prepare(t, gate, up, down, experts, hidden, ffn, expert_first=8, expert_count=8)
    assert not rq_ctx.moe_forward(bank, cuda(x), cuda(lonely), 1, include_shared=False).cpu().numpy().any()


def test_moe_argument_validation(rq_ctx, oracle):
    import ctypes

    lib = rq_ctx.lib
    out = ctypes.c_void_p()
    blocks = oracle.quantize(ol.Q4_K, oracle.normal(44, 0, 2 * 256 * 256, 0.05))
    p = blocks.ctypes.data
    assert lib.rq_moe_prepare(rq_ctx.handle, ol.Q4_K, p, p, p, 2, 0, 2, 250, 256, None, None, None, None, ctypes.byref(out)) == -1
    assert lib.rq_moe_prepare(rq_ctx.handle, ol.Q4_K, p, p, p, 2, 1, 2, 256, 256, None, None, None, None, ctypes.byref(out)) == -1
    assert lib.rq_moe_prepare(rq_ctx.handle, ol.Q4_K, p, p, p, 2, 0, 2, 256, 256, p, None, None, None, ctypes.byref(out)) == -1
    assert lib.rq_moe_route(rq_ctx.handle, None, 1, 1, 8, 2, 0, 1, None, 1, None, 1, 1, None) == -1
    s = cuda(np.zeros((8, 1), np.float32))
    assert lib.rq_moe_route(rq_ctx.handle, s.data_ptr(), 1, 1, 8, 9, 0, 1, None, 1, s.data_ptr(), 1, 1, None) == -1


@pytest.mark.parametrize("kind,count,scale", [("ungated", 1, 1.0), ("ungated", 2, 2.5), ("gated", 3, 0.5), ("none", 1, 1.75)])
def test_moe_routed_scale_and_shared_expert_variants(rq_ctx, oracle, kind, count, scale):
    """The rest of gguf_moe's arguments (recipe.rs:23415-23459): a routed scale other than one, an ungated shared expert,
    a shared expert that merges `count` experts (count times the expert width)."""
    t, experts, top, hidden, ffn, tokens = ol.Q4_K, 16, 4, 512, 256, 3
    gate, up, down, _ = make_bank(oracle, t, experts, hidden, ffn, 45)
    width = count * ffn
    sh = (oracle.quantize(t, oracle.normal(45, 4, width * hidden, 0.05)), oracle.quantize(t, oracle.normal(45, 5, width * hidden, 0.05)),
          oracle.quantize(t, oracle.normal(45, 6, hidden * width, 0.05)), oracle.normal(45, 7, hidden, 0.05))
    x = oracle.normal(45, 8, hidden * tokens, 1.0).reshape(hidden, tokens)
    scores = oracle.normal(45, 9, experts * tokens, 1.0).reshape(experts, tokens)
    routing = oracle.topk(scores, top, 0, True)
    shared_kind = {"none": 0, "ungated": 1, "gated": 2}[kind]
    want = oracle.moe_forward_ex(t, gate, up, down, experts, top, hidden, ffn, x, routing, routed_scale=scale, shared_kind=shared_kind, shared_count=count, shared=sh)
    bank = rq_ctx.moe_prepare(t, gate, up, down, experts, hidden, ffn)
    bank.set_routed_scale(scale)
    if shared_kind:
        bank.attach_shared(sh[0], sh[1], sh[2], count=count, gate_vector=sh[3] if shared_kind == 2 else None)
    got = rq_ctx.moe_forward(bank, cuda(x), rq_ctx.moe_route(cuda(scores), top), top).cpu().numpy()
    rq_ctx.check()
    assert rel_err(got, want) <= TOL
    # a second shared expert is refused, so is a non-finite scale, so is a count that leaves no room for the routed slots
    import ctypes

    if shared_kind:
        assert rq_ctx.lib.rq_moe_attach_shared(rq_ctx.handle, bank.handle, 0, 1, sh[0].ctypes.data, sh[1].ctypes.data, sh[2].ctypes.data, None) == -1
    assert rq_ctx.lib.rq_moe_set_routed_scale(bank.handle, ctypes.c_float(float("inf"))) == -1


def test_route_many_experts(rq_ctx, oracle):
    """4096 experts: beyond the default dynamic shared memory of a block."""
    experts, tokens, top = 4096, 2, 6
    scores = oracle.normal(46, 0, experts * tokens, 1.0).reshape(experts, tokens)
    got = rq_ctx.moe_route(cuda(scores), top).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), oracle.topk(scores, top, 0, True).view(np.uint32))
    rq_ctx.check()
