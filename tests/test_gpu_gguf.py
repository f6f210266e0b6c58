"""GGUF file -> resident weights -> matvec / expert bank, against the oracle on the file's own bytes. GPU only (-m gpu)."""
import numpy as np
import pytest

from tests import gguf_writer as gw
from tests import oracle_lib as ol
from tests.test_gpu_parity import rel_err, torch_cuda

pytestmark = pytest.mark.gpu


def test_bind_tensors_and_row_ranges(rq_ctx, oracle, tmp_path):
    import recipe_dev_b200 as rq

    shapes = {"blk.0.attn_q.weight": (ol.Q4_K, 96, 1024), "blk.0.ffn_down.weight": (ol.Q6_K, 64, 768), "output.weight": (ol.Q8_0, 50, 256), "blk.0.attn_k.weight": (ol.Q4_0, 33, 512)}
    blocks = {name: oracle.quantize(t, oracle.normal(91, i, rows * cols, 0.02)) for i, (name, (t, rows, cols)) in enumerate(shapes.items())}
    path = tmp_path / "layer.gguf"
    gw.write_gguf(path, [("general.architecture", gw.KIND_STRING, "llama")], [(name, [cols, rows], t, blocks[name]) for name, (t, rows, cols) in shapes.items()])
    g = rq.Gguf(path)
    for name, (t, rows, cols) in shapes.items():
        x = oracle.normal(91, 50 + t, cols, 1.0)
        w = g.bind(rq_ctx, name)
        assert (w.type, w.rows, w.cols) == (t, rows, cols)
        assert np.array_equal(rq_ctx.export(w), blocks[name])
        y = rq_ctx.matvec(w, torch_cuda(x), act_mode=rq.ACT_FLOAT).cpu().numpy()
        assert rel_err(y, oracle.matvec(t, blocks[name], rows, cols, x, ol.FLOAT_RUN)) <= 1e-3
        # a row range (a die's share of a row split) straight from the file
        part = g.bind(rq_ctx, name, row_first=5, row_count=17)
        yp = rq_ctx.matvec(part, torch_cuda(x), act_mode=rq.ACT_FLOAT).cpu().numpy()
        assert np.array_equal(yp, y[5:22])
    with pytest.raises(rq.RqError, match="absent"):
        g.bind(rq_ctx, "nope")
    # an F32 tensor is not a stored format this library dots
    gw.write_gguf(path, [], [("norm.weight", [8, 1], 0, np.ones(8, np.float32))])
    g2 = rq.Gguf(path)
    with pytest.raises(rq.RqError, match="F32"):
        g2.bind(rq_ctx, "norm.weight")
    rq_ctx.check()


def test_bind_expert_bank(rq_ctx, oracle, tmp_path):
    import torch

    import recipe_dev_b200 as rq

    t, experts, top, hidden, ffn, tokens = ol.Q4_K, 12, 3, 512, 256, 2
    gate = oracle.quantize(t, oracle.normal(92, 0, experts * ffn * hidden, 0.02))
    up = oracle.quantize(t, oracle.normal(92, 1, experts * ffn * hidden, 0.02))
    down = oracle.quantize(t, oracle.normal(92, 2, experts * hidden * ffn, 0.02))
    sh = (oracle.quantize(t, oracle.normal(92, 3, ffn * hidden, 0.02)), oracle.quantize(t, oracle.normal(92, 4, ffn * hidden, 0.02)),
          oracle.quantize(t, oracle.normal(92, 5, hidden * ffn, 0.02)), oracle.normal(92, 6, hidden, 0.02))
    path = tmp_path / "moe.gguf"
    gw.write_gguf(path, [("llama.expert_count", gw.KIND_U32, experts), ("llama.expert_used_count", gw.KIND_U32, top)],
                  [("blk.0.ffn_gate_exps.weight", [hidden, ffn, experts], t, gate), ("blk.0.ffn_up_exps.weight", [hidden, ffn, experts], t, up),
                   ("blk.0.ffn_down_exps.weight", [ffn, hidden, experts], t, down), ("blk.0.ffn_gate_shexp.weight", [hidden, ffn], t, sh[0]),
                   ("blk.0.ffn_up_shexp.weight", [hidden, ffn], t, sh[1]), ("blk.0.ffn_down_shexp.weight", [ffn, hidden], t, sh[2]),
                   ("blk.0.ffn_gate_inp_shexp.weight", [hidden], 0, sh[3])])
    g = rq.Gguf(path)
    assert g.integer("llama.expert_count") == experts
    names = ("blk.0.ffn_gate_exps.weight", "blk.0.ffn_up_exps.weight", "blk.0.ffn_down_exps.weight")
    shared = ("blk.0.ffn_gate_shexp.weight", "blk.0.ffn_up_shexp.weight", "blk.0.ffn_down_shexp.weight", "blk.0.ffn_gate_inp_shexp.weight")
    scores = oracle.normal(92, 7, experts * tokens, 1.0).reshape(experts, tokens)
    x = oracle.normal(92, 8, hidden * tokens, 1.0).reshape(hidden, tokens)
    routing = rq_ctx.moe_route(torch_cuda(scores), top)
    bank = g.bind_experts(rq_ctx, *names, shared=shared)
    y = rq_ctx.moe_forward(bank, torch_cuda(x), routing, top).cpu().numpy()
    ref = oracle.moe_forward(t, gate, up, down, experts, top, hidden, ffn, x, oracle.topk(scores, top, 0, True), shared=sh)
    assert rel_err(y, ref) <= 1e-3
    # an expert range (a rank's share of an expert-parallel split) straight from the file: the shares add up
    total = torch.zeros(hidden, tokens, device="cuda", dtype=torch.float64)
    for first in range(0, experts, 4):
        part = g.bind_experts(rq_ctx, *names, expert_first=first, expert_count=4, shared=shared if first == 0 else None)
        total += rq_ctx.moe_forward(part, torch_cuda(x), routing, top, include_shared=(first == 0)).double()
        part.free()
    assert rel_err(total.cpu().numpy(), ref) <= 1e-3
    rq_ctx.check()
