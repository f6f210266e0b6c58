"""Recorded sequences (rq_sequence_*): a decode layer's projections recorded once and replayed as one submission with
one copy in, one copy out and one synchronisation; the results are the direct calls' bits. GPU only (-m gpu)."""
import numpy as np
import pytest

from tests import oracle_lib as ol
from tests.test_gpu_parity import rel_err, torch_cuda

pytestmark = pytest.mark.gpu


def test_recorded_layer_matches_direct_calls(oracle):
    import torch

    import recipe_dev_b200 as rq

    ctx = rq.Context(0)
    try:
        hidden, kv, ffn = 1024, 256, 2560
        mk = lambda t, rows, cols, s: (oracle.quantize(t, oracle.normal(95, s, rows * cols, 0.02)), rows, cols, t)  # noqa: E731
        specs = {"q": mk(ol.Q4_K, hidden, hidden, 0), "k": mk(ol.Q4_K, kv, hidden, 1), "v": mk(ol.Q4_K, kv, hidden, 2), "o": mk(ol.Q4_K, hidden, hidden, 3),
                 "gate": mk(ol.Q4_K, ffn, hidden, 4), "up": mk(ol.Q4_K, ffn, hidden, 5), "down": mk(ol.Q6_K, hidden, ffn, 6)}
        w = {n: ctx.weight_from_host(t, b, r, c) for n, (b, r, c, t) in specs.items()}
        dev = "cuda"
        x = torch.empty(hidden, device=dev)
        qkv = torch.empty(hidden + 2 * kv, device=dev)
        o = torch.empty(hidden, device=dev)
        gu = torch.empty(2 * ffn, device=dev)
        y = torch.empty(hidden, device=dev)

        def layer(stream):
            ctx.matvec_multi([w["q"], w["k"], w["v"]], x, [qkv[:hidden], qkv[hidden:hidden + kv], qkv[hidden + kv:]], act_mode=rq.ACT_INT8, stream=stream)
            ctx.matvec(w["o"], qkv[:hidden], o, act_mode=rq.ACT_INT8, stream=stream)       # attention itself is not on this path: o reads q's plane
            ctx.matvec_multi([w["gate"], w["up"]], o, [gu[:ffn], gu[ffn:]], act_mode=rq.ACT_INT8, stream=stream)
            ctx.matvec(w["down"], gu[:ffn], y, act_mode=rq.ACT_INT8, stream=stream)

        # a recording cannot allocate: without a reservation a recorded call that needs a larger work area is refused
        # (before it touches the stream, so the recording itself stays valid and simply holds nothing)
        s = ctx.sequence_begin()
        with pytest.raises(rq.RqError, match="rq_reserve"):
            ctx.matvec(w["down"], gu[:ffn], y, act_mode=rq.ACT_INT8, stream=s)
        ctx.sequence_end().free()
        with pytest.raises(rq.RqError, match="not recording"):
            ctx.sequence_end()
        ctx.reserve(ffn, ffn, 1)
        xs = [oracle.normal(95, 10 + i, hidden, 1.0) for i in range(3)]
        x.copy_(torch_cuda(xs[0]))
        layer(None)  # warm-up outside the recording: module load
        torch.cuda.synchronize()
        s = ctx.sequence_begin()
        layer(s)
        seq = ctx.sequence_end()
        out = np.empty(hidden, np.float32)
        for xh in xs:
            seq.run_host(xh, x, y, out)
            x.copy_(torch_cuda(xh))
            layer(None)
            torch.cuda.synchronize()
            assert np.array_equal(out, y.cpu().numpy())
        # and the chain against the oracle, step by step
        xh = xs[-1]
        q_ref = oracle.matvec(ol.Q4_K, specs["q"][0], hidden, hidden, xh, ol.INT8, 32)
        o_ref = oracle.matvec(ol.Q4_K, specs["o"][0], hidden, hidden, q_ref, ol.INT8, 32)
        g_ref = oracle.matvec(ol.Q4_K, specs["gate"][0], ffn, hidden, o_ref, ol.INT8, 32)
        t8, b8 = ol.Q6_K, specs["down"][0]
        y_ref = oracle.matvec(t8, b8, hidden, ffn, g_ref, ol.INT8, 32)
        assert rel_err(out, y_ref) <= 1e-3
        # device-side replay on the caller's stream
        x.copy_(torch_cuda(xs[0]))
        seq.run()
        torch.cuda.synchronize()
        seq.run_host(xs[0], x, y, out)
        assert np.array_equal(out, y.cpu().numpy())
        ctx.check()
        seq.free()
    finally:
        ctx.close()
