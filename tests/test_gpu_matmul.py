"""The batched (tensor-core) product against the CPU oracle, through the C ABI. GPU only."""
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


@pytest.mark.parametrize("t,rows,cols,tokens", [(ol.Q4_K, 128, 256, 16), (ol.Q4_K, 200, 1024, 64), (ol.Q4_K, 384, 512, 130), (ol.Q6_K, 256, 768, 16),
                                                (ol.Q6_K, 130, 512, 200), (ol.Q8_0, 128, 192, 5), (ol.Q4_0, 140, 320, 33), (ol.Q4_K, 1, 256, 1),
                                                (ol.Q4_K, 150, 4096, 40), (ol.Q6_K, 64, 14336, 33)])
def test_matmul_float_parity(rq_ctx, oracle, t, rows, cols, tokens):
    blocks = oracle.quantize(t, oracle.normal(61, t + rows, rows * cols, 0.02))
    x = oracle.normal(61, 70 + t, tokens * cols, 1.0).reshape(tokens, cols)
    w = rq_ctx.weight_from_host(t, blocks, rows, cols)
    y = rq_ctx.matmul(w, cuda(x)).cpu().numpy()
    rq_ctx.check()
    ref = oracle.matvec(t, blocks, rows, cols, x, ol.FLOAT_RUN)
    assert rel_err(y, ref) <= TOL
    exact = x.astype(np.float64) @ oracle.dequantize(t, blocks).astype(np.float64).reshape(rows, cols).T
    # the dropped lo x lo term is 2^-22 of a product, and the long sums are added in fp32 registers with
    # round-to-nearest (the tensor core's own accumulation truncates): fp32-dot accuracy at any K
    assert rel_err(y, exact) <= 5e-4
    assert np.max(np.abs(y - exact)) <= 3e-6 * np.max(np.abs(exact))
    # the same rows the matvec kernel gives, to that noise
    one = rq_ctx.matvec(w, cuda(x[0])).cpu().numpy()
    assert rel_err(y[0], one) <= 5e-4


def test_matmul_channel_major_planes_and_int8(rq_ctx, oracle):
    import torch

    t, rows, cols, tokens = ol.Q4_K, 160, 512, 24
    blocks = oracle.quantize(t, oracle.normal(62, 0, rows * cols, 0.02))
    x = oracle.normal(62, 1, tokens * cols, 1.0).reshape(tokens, cols)
    w = rq_ctx.weight_from_host(t, blocks, rows, cols)
    y = rq_ctx.matmul(w, cuda(x)).cpu().numpy()
    # the reference's planes: x[k * len + pos], y[n * len + pos]
    xc = cuda(x.T)
    yc = torch.zeros((rows, tokens), dtype=torch.float32, device="cuda")
    rc = rq_ctx.lib.rq_matmul(rq_ctx.handle, w.handle, xc.data_ptr(), tokens, 1, tokens, yc.data_ptr(), tokens, 1, 0, 32, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert np.array_equal(yc.cpu().numpy().T, y)
    # int8 activations: the exact integer dots, same bits as the matvec entry point
    y8 = rq_ctx.matmul(w, cuda(x), act_mode=1, step=32).cpu().numpy()
    assert rel_err(y8, oracle.matvec(t, blocks, rows, cols, x, ol.INT8, 32)) <= 2e-4
    rq_ctx.check()
