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
    if exact.size >= 64:  # the largest of a handful of outputs is no measure of the sums' size
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
    # int8 activations: the tensor-core kernel over code * step; the integer dots' answer to fp32 summation noise
    y8 = rq_ctx.matmul(w, cuda(x), act_mode=1, step=32).cpu().numpy()
    assert rel_err(y8, oracle.matvec(t, blocks, rows, cols, x, ol.INT8, 32)) <= TOL
    rq_ctx.check()


# K-quant shapes that exercise the cut of the integer-operand kernel: one to fifty-six superblocks per row (windows of
# eight for the Q4_K minimum term, whole and partial, CTAs that start in the middle of a window), rows that are no
# multiple of 128, every token tile width and ragged last tiles.
KQ_SHAPES = [(ol.Q4_K, 128, 256, 4), (ol.Q4_K, 130, 768, 17), (ol.Q4_K, 300, 2304, 20), (ol.Q4_K, 257, 2048, 33), (ol.Q4_K, 140, 4352, 65),
             (ol.Q4_K, 129, 2560, 129), (ol.Q4_K, 64, 14336, 7), (ol.Q4_K, 4100, 1024, 300), (ol.Q6_K, 128, 256, 4), (ol.Q6_K, 300, 2304, 20),
             (ol.Q6_K, 200, 2560, 130), (ol.Q6_K, 70, 14336, 16), (ol.Q6_K, 4100, 768, 260),
             # a row tile per SM: no CTAs along K, so one CTA walks several windows of eight superblocks with narrow token tiles
             (ol.Q4_K, 18944, 4608, 8), (ol.Q4_K, 18944, 4608, 24), (ol.Q4_K, 18944, 2304, 70), (ol.Q6_K, 18944, 2560, 8)]


@pytest.mark.parametrize("t,rows,cols,tokens", KQ_SHAPES)
@pytest.mark.parametrize("mode", ["float", "int8_32", "int8_256"])
def test_kquant_matmul_parity(rq_ctx, oracle, t, rows, cols, tokens, mode):
    blocks = oracle.quantize(t, oracle.normal(63, t + rows, rows * cols, 0.02))
    x = oracle.normal(63, 70 + t + tokens, tokens * cols, 1.0).reshape(tokens, cols)
    w = rq_ctx.weight_from_host(t, blocks, rows, cols)
    # the oracle on a sample of rows keeps the CPU side to seconds
    pick = np.unique(np.concatenate([np.arange(0, rows, max(1, rows // 40)), [rows - 1, min(rows - 1, 127), min(rows - 1, 128)]]))
    per, stride = ol.GEOMETRY[t]
    sub = blocks.reshape(rows, cols // per * stride)[pick].reshape(-1)
    if mode == "float":
        y = rq_ctx.matmul(w, cuda(x)).cpu().numpy()
        ref = oracle.matvec(t, sub, pick.size, cols, x, ol.FLOAT_RUN)
        exact = x.astype(np.float64) @ oracle.dequantize(t, sub).astype(np.float64).reshape(pick.size, cols).T
        assert np.max(np.abs(y[:, pick] - exact)) <= 3e-6 * np.max(np.abs(exact))
    else:
        step = int(mode.split("_")[1])
        y = rq_ctx.matmul(w, cuda(x), act_mode=1, step=step).cpu().numpy()
        ref = oracle.matvec(t, sub, pick.size, cols, x, ol.INT8, step)
    rq_ctx.check()
    assert rel_err(y[:, pick], ref) <= TOL


@pytest.mark.parametrize("t,rows,cols,tokens", [(ol.Q4_K, 130, 2304, 20), (ol.Q6_K, 200, 2560, 130), (ol.Q4_K, 256, 4096, 512), (ol.Q6_K, 256, 14336, 64)])
@pytest.mark.parametrize("step", [32, 256])
def test_kquant_matmul_int8_equals_float_over_the_records(rq_ctx, oracle, t, rows, cols, tokens, step):
    """The batched INT8 call quantises while it prepares its operands; the result must equal, bit for bit, the batched
    FLOAT call over code * d of the standalone quantiser's records (themselves bit-exact with the oracle's), ties, zero
    groups and strided inputs included."""
    import torch

    x = oracle.normal(65, t + tokens + step, tokens * cols, 1.0).reshape(tokens, cols)
    x[0, :256] = 0.0                      # a group of zeros: inverse and d are zero
    x[1, 5], x[1, 9] = -3.5, 3.5          # equal magnitudes: the first one is the extreme
    x[2, 40], x[2, 300 % cols] = 7.0, -7.0
    x[3 % tokens, 64:96] = np.float32(1e-30)
    w = rq_ctx.weight_from_host(t, oracle.quantize(t, oracle.normal(65, t + rows, rows * cols, 0.02)), rows, cols)
    xd = cuda(x)
    rec = rq_ctx.activation_records(xd, step).cpu().numpy()
    d = rec[:, :, :4].copy().view(np.float32)
    back = (rec[:, :, 4:].view(np.int8).astype(np.float32) * d).reshape(tokens, cols)
    for i in range(min(tokens, 4)):
        assert np.array_equal(rec[i], oracle.activation_records(x[i], step))
    y8 = rq_ctx.matmul(w, xd, act_mode=1, step=step)
    yf = rq_ctx.matmul(w, cuda(back))
    rq_ctx.check()
    assert torch.equal(y8, yf)
    # a padded, strided view of the same inputs takes the scalar loads
    wide = torch.zeros((tokens, cols + 3), dtype=torch.float32, device="cuda")
    wide[:, 1:cols + 1] = xd
    assert torch.equal(rq_ctx.matmul(w, wide[:, 1:cols + 1], act_mode=1, step=step), y8)
    rq_ctx.check()


def test_kquant_matmul_extreme_blocks(rq_ctx, oracle):
    """Arbitrary block bytes: every six-bit scale and minimum, every int8 scale, codes at both ends of their range."""
    rng = np.random.default_rng(5)
    for t in (ol.Q4_K, ol.Q6_K):
        per, stride = ol.GEOMETRY[t]
        rows, cols, tokens = 256, 1024, 24
        raw = rng.integers(0, 256, size=(rows * cols // per, stride), dtype=np.uint8)
        for off in ([0, 2] if t == ol.Q4_K else [208]):
            raw[:, off + 1] = (raw[:, off + 1] & 0x83) | 0x10  # |d| in [2^-11, 2^-7): sums stay well inside fp32
        x = oracle.normal(64, t, tokens * cols, 1.0).reshape(tokens, cols)
        w = rq_ctx.weight_from_host(t, raw.reshape(-1), rows, cols)
        y = rq_ctx.matmul(w, cuda(x)).cpu().numpy()
        exact = x.astype(np.float64) @ oracle.dequantize(t, raw.reshape(-1)).astype(np.float64).reshape(rows, cols).T
        assert np.max(np.abs(y - exact)) <= 3e-6 * np.max(np.abs(exact)), t
        rq_ctx.check()
