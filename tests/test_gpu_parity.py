"""Parity of the CUDA path with the CPU oracle, through the C ABI. GPU only (-m gpu).

Bars: dequantised weights, quantised blocks and int8 activation records are bit / byte exact;
matvec outputs are within 1e-3 relative (fp32 accumulate) of the oracle in the same activation
mode, measured as max_i |y_i - ref_i| / max(|ref_i|, 1e-3 * max|ref|) -- the floor keeps outputs
that cancel to nearly zero from dominating the ratio.
"""
import numpy as np
import pytest

from tests import oracle_lib as ol

pytestmark = pytest.mark.gpu

TYPES = [ol.Q4_0, ol.Q8_0, ol.Q4_K, ol.Q6_K]
TOL = 1e-3


def rel_err(y, ref):
    y, ref = np.asarray(y, np.float64), np.asarray(ref, np.float64)
    floor = 1e-3 * np.max(np.abs(ref))
    return float(np.max(np.abs(y - ref) / np.maximum(np.abs(ref), floor)))


def torch_cuda(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("t", TYPES)
def test_dequant_bit_exact_and_export_roundtrip(rq_ctx, oracle, t):
    per, _ = ol.GEOMETRY[t]
    rows, cols = 37, 3 * 256
    blocks = oracle.quantize(t, oracle.normal(1, t, rows * cols, 0.02))
    w = rq_ctx.weight_from_host(t, blocks, rows, cols)
    assert w.nbytes == blocks.size
    got = rq_ctx.dequant(w).cpu().numpy().reshape(-1)
    assert np.array_equal(got.view(np.uint32), oracle.dequantize(t, blocks).view(np.uint32))
    assert np.array_equal(rq_ctx.export(w), blocks)
    # arbitrary bytes (finite scales): every code / scale pattern
    rng = np.random.default_rng(t)
    stride = ol.GEOMETRY[t][1]
    raw = rng.integers(0, 256, size=(rows * cols // per, stride), dtype=np.uint8)
    for off in ([0, 2] if t == ol.Q4_K else [208] if t == ol.Q6_K else [0]):
        raw[:, off + 1] &= 0xBF
    w2 = rq_ctx.weight_from_host(t, raw.reshape(-1), rows, cols)
    got = rq_ctx.dequant(w2).cpu().numpy().reshape(-1)
    assert np.array_equal(got.view(np.uint32), oracle.dequantize(t, raw.reshape(-1)).view(np.uint32))
    assert np.array_equal(rq_ctx.export(w2), raw.reshape(-1))


@pytest.mark.parametrize("t", TYPES)
def test_row_shard_upload(rq_ctx, oracle, t):
    """A die's share of a row split holds exactly its rows."""
    rows, cols = 20, 512
    blocks = oracle.quantize(t, oracle.normal(2, t, rows * cols, 0.02))
    full = oracle.dequantize(t, blocks).reshape(rows, cols)
    w = rq_ctx.weight_from_host(t, blocks, rows, cols, row_first=5, row_count=9)
    assert (w.rows, w.cols) == (9, cols)
    assert np.array_equal(rq_ctx.dequant(w).cpu().numpy(), full[5:14])


@pytest.mark.parametrize("t", TYPES)
def test_quantiser_byte_exact(rq_ctx, oracle, t):
    per, _ = ol.GEOMETRY[t]
    values = oracle.normal(3, t, 700 * per, 0.02)
    # edge blocks: zeros, a constant, one spike, equal magnitudes of both signs, tiny values
    edge = np.zeros((5, per), np.float32)
    edge[1, :] = 0.01
    edge[2, 3] = -0.5
    edge[3, ::2], edge[3, 1::2] = 0.25, -0.25
    edge[4, :] = -1e-20
    values = np.concatenate([values, edge.reshape(-1), oracle.normal(3, 50 + t, 64 * per, 3.0)])
    got = rq_ctx.quantize(t, torch_cuda(values)).cpu().numpy()
    want = oracle.quantize(t, values)
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, f"{bad.size} bytes differ, first at {bad[:5]} (block {bad[0] // ol.GEOMETRY[t][1]})"


@pytest.mark.parametrize("step", [32, 256])
def test_activation_records_bit_exact(rq_ctx, oracle, step):
    cols = 4096 + 32 * 3  # a partial trailing group under step 256
    x = oracle.normal(4, step, 3 * cols, 1.0).reshape(3, cols)
    x[1, 64:96] = 0.0
    x[2, 5], x[2, 9] = -7.0, 7.0  # a tie of opposite signs: the first wins
    got = rq_ctx.activation_records(torch_cuda(x), step).cpu().numpy()
    for p in range(3):
        assert np.array_equal(got[p], oracle.activation_records(x[p], step)), p


SHAPES = [(ol.Q4_K, 64, 4096), (ol.Q4_K, 33, 512), (ol.Q4_K, 7, 2048), (ol.Q6_K, 64, 14336 // 4), (ol.Q6_K, 33, 2560), (ol.Q6_K, 5, 256),
          (ol.Q8_0, 64, 4096), (ol.Q8_0, 9, 96), (ol.Q4_0, 64, 4096), (ol.Q4_0, 17, 160), (ol.Q4_K, 1, 256), (ol.Q8_0, 1, 32)]


@pytest.mark.parametrize("t,rows,cols", SHAPES)
def test_matvec_float_parity(rq_ctx, oracle, t, rows, cols):
    blocks = oracle.quantize(t, oracle.normal(5, t + rows, rows * cols, 0.02))
    x = oracle.normal(5, 70 + t, cols, 1.0)
    w = rq_ctx.weight_from_host(t, blocks, rows, cols)
    y = rq_ctx.matvec(w, torch_cuda(x)).cpu().numpy()
    ref = oracle.matvec(t, blocks, rows, cols, x, ol.FLOAT_RUN)
    assert rel_err(y, ref) <= TOL
    # both of the reference's fp32 orders and the float64 product sit inside the same band
    assert rel_err(y, oracle.matvec(t, blocks, rows, cols, x, ol.FLOAT_EXACT)) <= TOL
    exact = oracle.dequantize(t, blocks).astype(np.float64).reshape(rows, cols) @ x.astype(np.float64)
    assert rel_err(y, exact) <= 1e-4


@pytest.mark.parametrize("step", [32, 256])
@pytest.mark.parametrize("t,rows,cols", SHAPES)
def test_matvec_int8_parity(rq_ctx, oracle, t, rows, cols, step):
    blocks = oracle.quantize(t, oracle.normal(6, t + rows, rows * cols, 0.02))
    x = oracle.normal(6, 80 + t, cols, 1.0)
    w = rq_ctx.weight_from_host(t, blocks, rows, cols)
    y = rq_ctx.matvec(w, torch_cuda(x), act_mode=1, step=step).cpu().numpy()
    ref = oracle.matvec(t, blocks, rows, cols, x, ol.INT8, step)
    assert rel_err(y, ref) <= TOL
    # the integer parts are exact, so the distance to the oracle is fp32 summation order only
    assert rel_err(y, ref) <= 5e-5


@pytest.mark.parametrize("mode,step", [(0, 32), (1, 32), (1, 256)])
@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("tokens", [2, 4, 5])
def test_matvec_tokens_and_strides(rq_ctx, oracle, t, tokens, mode, step):
    """Several positions, token-major and the reference's channel-major planes (x[k*len + pos])."""
    import torch

    rows, cols = 45, 768
    blocks = oracle.quantize(t, oracle.normal(8, t, rows * cols, 0.02))
    x = oracle.normal(8, 90 + t, tokens * cols, 1.0).reshape(tokens, cols)
    w = rq_ctx.weight_from_host(t, blocks, rows, cols)
    omode = ol.FLOAT_RUN if mode == 0 else ol.INT8
    # step 256 on Q4_K is position-dependent in the reference (gemm rows vs gemv rows): same band
    ref = oracle.matvec(t, blocks, rows, cols, x, omode, step)
    y = rq_ctx.matvec(w, torch_cuda(x), act_mode=mode, step=step).cpu().numpy()
    assert rel_err(y, ref) <= TOL
    # channel-major planes through the raw strides
    xc = torch_cuda(x.T)  # [cols][tokens]
    yc = torch.zeros((rows, tokens), dtype=torch.float32, device="cuda")
    rc = rq_ctx.matvec_raw(w, xc.data_ptr(), tokens, 1, tokens, yc.data_ptr(), tokens, 1, mode, step, stream=torch.cuda.current_stream())
    assert rc == 0
    assert np.array_equal(yc.cpu().numpy().T, y)
    # a window equals its positions one at a time, bit for bit (suite.rs:343-371)
    for p in range(tokens):
        one = rq_ctx.matvec(w, torch_cuda(x[p]), act_mode=mode, step=step).cpu().numpy()
        assert np.array_equal(one.view(np.uint32), y[p].view(np.uint32)), p


def test_matvec_host_entry(rq_ctx, oracle):
    rows, cols = 130, 1024
    blocks = oracle.quantize(ol.Q4_K, oracle.normal(9, 0, rows * cols, 0.02))
    x = oracle.normal(9, 1, 2 * cols, 1.0).reshape(2, cols)
    w = rq_ctx.weight_from_host(ol.Q4_K, blocks, rows, cols)
    for mode, omode in ((0, ol.FLOAT_RUN), (1, ol.INT8)):
        y = rq_ctx.matvec_host(w, x, act_mode=mode, step=32)
        assert rel_err(y, oracle.matvec(ol.Q4_K, blocks, rows, cols, x, omode, 32)) <= TOL


def test_golden_vectors_on_gpu(rq_ctx, oracle):
    """The reference's own vectors through the CUDA path."""
    from pathlib import Path

    golden = Path(__file__).resolve().parent / "golden"
    g = np.load(golden / "suite_q8_0_table.npz")
    w = rq_ctx.weight_from_host(ol.Q8_0, g["blocks"], 4, 32)
    assert np.array_equal(rq_ctx.dequant(w).cpu().numpy(), g["expected"])
    k = np.load(golden / "bench_q4k_kat.npz")
    rows = int(k["rows"])
    wk = rq_ctx.weight_from_host(ol.Q4_K, k["blocks"], rows, 4096)
    y = rq_ctx.matvec(wk, torch_cuda(k["x_dequant"])).cpu().numpy()
    assert np.max(np.abs(y - k["expected"])) <= 2e-6 * np.max(np.abs(k["expected"]))
    # the check's activations are integers times a power-of-two-grid step: the int8 path sees them too
    y8 = rq_ctx.matvec(wk, torch_cuda(k["x_dequant"]), act_mode=1, step=32).cpu().numpy()
    assert rel_err(y8, oracle.matvec(ol.Q4_K, k["blocks"], rows, 4096, k["x_dequant"], ol.INT8, 32)) <= 5e-5


def test_argument_validation(rq_ctx, oracle):
    """Bad handles, shapes and enums come back as a status with text; nothing aborts."""
    import ctypes

    import recipe_dev_b200 as rq

    lib = rq_ctx.lib
    blocks = oracle.quantize(ol.Q4_K, oracle.normal(10, 0, 4 * 256, 0.02))
    out = ctypes.c_void_p()
    assert lib.rq_weight_prepare(rq_ctx.handle, 16, blocks.ctypes.data, 4, 256, 0, 4, ctypes.byref(out)) == -1  # IQ2_XXS: a grid format, not served
    assert lib.rq_weight_prepare(rq_ctx.handle, ol.Q4_K, blocks.ctypes.data, 4, 250, 0, 4, ctypes.byref(out)) == -1
    assert b"multiple" in lib.rq_last_error()
    assert lib.rq_weight_prepare(rq_ctx.handle, ol.Q4_K, blocks.ctypes.data, 4, 256, 2, 3, ctypes.byref(out)) == -1
    assert lib.rq_weight_prepare(rq_ctx.handle, ol.Q4_K, None, 4, 256, 0, 4, ctypes.byref(out)) == -1
    w = rq_ctx.weight_from_host(ol.Q4_K, blocks, 4, 256)
    x = torch_cuda(np.zeros(256, np.float32))
    y = torch_cuda(np.zeros(4, np.float32))
    assert rq_ctx.matvec_raw(w, x.data_ptr(), 1, 256, 1, y.data_ptr(), 1, 4, 7, 32) == -1
    assert rq_ctx.matvec_raw(w, x.data_ptr(), 1, 256, 1, y.data_ptr(), 1, 4, 1, 64) == -1
    assert rq_ctx.matvec_raw(w, 0, 1, 256, 1, y.data_ptr(), 1, 4, 0, 32) == -1
    assert rq_ctx.matvec_raw(w, x.data_ptr(), 1, 256, 0, y.data_ptr(), 1, 4, 0, 32) == -1
    with pytest.raises(rq.RqError):
        rq_ctx.quantize(ol.Q4_K, torch_cuda(np.zeros(100, np.float32)))
    # the context still works afterwards
    assert np.all(np.isfinite(rq_ctx.matvec(w, x).cpu().numpy()))


@pytest.mark.parametrize("mode,step", [(0, 32), (1, 32), (1, 256)])
@pytest.mark.parametrize("t,cols", [(ol.Q4_K, 1024), (ol.Q6_K, 768), (ol.Q8_0, 512), (ol.Q4_0, 96)])
def test_matvec_multi_equals_single(rq_ctx, oracle, t, cols, mode, step):
    """q/k/v-style siblings in one call give, bit for bit, what one call per matrix gives."""
    import torch

    row_counts = [70, 19, 33]
    x = oracle.normal(12, t, 2 * cols, 1.0).reshape(2, cols)
    xd = torch_cuda(x)
    ws, singles = [], []
    for i, rows in enumerate(row_counts):
        blocks = oracle.quantize(t, oracle.normal(12, 10 * t + i, rows * cols, 0.02))
        w = rq_ctx.weight_from_host(t, blocks, rows, cols)
        ws.append(w)
        singles.append(rq_ctx.matvec(w, xd, act_mode=mode, step=step).cpu().numpy())
        omode = ol.FLOAT_RUN if mode == 0 else ol.INT8
        assert rel_err(singles[-1], oracle.matvec(t, blocks, rows, cols, x, omode, step)) <= TOL
    # the siblings' outputs side by side in one [tokens, all rows] plane: one token stride for all
    plane = torch.zeros((2, sum(row_counts)), dtype=torch.float32, device="cuda")
    ys, at = [], 0
    for rows in row_counts:
        ys.append(plane[:, at:at + rows])
        at += rows
    rq_ctx.matvec_multi(ws, xd, ys, act_mode=mode, step=step)
    for y, ref in zip(ys, singles):
        assert np.array_equal(y.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    rq_ctx.check()


@pytest.mark.parametrize("step", [32, 256])
@pytest.mark.parametrize("t,rows,cols", [(ol.Q4_K, 70, 4096), (ol.Q6_K, 33, 14336), (ol.Q6_K, 61, 2560), (ol.Q4_K, 50, 512), (ol.Q4_K, 9, 14336),
                                         (ol.Q8_0, 40, 2048), (ol.Q4_0, 40, 1024), (ol.Q4_K, 21, 8192)])
def test_int8_window_equals_positions_on_every_kernel_scheme(rq_ctx, oracle, t, rows, cols, step):
    """The single-token int8 matvec runs one of three schemes by row length (a row inside a warp, a row
    split over the warps, partial sums through shared memory); a multi-token window must give every
    position the bits its own single-token call gives (suite.rs:343-371), whichever scheme that is."""
    tokens = 3
    blocks = oracle.quantize(t, oracle.normal(14, t + cols, rows * cols, 0.02))
    x = oracle.normal(14, 7 + t, tokens * cols, 1.0).reshape(tokens, cols)
    w = rq_ctx.weight_from_host(t, blocks, rows, cols)
    y = rq_ctx.matvec(w, torch_cuda(x), act_mode=1, step=step).cpu().numpy()
    # integer dots are exact; what is left is fp32 summation order over up to 14336 inputs
    assert rel_err(y, oracle.matvec(t, blocks, rows, cols, x, ol.INT8, step)) <= 2e-4
    for p in range(tokens):
        one = rq_ctx.matvec(w, torch_cuda(x[p]), act_mode=1, step=step).cpu().numpy()
        assert np.array_equal(one.view(np.uint32), y[p].view(np.uint32)), p
        # the records the fused launch left behind serve a cached call with the same bits
        again = rq_ctx.matvec(w, torch_cuda(x[p]), act_mode=2, step=step).cpu().numpy()
        assert np.array_equal(one.view(np.uint32), again.view(np.uint32)), p
    rq_ctx.check()


@pytest.mark.parametrize("t,cols", [(ol.Q4_K, 4096), (ol.Q6_K, 14336), (ol.Q6_K, 2560)])
def test_fused_quantiser_equals_standalone_quantiser(rq_ctx, oracle, t, cols):
    """rq_matvec (int8) quantises x inside the matvec launch; rq_matvec_int8_static runs the standalone
    quantiser kernel first. Same records, same kernel after them: the same bits."""
    rows = 40
    blocks = oracle.quantize(t, oracle.normal(15, t, rows * cols, 0.02))
    x = oracle.normal(15, 1, cols, 1.0)
    big = float(np.abs(x).max()) * 2
    x[5], x[20] = big, -big  # a tie in magnitude inside one group: the first index wins
    w = rq_ctx.weight_from_host(t, blocks, rows, cols)
    for step in (32, 256):
        fused = rq_ctx.matvec(w, torch_cuda(x), act_mode=1, step=step).cpu().numpy()
        static = rq_ctx.matvec_int8_static(w, torch_cuda(x), step=step).cpu().numpy()
        assert np.array_equal(fused.view(np.uint32), static.view(np.uint32))


def test_matvec_multi_host_equals_single_host_calls(rq_ctx, oracle):
    """Sibling projections through host buffers in one call: the bits of one rq_matvec_host call per matrix."""
    t, cols = ol.Q4_K, 1024
    rows = [96, 32, 40]
    ws = [rq_ctx.weight_from_host(t, oracle.quantize(t, oracle.normal(31, i, r * cols, 0.02)), r, cols) for i, r in enumerate(rows)]
    for tokens in (1, 3):
        x = oracle.normal(31, 9, tokens * cols, 1.0).reshape(tokens, cols)
        xs = x[0] if tokens == 1 else x
        for mode in (0, 1):
            got = rq_ctx.matvec_multi_host(ws, xs, act_mode=mode, step=32)
            for w, y in zip(ws, got):
                one = rq_ctx.matvec_host(w, xs, act_mode=mode, step=32)
                assert np.array_equal(np.ascontiguousarray(y).view(np.uint32), one.view(np.uint32))
    rq_ctx.check()


EDGE_SHAPES = [
    # (type, rows, cols): every row layout of the streaming kernel, with row counts around the stage sizes
    (ol.Q4_K, 1, 256), (ol.Q4_K, 3, 512), (ol.Q4_K, 29, 1024), (ol.Q6_K, 57, 2048), (ol.Q4_K, 15, 4096), (ol.Q4_K, 113, 4096),
    (ol.Q6_K, 5, 14336), (ol.Q4_K, 2, 7168), (ol.Q6_K, 41, 5120), (ol.Q4_K, 9, 1280), (ol.Q6_K, 8, 2560), (ol.Q4_K, 3, 32768),
    (ol.Q4_K, 6, 8192), (ol.Q8_0, 23, 4096), (ol.Q4_0, 31, 2560), (ol.Q8_0, 2, 14336), (ol.Q4_K, 300, 768), (ol.Q6_K, 1, 3072),
    # wide rows with enough of them for several ring stages per CTA: the fp32 records of 14336 inputs (62 KB) leave two CTAs per
    # SM no room for a ring, so these launches run one CTA per SM
    (ol.Q6_K, 700, 14336), (ol.Q4_K, 450, 14336),
]


@pytest.mark.parametrize("t,rows,cols", EDGE_SHAPES)
def test_matvec_every_row_layout_and_ragged_row_counts(rq_ctx, oracle, t, rows, cols):
    """Widths that take the in-warp layout (powers of two, padded), the split layouts (7, 5 and 8 warps) and the
    shared-memory partial sums, with row counts that leave stages and CTAs partly empty; both activation modes,
    one token and a window of three."""
    blocks = oracle.quantize(t, oracle.normal(41, t + cols, rows * cols, 0.02))
    x = oracle.normal(41, 3 + t, 3 * cols, 1.0).reshape(3, cols)
    w = rq_ctx.weight_from_host(t, blocks, rows, cols)
    for mode, omode in ((1, ol.INT8), (0, ol.FLOAT_RUN)):
        ref = oracle.matvec(t, blocks, rows, cols, x, omode, 32)
        y = rq_ctx.matvec(w, torch_cuda(x), act_mode=mode, step=32).cpu().numpy()
        assert rel_err(y, ref) <= TOL, (mode, "window")
        for p in range(3):
            one = rq_ctx.matvec(w, torch_cuda(x[p]), act_mode=mode, step=32).cpu().numpy()
            assert rel_err(one, ref[p]) <= TOL, (mode, p)
            assert np.array_equal(one.view(np.uint32), y[p].view(np.uint32)), (mode, p)
    rq_ctx.check()


def test_matvec_multi_ragged_segments(rq_ctx, oracle):
    """Four matrices of unequal, awkward row counts in one launch: stages never straddle a matrix."""
    t, cols = ol.Q4_K, 4096
    rows = [1, 33, 14, 200]
    bl = [oracle.quantize(t, oracle.normal(42, i, r * cols, 0.02)) for i, r in enumerate(rows)]
    ws = [rq_ctx.weight_from_host(t, b, r, cols) for b, r in zip(bl, rows)]
    x = oracle.normal(42, 9, cols, 1.0)
    import torch

    for mode in (1, 0):
        plane = torch.zeros(sum(rows), dtype=torch.float32, device="cuda")
        offs = np.cumsum([0] + rows)
        ys = [plane[int(offs[i]):int(offs[i + 1])] for i in range(4)]
        rq_ctx.matvec_multi(ws, torch_cuda(x), ys, act_mode=mode, step=32)
        for w, y in zip(ws, ys):
            one = rq_ctx.matvec(w, torch_cuda(x), act_mode=mode, step=32)
            assert torch.equal(one, y)
    rq_ctx.check()


@pytest.mark.parametrize("t,cols", [(ol.Q6_K, 2560), (ol.Q8_0, 2560), (ol.Q4_K, 1280), (ol.Q4_0, 5120)])
@pytest.mark.parametrize("tokens", [2, 3, 5])
def test_int8_windows_over_rows_of_five_warps(rq_ctx, oracle, t, cols, tokens):
    """Rows of 5 x 2^k items take token pairs in registers: every position of a window (even and odd lengths, one matrix and
    several in one launch) gets the bits its own single-token call gives, and the oracle's int8 answer."""
    import torch

    rows = [300, 17, 64]
    bl = [oracle.quantize(t, oracle.normal(43, 10 * t + i, r * cols, 0.02)) for i, r in enumerate(rows)]
    ws = [rq_ctx.weight_from_host(t, b, r, cols) for b, r in zip(bl, rows)]
    x = oracle.normal(43, 99 + tokens, tokens * cols, 1.0).reshape(tokens, cols)
    xd = torch_cuda(x)
    for step in (32, 256):
        singles = [[rq_ctx.matvec(w, xd[p], act_mode=1, step=step) for p in range(tokens)] for w in ws]
        for w, b, r, ones in zip(ws, bl, rows, singles):
            y = rq_ctx.matvec(w, xd, act_mode=1, step=step)
            for p in range(tokens):
                assert torch.equal(y[p], ones[p]), (step, p)
            ref = oracle.matvec(t, b, r, cols, x, ol.INT8, step)
            assert rel_err(y.cpu().numpy(), ref) <= 2e-4  # exact integer dots; the fp32 sums over 2560 .. 5120 inputs are added in another order
        plane = torch.zeros(tokens, sum(rows), dtype=torch.float32, device="cuda")
        offs = np.cumsum([0] + rows)
        ys = [plane[:, int(offs[i]):int(offs[i + 1])] for i in range(len(rows))]
        rq_ctx.matvec_multi(ws, xd, ys, act_mode=1, step=step)
        for y, ones in zip(ys, singles):
            for p in range(tokens):
                assert torch.equal(y[p], ones[p]), ("multi", step, p)
    rq_ctx.check()
