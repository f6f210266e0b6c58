"""The CPU oracle against the reference's own vectors, an independent NumPy restatement and
domain properties. No GPU."""
from pathlib import Path

import numpy as np
import pytest

from oracle import np_unpack
from tests import oracle_lib as ol

GOLDEN = Path(__file__).resolve().parent / "golden"
TYPES = [ol.Q4_0, ol.Q8_0, ol.Q4_K, ol.Q6_K]


def test_suite_q8_0_table(oracle):
    """.github/runtime/suite.rs:191-194: d = 0x2400, codes 32, 96, -80, 48."""
    g = np.load(GOLDEN / "suite_q8_0_table.npz")
    got = oracle.dequantize(ol.Q8_0, g["blocks"]).reshape(4, 32)
    assert np.array_equal(got.view(np.uint32), g["expected"].view(np.uint32))
    assert np.array_equal(np_unpack.dequantize(ol.Q8_0, g["blocks"]).reshape(4, 32), g["expected"])
    # a matvec over the table: every row is a constant, so y = c * sum(x)
    x = np.arange(32, dtype=np.float32) - 10.0
    y = oracle.matvec(ol.Q8_0, g["blocks"], 4, 32, x, ol.FLOAT_RUN)
    assert np.allclose(y, np.array([0.5, 1.5, -1.25, 0.75]) * x.sum(), rtol=1e-6)


def test_bench_q4k_kat(oracle):
    """evidence/2026-10-10-m60-p2p/bench.rs:177-228: Q4_K nibble order, six-bit scale unpack and the
    (sc*dot*d - m*sum*dmin)*d8 algebra, checked through the dequantised activations."""
    g = np.load(GOLDEN / "bench_q4k_kat.npz")
    rows = int(g["rows"])
    expected = g["expected"].astype(np.float64)
    for mode in (ol.FLOAT_RUN, ol.FLOAT_EXACT):
        y = oracle.matvec(ol.Q4_K, g["blocks"], rows, 4096, g["x_dequant"], mode).astype(np.float64)
        assert np.max(np.abs(y - expected)) <= 2e-6 * np.max(np.abs(expected)), mode
    # and against the NumPy restatement of the unpacking in float64
    w = np_unpack.dequantize(ol.Q4_K, g["blocks"]).astype(np.float64).reshape(rows, 4096)
    ref = w @ g["x_dequant"].astype(np.float64)
    assert np.max(np.abs(ref - expected)) <= 1e-6 * np.max(np.abs(expected))


def test_oracle_regression(oracle):
    """Committed outputs of the oracle on seeded inputs: any edit that moves a bit is visible."""
    g = np.load(GOLDEN / "oracle_regression.npz")
    rows, cols = 6, 512
    for name, t in (("q4_0", ol.Q4_0), ("q8_0", ol.Q8_0), ("q4_k", ol.Q4_K), ("q6_k", ol.Q6_K)):
        w = oracle.normal(7, t, rows * cols, 0.02)
        x = oracle.normal(7, 100 + t, 2 * cols, 1.0).reshape(2, cols)
        blocks = oracle.quantize(t, w)
        assert np.array_equal(blocks, g[f"{name}_blocks"]), name
        assert np.array_equal(oracle.dequantize(t, blocks).view(np.uint32), g[f"{name}_dequant_bits"]), name
        for mode, label in ((ol.FLOAT_RUN, "run"), (ol.FLOAT_EXACT, "exact")):
            assert np.array_equal(oracle.matvec(t, blocks, rows, cols, x, mode).view(np.uint32), g[f"{name}_y_{label}"]), (name, label)
        for step in (32, 256):
            assert np.array_equal(oracle.matvec(t, blocks, rows, cols, x, ol.INT8, step).view(np.uint32), g[f"{name}_y_int8_{step}"]), (name, step)
    x = oracle.normal(7, 999, 512, 1.0)
    assert np.array_equal(oracle.activation_records(x, 32), g["act_records_32"])
    assert np.array_equal(oracle.activation_records(x, 256), g["act_records_256"])
    scores = oracle.normal(7, 1000, 64 * 3, 1.0).reshape(64, 3)
    assert np.array_equal(oracle.topk(scores, 8, 0, True).view(np.uint32), g["topk_softmax_renorm"])
    assert np.array_equal(oracle.topk(scores, 8, 0, False).view(np.uint32), g["topk_softmax_plain"])
    assert np.array_equal(oracle.topk(scores, 8, 1, True).view(np.uint32), g["topk_sigmoid_renorm"])


def test_fp16_codec_matches_ieee(oracle):
    """recipe.rs:15098-15132 is IEEE round-to-nearest-even wherever the result is finite."""
    rng = np.random.default_rng(1)
    vals = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * np.float32(0.02),
        rng.standard_normal(2000).astype(np.float32) * np.float32(100.0),
        (rng.standard_normal(2000) * 1e-6).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 6.1035156e-05, 5.9604645e-08, 2.9802322e-08, 1.0, -1.0, 0.33333334], np.float32),
    ])
    for v in vals:
        assert oracle.fp16(float(v)) == int(np.float32(v).astype(np.float16).view(np.uint16)), v
    for h in range(0, 0x7C00, 7):  # every finite half value decodes exactly
        assert oracle.unfp16(h) == float(np.array([h], np.uint16).view(np.float16)[0])


@pytest.mark.parametrize("t", TYPES)
def test_dequant_matches_numpy_restatement(oracle, t):
    """Two independent restatements of recipe.rs:3687-3833 agree bit for bit, on quantiser output
    and on arbitrary bytes (every scale / code pattern, including ones no quantiser emits)."""
    per, stride = ol.GEOMETRY[t]
    w = oracle.normal(11, t, 64 * per, 0.02)
    blocks = oracle.quantize(t, w)
    a, b = oracle.dequantize(t, blocks), np_unpack.dequantize(t, blocks)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    rng = np.random.default_rng(t)
    raw = rng.integers(0, 256, size=200 * stride, dtype=np.uint8).reshape(200, stride)
    # keep the fp16 scales finite: clear the top exponent bit of each half
    for off in ([0, 2] if t == ol.Q4_K else [208] if t == ol.Q6_K else [0]):
        raw[:, off + 1] &= 0xBF
    a, b = oracle.dequantize(t, raw), np_unpack.dequantize(t, raw)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("t,bound", [(ol.Q8_0, 0.57 / 127), (ol.Q4_0, 0.13), (ol.Q4_K, 0.12), (ol.Q6_K, 0.02)])
def test_quantise_dequantise_error_bound(oracle, t, bound):
    """dequant(quantise(x)) stays within the format's step of x (relative to the block maximum).
    Q8_0: half a step plus the fp16 rounding of the step over 127 codes. Q4_0: the extreme maps to -8,
    so a value of the opposite sign and equal size clips at 7 steps, one eighth of the maximum away."""
    per, _ = ol.GEOMETRY[t]
    w = oracle.normal(3, t, 256 * per, 0.02)
    back = oracle.dequantize(t, oracle.quantize(t, w))
    err = np.abs(back - w).reshape(-1, per).max(axis=1)
    peak = np.abs(w).reshape(-1, per).max(axis=1)
    assert np.all(err <= bound * peak * 1.02 + 1e-9)


@pytest.mark.parametrize("t", TYPES)
def test_quantiser_edge_blocks(oracle, t):
    """All-zero, constant, single-spike and tie blocks quantise without NaN and dequantise sanely."""
    per, _ = ol.GEOMETRY[t]
    cases = np.zeros((5, per), np.float32)
    cases[1, :] = 0.01
    cases[2, 3] = -0.5
    cases[3, ::2], cases[3, 1::2] = 0.25, -0.25  # equal magnitudes of both signs
    cases[4, :] = -1e-20
    back = oracle.dequantize(t, oracle.quantize(t, cases.reshape(-1))).reshape(5, per)
    assert np.all(np.isfinite(back))
    assert np.array_equal(back[0], np.zeros(per, np.float32))
    assert abs(back[2, 3] + 0.5) < 0.05 and np.max(np.abs(np.delete(back[2], 3))) < 0.05


def test_partial_block_pads_with_zeros(oracle):
    """encode_blocks pads a trailing partial slice with zeros (recipe.rs:16171-16173)."""
    w = oracle.normal(5, 0, 40, 0.02)
    padded = np.concatenate([w, np.zeros(24, np.float32)])
    assert np.array_equal(oracle.quantize(ol.Q8_0, w), oracle.quantize(ol.Q8_0, padded))


def test_activation_records(oracle):
    """amd-nv-cpu.ll:1381-1517: the extreme codes to -127, d = 1/(-127/extreme), zero groups give d = 0,
    and a 256 step shares one d across eight records."""
    x = oracle.normal(9, 1, 512, 1.0)
    x[64:96] = 0.0
    r32 = oracle.activation_records(x, 32)
    d = r32[:, :4].copy().view(np.float32).reshape(-1)
    codes = r32[:, 4:].view(np.int8)
    for b in range(16):
        blk = x[b * 32:(b + 1) * 32]
        if b == 2:
            assert d[b] == 0.0 and not codes[b].any()
            continue
        ext = blk[np.argmax(np.abs(blk))]
        inv = np.float32(-127.0) / np.float32(ext)
        assert d[b] == np.float32(1.0) / inv
        assert codes[b][np.argmax(np.abs(blk))] == -127
        assert np.array_equal(codes[b], np.clip(np.rint(blk * inv), -128, 127).astype(np.int8))
    r256 = oracle.activation_records(x, 256)
    d256 = r256[:, :4].copy().view(np.float32).reshape(-1)
    assert len(set(d256[:8])) == 1 and len(set(d256[8:])) == 1
    # ties: the first of two equal magnitudes wins, whatever its sign
    t = np.zeros(32, np.float32)
    t[5], t[9] = -2.0, 2.0
    rec = oracle.activation_records(t, 32)
    assert rec[0, :4].copy().view(np.float32)[0] > 0 and rec[0, 4:].view(np.int8)[5] == -127 and rec[0, 4:].view(np.int8)[9] == 127


@pytest.mark.parametrize("t", TYPES)
def test_dot_semantics_agree(oracle, t):
    """The three dot semantics of one row agree to their own rounding: the two FLOAT orders to
    fp32 summation error, INT8 to the int8 rounding of the activations (about 1 %)."""
    per, _ = ol.GEOMETRY[t]
    rows, cols = 24, 1024
    blocks = oracle.quantize(t, oracle.normal(21, t, rows * cols, 0.02))
    x = oracle.normal(21, 50 + t, cols, 1.0)
    w = oracle.dequantize(t, blocks).astype(np.float64).reshape(rows, cols)
    exact = w @ x.astype(np.float64)
    scale = np.max(np.abs(exact))
    for mode in (ol.FLOAT_RUN, ol.FLOAT_EXACT):
        y = oracle.matvec(t, blocks, rows, cols, x, mode)
        assert np.max(np.abs(y - exact)) <= 5e-6 * scale
    for step in (32, 256):
        y = oracle.matvec(t, blocks, rows, cols, x, ol.INT8, step)
        assert np.max(np.abs(y - exact)) <= 3e-2 * scale
        # against the dequantised records the int8 dot is exact up to fp32 rounding
        rec = oracle.activation_records(x, step)
        xq = (rec[:, 4:].view(np.int8).astype(np.float64) * rec[:, :4].copy().view(np.float32).astype(np.float64)).reshape(-1)
        assert np.max(np.abs(y - w @ xq)) <= 5e-6 * scale


@pytest.mark.parametrize("t", TYPES)
def test_prefill_equals_steps(oracle, t):
    """suite.rs:343-371: a window of positions gives, bit for bit, what the positions give one at a
    time (FLOAT and INT8 step 32; the 256-step Q4_K order is position-dependent by design)."""
    rows, cols, tokens = 8, 512, 5
    blocks = oracle.quantize(t, oracle.normal(31, t, rows * cols, 0.02))
    x = oracle.normal(31, 60 + t, tokens * cols, 1.0).reshape(tokens, cols)
    for mode, step in ((ol.FLOAT_RUN, 32), (ol.FLOAT_EXACT, 32), (ol.INT8, 32)):
        whole = oracle.matvec(t, blocks, rows, cols, x, mode, step)
        for p in range(tokens):
            one = oracle.matvec(t, blocks, rows, cols, x[p], mode, step)
            assert np.array_equal(one.view(np.uint32), whole[p].view(np.uint32))


def test_linearity_and_thread_invariance(oracle):
    rows, cols = 33, 768
    blocks = oracle.quantize(ol.Q6_K, oracle.normal(41, 0, rows * cols, 0.02))
    x = oracle.normal(41, 1, cols, 1.0)
    a = oracle.matvec(ol.Q6_K, blocks, rows, cols, x, ol.FLOAT_RUN, threads=1)
    b = oracle.matvec(ol.Q6_K, blocks, rows, cols, x, ol.FLOAT_RUN, threads=7)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    two = oracle.matvec(ol.Q6_K, blocks, rows, cols, 2.0 * x, ol.FLOAT_RUN)
    assert np.array_equal(two.view(np.uint32), (2.0 * a).astype(np.float32).view(np.uint32))  # scaling by two is exact


def test_topk_properties(oracle):
    """amd-nv-cpu.ll:4666-4716: exactly top-k non-zero weights; renormalised weights sum to one; ties go
    to the lower expert; a plain softmax divides by every expert."""
    scores = oracle.normal(51, 0, 256 * 4, 1.0).reshape(256, 4)
    w = oracle.topk(scores, 8, 0, True)
    assert np.all((w != 0).sum(axis=0) == 8)
    assert np.allclose(w.sum(axis=0), 1.0, atol=1e-6)
    for p in range(4):
        assert set(np.nonzero(w[:, p])[0]) == set(np.argsort(-scores[:, p], kind="stable")[:8])
    plain = oracle.topk(scores, 8, 0, False)
    soft = np.exp(scores.astype(np.float64) - scores.max(axis=0)) / np.exp(scores.astype(np.float64) - scores.max(axis=0)).sum(axis=0)
    assert np.allclose(plain[plain != 0], soft[plain != 0], rtol=1e-5)
    tie = np.zeros((6, 1), np.float32)
    assert list(np.nonzero(oracle.topk(tie, 2, 0, True)[:, 0])[0]) == [0, 1]
    sig = oracle.topk(scores, 8, 1, False)
    assert np.allclose(sig[sig != 0], 1.0 / (1.0 + np.exp(-scores[sig != 0].astype(np.float64))), rtol=1e-5)


def test_portable_math(oracle):
    """build.rs:1079-1176: exp / tanh agree with libm to a few ulp."""
    xs = np.linspace(-20, 20, 801, dtype=np.float32)
    e = np.array([oracle.lib.rqo_exp(float(v)) for v in xs], np.float64)
    t = np.array([oracle.lib.rqo_tanh(float(v)) for v in xs], np.float64)
    assert np.allclose(e, np.exp(xs.astype(np.float64)), rtol=2e-6)  # fp32 argument reduction: error grows with |x|
    assert np.allclose(t, np.tanh(xs.astype(np.float64)), rtol=2e-7, atol=1e-30)


def test_moe_matches_dense_reference(oracle):
    """recipe.rs:23386-23459: routed experts in ascending order, silu(gate)*up, down scaled by the
    routing weight, plus a sigmoid-gated shared expert -- against float64 algebra on the dequantised banks."""
    experts, top, hidden, ffn, tokens = 6, 2, 256, 256, 3
    t = ol.Q4_K
    gate = oracle.quantize(t, oracle.normal(61, 1, experts * ffn * hidden, 0.05))
    up = oracle.quantize(t, oracle.normal(61, 2, experts * ffn * hidden, 0.05))
    down = oracle.quantize(t, oracle.normal(61, 3, experts * hidden * ffn, 0.05))
    sg = oracle.quantize(t, oracle.normal(61, 4, ffn * hidden, 0.05))
    su = oracle.quantize(t, oracle.normal(61, 5, ffn * hidden, 0.05))
    sd = oracle.quantize(t, oracle.normal(61, 6, hidden * ffn, 0.05))
    sw = oracle.normal(61, 7, hidden, 0.05)
    x = oracle.normal(61, 8, hidden * tokens, 1.0).reshape(hidden, tokens)
    routing = oracle.topk(oracle.normal(61, 9, experts * tokens, 1.0).reshape(experts, tokens), top, 0, True)
    y = oracle.moe_forward(t, gate, up, down, experts, top, hidden, ffn, x, routing, shared=(sg, su, sd, sw))
    G = oracle.dequantize(t, gate).astype(np.float64).reshape(experts, ffn, hidden)
    U = oracle.dequantize(t, up).astype(np.float64).reshape(experts, ffn, hidden)
    D = oracle.dequantize(t, down).astype(np.float64).reshape(experts, hidden, ffn)
    SG, SU, SD = (oracle.dequantize(t, a).astype(np.float64) for a in (sg, su, sd))
    SG, SU, SD = SG.reshape(ffn, hidden), SU.reshape(ffn, hidden), SD.reshape(hidden, ffn)
    silu = lambda z: z / (1.0 + np.exp(-z))
    ref = np.zeros((hidden, tokens))
    for p in range(tokens):
        xp = x[:, p].astype(np.float64)
        for e in range(experts):
            if routing[e, p] != 0:
                ref[:, p] += routing[e, p] * (D[e] @ (silu(G[e] @ xp) * (U[e] @ xp)))
        s = 1.0 / (1.0 + np.exp(-(sw.astype(np.float64) @ xp)))
        ref[:, p] += s * (SD @ (silu(SG @ xp) * (SU @ xp)))
    assert np.max(np.abs(y - ref)) <= 2e-5 * np.max(np.abs(ref))
