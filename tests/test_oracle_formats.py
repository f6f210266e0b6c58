"""The other stored formats (Q4_1, Q5_0, Q5_1, Q5_K, IQ4_NL, Q8_1, Q2_K, Q3_K, Q8_K, IQ4_XS): the C oracle and the independent NumPy
restatement read every layout the same way, hand-built blocks decode to the values their definition
gives, and the entry points that need an encoder or an int8 slice helper refuse them."""
import numpy as np
import pytest

from oracle import np_unpack
from tests import oracle_lib as ol

TYPES = [ol.Q4_1, ol.Q5_0, ol.Q5_1, ol.Q5_K, ol.IQ4_NL, ol.Q8_1, ol.Q2_K, ol.Q3_K, ol.Q8_K, ol.IQ4_XS]


@pytest.mark.parametrize("t", TYPES)
def test_two_restatements_agree_bit_for_bit(t):
    oracle = ol.load()
    rng = np.random.default_rng(100 + t)
    values, stride = ol.GEOMETRY[t]
    blocks = ol.random_blocks(t, 300, rng)
    a = oracle.dequantize(t, blocks)
    b = np_unpack.dequantize(t, blocks)
    assert a.shape == (300 * values,)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    # arbitrary bytes too (any fp16 header that is finite)
    raw = ol.arbitrary_blocks(t, 200, rng)  # any code and scale pattern, finite headers
    a = oracle.dequantize(t, raw)
    b = np_unpack.dequantize(t, raw)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def _half_bytes(v):
    return list(np.asarray([v], np.float16).view(np.uint8))


def test_hand_built_blocks():
    oracle = ol.load()
    # Q4_1: d = 0.5, m = -1; byte k holds value k (low nibble) and value 16 + k (high nibble)
    blk = _half_bytes(0.5) + _half_bytes(-1.0) + [(k & 15) | (((15 - k) & 15) << 4) for k in range(16)]
    out = oracle.dequantize(ol.Q4_1, np.array(blk, np.uint8))
    assert np.array_equal(out, np.array([0.5 * k - 1 for k in range(16)] + [0.5 * (15 - k) - 1 for k in range(16)], np.float32))
    # Q5_0: d = 0.25; fifth bits 0x0000FFFF: values 0..15 carry it
    blk = _half_bytes(0.25) + [0xFF, 0xFF, 0, 0] + [3 | (5 << 4)] * 16
    out = oracle.dequantize(ol.Q5_0, np.array(blk, np.uint8))
    assert np.array_equal(out, np.array([0.25 * (3 + 16 - 16)] * 16 + [0.25 * (5 - 16)] * 16, np.float32))
    # Q5_1: d = 2, m = 1; only value 9 carries the fifth bit (bit 1 of the second byte)
    blk = _half_bytes(2.0) + _half_bytes(1.0) + [0, 2, 0, 0] + [1] * 16
    out = oracle.dequantize(ol.Q5_1, np.array(blk, np.uint8))
    want = np.array([2.0 * 1 + 1] * 16 + [1.0] * 16, np.float32)
    want[9] = 2.0 * 17 + 1
    assert np.array_equal(out, want)
    # IQ4_NL: d = 1: the level table itself, values 0..15 from the low nibbles of bytes 0..15
    blk = _half_bytes(1.0) + [k | ((15 - k) << 4) for k in range(16)]
    out = oracle.dequantize(ol.IQ4_NL, np.array(blk, np.uint8))
    levels = [-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113]
    assert np.array_equal(out, np.array(levels + levels[::-1], np.float32))
    # Q5_K: d = 1, dmin = 0, every scale 1 (first four sub-blocks: low six bits), nibbles 2, fifth bit of value 0 in sub-block 3
    scales = [1, 1, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1]
    qh = [0] * 32
    qh[0] = 1 << 3
    blk = _half_bytes(1.0) + _half_bytes(0.0) + scales + qh + [2 | (2 << 4)] * 128
    out = oracle.dequantize(ol.Q5_K, np.array(blk, np.uint8))
    want = np.full(256, 2.0, np.float32)
    want[3 * 32] = 18.0
    assert np.array_equal(out, want)


def test_hand_built_blocks_of_the_k_and_iq_formats():
    oracle = ol.load()
    # Q2_K: d = 1, dmin = 0.5; group g has scale g and minimum 15 - g; every code 2 -> value 2 g - 0.5 (15 - g)
    blk = [g | ((15 - g) << 4) for g in range(16)] + [0xAA] * 64 + _half_bytes(1.0) + _half_bytes(0.5)
    out = oracle.dequantize(ol.Q2_K, np.array(blk, np.uint8)).reshape(16, 16)
    assert np.array_equal(out, np.repeat(np.array([2.0 * g - 0.5 * (15 - g) for g in range(16)], np.float32)[:, None], 16, axis=1))
    # Q3_K: d = 1, every scale code 33 (low four bits 1, high two bits 2 -> 33 - 32 = 1), codes 3, mask set only for values of part 0
    blk = [1] * 32 + [0xFF] * 64 + [0x11] * 8 + [0xAA] * 4 + _half_bytes(1.0)
    out = oracle.dequantize(ol.Q3_K, np.array(blk, np.uint8))
    want = np.full(256, -1.0, np.float32)   # 3 - 4
    want[:32] = 3.0
    assert np.array_equal(out, want)
    # Q8_K: an fp32 step of 0.25 and codes -128 .. 127
    blk = list(np.array([0.25], np.float32).view(np.uint8)) + list(np.arange(-128, 128, dtype=np.int8).view(np.uint8)) + [0] * 32
    out = oracle.dequantize(ol.Q8_K, np.array(blk, np.uint8))
    assert np.array_equal(out, 0.25 * np.arange(-128, 128, dtype=np.float32))
    # Q8_1: d = 0.5, the stored sum is not part of a value
    blk = _half_bytes(0.5) + _half_bytes(123.0) + list(np.arange(-16, 16, dtype=np.int8).view(np.uint8))
    out = oracle.dequantize(ol.Q8_1, np.array(blk, np.uint8))
    assert np.array_equal(out, 0.5 * np.arange(-16, 16, dtype=np.float32))
    # IQ4_XS: d = 1; block b of 32 values has exponent code 32 + b (low bits b, high bits 2) -> exponent b; nibble 8 -> level 1
    hi = sum(2 << (2 * b) for b in range(8))
    blk = _half_bytes(1.0) + [hi & 0xFF, hi >> 8] + [(2 * k) | ((2 * k + 1) << 4) for k in range(4)] + [0x88] * 128
    out = oracle.dequantize(ol.IQ4_XS, np.array(blk, np.uint8)).reshape(8, 32)
    assert np.array_equal(out, np.repeat(np.arange(8, dtype=np.float32)[:, None], 32, axis=1))


@pytest.mark.parametrize("t", TYPES)
def test_run_decoder_product_and_reencode(t):
    oracle = ol.load()
    rng = np.random.default_rng(7 + t)
    values, _ = ol.GEOMETRY[t]
    rows, cols = 24, 1024
    blocks = ol.random_blocks(t, rows * cols // values, rng)
    w = oracle.dequantize(t, blocks).reshape(rows, cols).astype(np.float64)
    x = rng.normal(size=(2, cols)).astype(np.float32)  # token-major
    y = oracle.matvec(t, blocks, rows, cols, x, ol.FLOAT_RUN)
    exact = x.astype(np.float64) @ w.T
    assert np.max(np.abs(y - exact)) <= 1e-5 * np.max(np.abs(exact))
    # the other two activation handlings need helpers these formats do not have
    if t != ol.Q4_1:  # Q4_1 is `.int(4)`'s storage and has an int8 slice helper (block32 slice kind 3)
        with pytest.raises(Exception):
            oracle.matvec(t, blocks, rows, cols, x, ol.INT8)
    with pytest.raises(Exception):
        oracle.matvec(t, blocks, rows, cols, x, ol.FLOAT_EXACT)
    with pytest.raises(Exception):
        oracle.quantize(t, np.zeros(values, np.float32))
    # `.int(8)`: decoded, then encoded as Q8_0 by the load kernel's encoder; one fp16 step per 32 values: half a step of rounding plus the step's own fp16 rounding (127 * 2^-11 of a step)
    q8 = oracle.requantize_q8_0(t, blocks)
    back = oracle.dequantize(ol.Q8_0, q8).reshape(rows, cols)
    step = np.abs(w).reshape(rows, cols // 32, 32).max(axis=2) / 127
    assert np.all(np.abs(back - w).reshape(rows, cols // 32, 32) <= 0.57 * step[:, :, None] + 127 * 2.0 ** -25)  # the last term: a step that is a subnormal fp16


def test_int4_storage_is_q4_1():
    """`.int(4)` (recipe.rs:22348): the load kernel's Q4_1 encoder on hand-checked blocks, its error bound on random
    tensors, and the int dot over Q4_1 blocks against the exact product of the decoded weights and the decoded records."""
    oracle = ol.load()
    # values 0, 1, .., 15 twice: minimum 0, maximum 15, step exactly 1, codes = the values
    v = np.array(list(range(16)) * 2, np.float32)
    q8 = oracle.quantize(ol.Q8_0, v / 8)            # an exactly representable source: codes 0..15 * 8.47 -> decode gives k * d
    src = oracle.dequantize(ol.Q8_0, q8)
    q41 = oracle.requantize_q4_1(ol.Q8_0, q8)
    assert q41.size == 20
    back = oracle.dequantize(ol.Q4_1, q41)
    step = (src.max() - src.min()) / 15
    assert np.all(np.abs(back - src) <= 0.51 * step + 2e-3 * np.abs(src).max())  # half a step, plus fp16 rounding of step and minimum
    codes = np.concatenate([q41[4:] & 15, q41[4:] >> 4])
    assert codes.min() == 0 and codes.max() == 15 and np.all(np.diff(codes[:16]) >= 0)
    # a constant block: zero step, every code 0, the minimum carries the value
    const = oracle.requantize_q4_1(ol.Q8_0, oracle.quantize(ol.Q8_0, np.full(32, 0.5, np.float32)))
    assert np.all(const[4:] == 0) and const[0] == 0 and const[1] == 0
    assert np.allclose(oracle.dequantize(ol.Q4_1, const), 0.5, rtol=1e-3)
    # random tensors in every source format
    rng = np.random.default_rng(5)
    for t in (ol.Q4_K, ol.Q6_K, ol.Q8_0, ol.Q4_0, ol.Q5_K, ol.IQ4_NL):
        rows, cols = 16, 1024
        blocks = oracle.quantize(t, rng.normal(0, 0.02, rows * cols).astype(np.float32)) if t in (ol.Q4_K, ol.Q6_K, ol.Q8_0, ol.Q4_0) else ol.random_blocks(t, rows * cols // ol.GEOMETRY[t][0], rng)
        w = oracle.dequantize(t, blocks).astype(np.float64)
        t4, b4 = oracle.int4_blocks(t, blocks)
        assert t4 == ol.Q4_1 and b4.size == rows * cols // 32 * 20
        w4 = oracle.dequantize(ol.Q4_1, b4).astype(np.float64)
        g = w.reshape(-1, 32)
        step = (g.max(axis=1) - g.min(axis=1)) / 15
        bound = 0.51 * step + 2.0 ** -10 * (np.abs(g).max(axis=1) + 15 * step) + 2.0 ** -23
        assert np.all(np.abs(w4.reshape(-1, 32) - g) <= bound[:, None])
        # the int dot: q8_d * (d * dot + m * sum), slice by slice
        x = rng.normal(size=cols).astype(np.float32)
        y = oracle.matvec(ol.Q4_1, b4, rows, cols, x, ol.INT8, 32)
        recs = oracle.activation_records(x, 32)
        xq = (recs[:, 4:].view(np.int8).astype(np.float64) * recs[:, :4].copy().view(np.float32).astype(np.float64)).reshape(-1)
        exact = w4.reshape(rows, cols) @ xq
        assert np.max(np.abs(y - exact)) <= 2e-5 * np.max(np.abs(exact))
    assert oracle.int4_blocks(ol.Q4_1, np.zeros(20, np.uint8))[0] == ol.Q4_1
