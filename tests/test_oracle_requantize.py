"""The oracle's load-time Q8_0 re-encode (emit_requantize, recipe.rs:8016-8127) against a second,
independent NumPy restatement and hand-made blocks that separate it from the host encoder. No GPU."""
import numpy as np
import pytest

from tests import oracle_lib as ol


def np_requant_q8_0(values: np.ndarray) -> np.ndarray:
    """NumPy restatement, vectorised over blocks; every step is one fp32 operation."""
    v = np.ascontiguousarray(values, np.float32).reshape(-1, 32)
    mag = np.abs(v)
    first = np.argmax(mag, axis=1)  # argmax returns the FIRST of equal maxima, as the running scan keeps it
    ext = mag[np.arange(v.shape[0]), first]
    scale = (ext / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inverse = np.where(scale == 0, np.float32(0), (np.float32(1.0) / scale).astype(np.float32)).astype(np.float32)
    q = (v * inverse[:, None]).astype(np.float32)
    r = np.where(q >= 0, (q + np.float32(0.5)).astype(np.float32), (q + np.float32(-0.5)).astype(np.float32))
    codes = np.clip(np.trunc(r).astype(np.int32), -128, 127).astype(np.int8)
    out = np.empty((v.shape[0], 34), np.uint8)
    out[:, :2] = scale.astype(np.float16).view(np.uint8).reshape(-1, 2)  # IEEE round to nearest even
    out[:, 2:] = codes.view(np.uint8)
    return out.reshape(-1)


@pytest.mark.parametrize("t", [ol.Q6_K, ol.Q4_0, ol.Q4_K, ol.Q8_0])
def test_two_restatements_agree(oracle, t):
    blocks = oracle.quantize(t, oracle.normal(51, t, 64 * 1024, 0.02))
    got = oracle.requantize_q8_0(t, blocks)
    want = np_requant_q8_0(oracle.dequantize(t, blocks))
    assert np.array_equal(got, want)
    # the re-encode is within half a step of the decoded values
    back = oracle.dequantize(ol.Q8_0, got).reshape(-1, 32)
    src = oracle.dequantize(t, blocks).reshape(-1, 32)
    step = np.abs(src).max(axis=1, keepdims=True) / 127.0
    assert np.all(np.abs(back - src) <= 0.51 * step + 1e-3 * np.abs(src).max())


def test_half_away_by_truncation_and_first_extreme(oracle):
    """Blocks written as Q8_0 with d = 1 decode to their codes, so the re-encoder's input is known exactly."""
    def q8(codes, d=1.0):
        b = np.zeros(34, np.uint8)
        b[:2] = np.array([d], np.float16).view(np.uint8)
        b[2:] = np.asarray(codes, np.int8).view(np.uint8)
        return b

    # extreme 127 -> scale 1, inverse 1: codes come back unchanged, sign and all
    codes = np.array([127, -127, 5, -5, 0, 1, -1, 64] + [0] * 24)
    out = oracle.requantize_q8_0(ol.Q8_0, q8(codes))
    assert np.array_equal(out[2:].view(np.int8), codes.astype(np.int8)) and out[:2].view(np.float16)[0] == 1.0
    # equal magnitudes of both signs: the first one is the extreme; the scale is its magnitude either way
    codes = np.array([-100, 100] + [50] * 30)
    out = oracle.requantize_q8_0(ol.Q8_0, q8(codes))
    assert np.array_equal(out[2:4].view(np.int8), np.array([-127, 127], np.int8))
    # a value whose q is just under .5: q + 0.5 rounds UP to the next integer in fp32 and truncation keeps it,
    # where f32::round (the host encoder) would give the integer below
    v = np.float32(0.49999997)
    blocks = q8([127] + [0] * 31)
    vals = np.zeros(32, np.float32); vals[0] = 127.0; vals[1] = v
    assert np.float32(v + np.float32(0.5)) == np.float32(1.0) and np.round(v) == 0.0
    got = np_requant_q8_0(vals)
    assert got[2:].view(np.int8)[1] == 1
    # all zeros: scale 0, inverse 0, codes 0
    out = oracle.requantize_q8_0(ol.Q8_0, q8([0] * 32, d=0.0))
    assert not out.any()
    assert blocks.size == 34


def test_int8_blocks_rule(oracle):
    """finish_int_sums (recipe.rs:22345-22369): Q8_0 and Q4_K are kept, Q6_K and Q4_0 become Q8_0."""
    for t in (ol.Q8_0, ol.Q4_K):
        b = oracle.quantize(t, oracle.normal(52, t, 1024, 0.02))
        assert oracle.int8_blocks(t, b)[0] == t
    for t in (ol.Q6_K, ol.Q4_0):
        b = oracle.quantize(t, oracle.normal(52, t, 1024, 0.02))
        t8, b8 = oracle.int8_blocks(t, b)
        assert t8 == ol.Q8_0 and b8.size == 1024 // 32 * 34
