"""Generates the committed golden fixtures under tests/golden/.

Run from the repository root: ``python tests/golden/make_golden.py``.

1. suite_q8_0_table.npz -- the Q8_0 table the reference's own integration suite writes
   (.github/runtime/suite.rs:191-194): four rows, each d = 0x2400 (2^-6) with 32 equal codes
   32, 96, -80, 48, whose dequantised rows are the constants 0.5, 1.5, -1.25, 0.75.
2. bench_q4k_kat.npz -- the deterministic Q4_K blocks and the independent scalar
   Q4_K x Q8_1 check of evidence/2026-10-10-m60-p2p/bench.rs:177-228, restated here in
   integer / float64 NumPy: xorshift32 nibble bytes, hand scale bytes, input
   x_i = ((37 i + 13) mod 255) - 127, and the expected row sums. The reference computes those
   at run time and stores none, so this script is their record. The activation quantiser of
   that check (max/127, round half away, fp16-rounded step) is NOT the template's
   (amd-nv-cpu.ll:1381-1517); the fixture therefore also stores the dequantised activations
   q*d, which are exact in fp32, so that a FLOAT-mode matvec over them must reproduce the sums.
3. oracle_regression.npz -- seeded outputs of oracle/rq_oracle.c itself (blocks, dequantised
   values, activation records, matvec rows in every mode), so that an edit to the oracle that
   changes any byte shows up as a diff against the committed file.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))


def suite_table():
    rows = []
    for code in (32, 96, -80, 48):
        rows.append(np.concatenate([np.array([0x00, 0x24], np.uint8), np.full(32, code, np.int8).view(np.uint8)]))
    blocks = np.concatenate(rows)
    expected = np.repeat(np.array([0.5, 1.5, -1.25, 0.75], np.float32), 32).reshape(4, 32)
    np.savez(HERE / "suite_q8_0_table.npz", blocks=blocks, expected=expected)


def half_value(bits: int) -> float:
    return float(np.array([bits], np.uint16).view(np.float16)[0])


def bench_kat(rows: int = 16, seed: int = 0x12345678, scale_bits: int = 0x0400):
    w = np.zeros(rows * 16 * 144, np.uint8)
    state = seed
    for blk in range(rows * 16):
        b = w[blk * 144:(blk + 1) * 144]
        b[0], b[1] = scale_bits & 0xFF, scale_bits >> 8
        b[2], b[3] = scale_bits & 0xFF, scale_bits >> 8
        for i in range(4):
            b[4 + i] = 1 + ((state >> (i * 2)) % 3)
            b[8 + i] = 1 + ((state >> (i * 3)) % 3)
        for i in range(4):
            b[12 + i] = (1 + ((state >> (i * 2)) % 3)) | ((1 + ((state >> (i * 3)) % 3)) << 4)
        for q in range(16, 144):
            state ^= (state << 13) & 0xFFFFFFFF
            state ^= state >> 17
            state ^= (state << 5) & 0xFFFFFFFF
            b[q] = state & 0xFF
    x = np.array([((i * 37 + 13) % 255) - 127 for i in range(4096)], np.float32)
    q = np.zeros(4096, np.int64)
    d = np.zeros(128, np.float64)
    for b in range(128):
        blk = x[b * 32:(b + 1) * 32]
        mx = np.float32(np.max(np.abs(blk)))
        raw_d = np.float32(mx / np.float32(127.0))
        if mx == 0:
            continue
        d[b] = float(np.float32(raw_d).astype(np.float16))  # round-to-nearest-even onto the fp16 grid
        ratio = (blk / raw_d).astype(np.float32)
        q[b * 32:(b + 1) * 32] = np.where(ratio >= 0, np.floor(ratio + np.float32(0.5)), -np.floor(-ratio + np.float32(0.5))).astype(np.int64)
    expected = np.zeros(rows, np.float32)
    for row in range(rows):
        acc = 0.0
        for sb in range(16):
            b = w[(row * 16 + sb) * 144:(row * 16 + sb + 1) * 144].astype(np.int64)
            wd, wm = half_value(int(b[0] | (b[1] << 8))), half_value(int(b[2] | (b[3] << 8)))
            for sub in range(8):
                if sub < 4:
                    scale, mn = b[4 + sub] & 63, b[8 + sub] & 63
                else:
                    scale = (b[12 + sub - 4] & 15) | ((b[4 + sub - 4] >> 6) << 4)
                    mn = (b[12 + sub - 4] >> 4) | ((b[8 + sub - 4] >> 6) << 4)
                packed = b[16 + (sub // 2) * 32:16 + (sub // 2) * 32 + 32]
                weight = (packed & 15) if sub % 2 == 0 else (packed >> 4)
                act = q[sb * 256 + sub * 32:sb * 256 + sub * 32 + 32]
                dot, total = int(np.sum(weight * act)), int(np.sum(act))
                acc += (float(scale * dot) * wd - float(mn * total) * wm) * d[sb * 8 + sub]
        expected[row] = np.float32(acc)
    x_dequant = (q.astype(np.float64) * np.repeat(d, 32)).astype(np.float32)
    assert np.all(x_dequant.astype(np.float64) == q * np.repeat(d, 32))  # exact in fp32
    np.savez(HERE / "bench_q4k_kat.npz", blocks=w, x=x, x_dequant=x_dequant, q=q.astype(np.int32), d=d, expected=expected, rows=rows)


def oracle_regression():
    from tests import oracle_lib as ol

    o = ol.load()
    out = {}
    rows, cols = 6, 512
    for name, t in (("q4_0", ol.Q4_0), ("q8_0", ol.Q8_0), ("q4_k", ol.Q4_K), ("q6_k", ol.Q6_K)):
        w = o.normal(7, t, rows * cols, 0.02)
        x = o.normal(7, 100 + t, 2 * cols, 1.0).reshape(2, cols)
        blocks = o.quantize(t, w)
        out[f"{name}_blocks"] = blocks
        out[f"{name}_dequant_bits"] = o.dequantize(t, blocks).view(np.uint32)
        for mode, label in ((ol.FLOAT_RUN, "run"), (ol.FLOAT_EXACT, "exact")):
            out[f"{name}_y_{label}"] = o.matvec(t, blocks, rows, cols, x, mode).view(np.uint32)
        for step in (32, 256):
            out[f"{name}_y_int8_{step}"] = o.matvec(t, blocks, rows, cols, x, ol.INT8, step).view(np.uint32)
    x = o.normal(7, 999, 512, 1.0)
    out["act_records_32"] = o.activation_records(x, 32)
    out["act_records_256"] = o.activation_records(x, 256)
    scores = o.normal(7, 1000, 64 * 3, 1.0).reshape(64, 3)
    out["topk_softmax_renorm"] = o.topk(scores, 8, 0, True).view(np.uint32)
    out["topk_softmax_plain"] = o.topk(scores, 8, 0, False).view(np.uint32)
    out["topk_sigmoid_renorm"] = o.topk(scores, 8, 1, True).view(np.uint32)
    np.savez_compressed(HERE / "oracle_regression.npz", **out)


if __name__ == "__main__":
    suite_table()
    bench_kat()
    oracle_regression()
    print("written:", sorted(p.name for p in HERE.glob("*.npz")))
