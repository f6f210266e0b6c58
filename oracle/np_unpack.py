"""Independent NumPy restatement of the reference unpacking -- TEST INFRASTRUCTURE ONLY.

A second, vectorised statement of recipe.rs:3687-3958 (dequant_q45k, dequant_q6k, dequant_scalar,
dequant_q2k, dequant_q3k, dequant_q8k, dequant_iq4) evaluated as HostQuantOps does (recipe.rs:3973-4057): every product and the
final subtract in float64, the result rounded once to float32. It shares no code with
rq_oracle.c, so agreement between the two pins the layout reading of each. Only tests import it.
"""
from __future__ import annotations

import numpy as np

Q4_0, Q8_0, Q4_K, Q6_K = 2, 8, 12, 14
Q4_1, Q5_0, Q5_1, Q5_K, IQ4_NL = 3, 6, 7, 13, 20
Q8_1, Q2_K, Q3_K, Q8_K, IQ4_XS = 9, 10, 11, 15, 23
GEOMETRY = {Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210),
            Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24), Q5_K: (256, 176), IQ4_NL: (32, 18),
            Q8_1: (32, 36), Q2_K: (256, 84), Q3_K: (256, 110), Q8_K: (256, 292), IQ4_XS: (256, 136)}
IQ4_LEVELS = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.float64)  # recipe.rs:15211


def _fifth_bits(qh: np.ndarray) -> np.ndarray:
    """Four bytes per block -> 32 bits, value i = bit i % 8 of byte i // 8 (dequant_scalar, man 5)."""
    return np.unpackbits(qh, axis=1, bitorder="little").astype(np.int64)


def _half(raw: np.ndarray) -> np.ndarray:
    """Two little-endian bytes -> float64 value of the IEEE half."""
    return np.ascontiguousarray(raw).view("<f2").astype(np.float64)[..., 0]


def dequantize(ggml_type: int, blocks: np.ndarray) -> np.ndarray:
    values, stride = GEOMETRY[ggml_type]
    b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, stride)
    n = b.shape[0]
    if ggml_type == Q8_0:
        d = _half(b[:, 0:2])
        q = b[:, 2:34].view(np.int8).astype(np.float64)
        out = q * d[:, None]
    elif ggml_type == Q4_0:
        d = _half(b[:, 0:2])
        qs = b[:, 2:18]
        q = np.concatenate([qs & 15, qs >> 4], axis=1).astype(np.float64) - 8.0
        out = q * d[:, None]
    elif ggml_type == Q4_K:
        d, dmin = _half(b[:, 0:2]), _half(b[:, 2:4])
        s = b[:, 4:16].astype(np.int64)
        sc = np.empty((n, 8), np.int64)
        mn = np.empty((n, 8), np.int64)
        sc[:, :4] = s[:, 0:4] & 63
        mn[:, :4] = s[:, 4:8] & 63
        sc[:, 4:] = (s[:, 8:12] & 15) | ((s[:, 0:4] >> 6) << 4)
        mn[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
        qs = b[:, 16:144].reshape(n, 4, 32)
        q = np.stack([qs & 15, qs >> 4], axis=2).reshape(n, 8, 32).astype(np.float64)  # sub-block 2p low, 2p+1 high
        step = d[:, None] * sc
        base = dmin[:, None] * mn
        out = (step[:, :, None] * q - base[:, :, None]).reshape(n, 256)
    elif ggml_type == Q6_K:
        ql = b[:, 0:128].reshape(n, 2, 2, 32)          # [chunk][g & 1][w]
        qh = b[:, 128:192].reshape(n, 2, 32)           # [chunk][w]
        sc = b[:, 192:208].view(np.int8).astype(np.float64).reshape(n, 2, 4, 2)  # [chunk][g][w // 16]
        d = _half(b[:, 208:210])
        out = np.empty((n, 2, 4, 32), np.float64)
        for g in range(4):
            lo = (ql[:, :, g & 1, :] >> (4 * (g // 2))) & 15
            hi = (qh >> (2 * g)) & 3
            code = (lo | (hi << 4)).astype(np.float64) - 32.0
            scale = np.repeat(sc[:, :, g, :], 16, axis=2)
            out[:, :, g, :] = (d[:, None, None] * scale) * code
        out = out.reshape(n, 256)
    elif ggml_type == Q4_1:
        d, m = _half(b[:, 0:2]), _half(b[:, 2:4])
        qs = b[:, 4:20]
        q = np.concatenate([qs & 15, qs >> 4], axis=1).astype(np.float64)
        out = q * d[:, None] + m[:, None]
    elif ggml_type in (Q5_0, Q5_1):
        header = 4 if ggml_type == Q5_1 else 2
        d = _half(b[:, 0:2])
        qs = b[:, header + 4:header + 20]
        low = np.concatenate([qs & 15, qs >> 4], axis=1).astype(np.int64)
        code = low | (_fifth_bits(b[:, header:header + 4]) << 4)
        if ggml_type == Q5_0:
            out = (code - 16).astype(np.float64) * d[:, None]
        else:
            out = code.astype(np.float64) * d[:, None] + _half(b[:, 2:4])[:, None]
    elif ggml_type == Q5_K:
        d, dmin = _half(b[:, 0:2]), _half(b[:, 2:4])
        s = b[:, 4:16].astype(np.int64)
        sc = np.empty((n, 8), np.int64)
        mn = np.empty((n, 8), np.int64)
        sc[:, :4] = s[:, 0:4] & 63
        mn[:, :4] = s[:, 4:8] & 63
        sc[:, 4:] = (s[:, 8:12] & 15) | ((s[:, 0:4] >> 6) << 4)
        mn[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
        qh = b[:, 16:48].astype(np.int64)                     # bit `sub` of byte w is the fifth bit of value w of sub-block `sub`
        qs = b[:, 48:176].reshape(n, 4, 32)
        low = np.stack([qs & 15, qs >> 4], axis=2).reshape(n, 8, 32).astype(np.int64)
        high = np.stack([(qh >> sub) & 1 for sub in range(8)], axis=1)
        q = (low | (high << 4)).astype(np.float64)
        out = ((d[:, None] * sc)[:, :, None] * q - (dmin[:, None] * mn)[:, :, None]).reshape(n, 256)
    elif ggml_type == IQ4_NL:
        d = _half(b[:, 0:2])
        qs = b[:, 2:18]
        code = np.concatenate([qs & 15, qs >> 4], axis=1)
        out = (d[:, None] * 1.0) * IQ4_LEVELS[code]
    elif ggml_type == Q8_1:
        out = b[:, 4:36].view(np.int8).astype(np.float64) * _half(b[:, 0:2])[:, None]
    elif ggml_type == Q2_K:
        meta = b[:, 0:16].astype(np.int64)                         # group g of sixteen values: scale | minimum << 4
        qs = b[:, 16:80].reshape(n, 2, 32).astype(np.int64)        # [section][byte]
        d, dmin = _half(b[:, 80:82]), _half(b[:, 82:84])
        out = np.empty((n, 16, 16), np.float64)
        for g in range(16):
            section, pair, half = g // 8, (g % 8) // 2, g % 2
            code = (qs[:, section, 16 * half:16 * half + 16] >> (2 * pair)) & 3
            out[:, g, :] = (d * (meta[:, g] & 15))[:, None] * code - (dmin * (meta[:, g] >> 4))[:, None]
        out = out.reshape(n, 256)
    elif ggml_type == Q3_K:
        hmask = b[:, 0:32].astype(np.int64)
        qs = b[:, 32:96].reshape(n, 2, 32).astype(np.int64)
        sc = b[:, 96:108].astype(np.int64)
        d = _half(b[:, 108:110])
        out = np.empty((n, 8, 32), np.float64)                     # [i // 32][i % 32]
        for part in range(8):
            section, pair = part // 4, part % 4
            code = (qs[:, section, :] >> (2 * pair)) & 3
            code = code - np.where((hmask >> part) & 1, 0, 4)
            for half in range(2):
                g = 2 * part + half                                 # group of sixteen values
                low = (sc[:, g if g < 8 else g - 8] >> (0 if g < 8 else 4)) & 15
                high = (sc[:, 8 + g % 4] >> (2 * (g // 4))) & 3
                scale = (low | (high << 4)) - 32
                out[:, part, 16 * half:16 * half + 16] = (d * scale)[:, None] * code[:, 16 * half:16 * half + 16]
        out = out.reshape(n, 256)
    elif ggml_type == Q8_K:
        d = np.ascontiguousarray(b[:, 0:4]).view("<f4").astype(np.float32)[:, 0]
        q = b[:, 4:260].view(np.int8).astype(np.float32)
        return (d[:, None] * q).astype(np.float32).reshape(-1)     # an fp32 step times an int8 code: one fp32 rounding, not exact in f64 first
    elif ggml_type == IQ4_XS:
        d = _half(b[:, 0:2])
        hi = np.ascontiguousarray(b[:, 2:4]).view("<u2").astype(np.int64)[:, 0]
        lo = b[:, 4:8].astype(np.int64)
        qs = b[:, 8:136].reshape(n, 8, 16)
        out = np.empty((n, 8, 32), np.float64)
        for blk in range(8):
            exponent = (((lo[:, blk // 2] >> (4 * (blk % 2))) & 15) | (((hi >> (2 * blk)) & 3) << 4)) - 32
            code = np.concatenate([qs[:, blk, :] & 15, qs[:, blk, :] >> 4], axis=1)
            out[:, blk, :] = (d * exponent)[:, None] * IQ4_LEVELS[code]
        out = out.reshape(n, 256)
    else:
        raise ValueError(f"type {ggml_type}")
    return out.astype(np.float32).reshape(-1)
