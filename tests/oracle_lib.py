"""ctypes access to the CPU oracle for the tests (never imported by the product)."""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"
LIB_PATH = ORACLE_DIR / "librq_oracle.so"

Q4_0, Q8_0, Q4_K, Q6_K = 2, 8, 12, 14
Q4_1, Q5_0, Q5_1, Q5_K, IQ4_NL = 3, 6, 7, 13, 20   # decoded and run-decoder dotted only; no encoder, no int8 slice helper
Q8_1, Q2_K, Q3_K, Q8_K, IQ4_XS = 9, 10, 11, 15, 23
STORED_ONLY = (Q4_1, Q5_0, Q5_1, Q5_K, IQ4_NL, Q8_1, Q2_K, Q3_K, Q8_K, IQ4_XS)
FLOAT_RUN, FLOAT_EXACT, INT8 = 0, 1, 2
GEOMETRY = {Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210),
            Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24), Q5_K: (256, 176), IQ4_NL: (32, 18),
            Q8_1: (32, 36), Q2_K: (256, 84), Q3_K: (256, 110), Q8_K: (256, 292), IQ4_XS: (256, 136)}


# where a block's floating-point header fields sit: (byte offset, bytes)
HEADERS = {Q4_0: [(0, 2)], Q8_0: [(0, 2)], Q4_K: [(0, 2), (2, 2)], Q6_K: [(208, 2)], Q4_1: [(0, 2), (2, 2)], Q5_0: [(0, 2)], Q5_1: [(0, 2), (2, 2)],
           Q5_K: [(0, 2), (2, 2)], IQ4_NL: [(0, 2)], Q8_1: [(0, 2), (2, 2)], Q2_K: [(80, 2), (82, 2)], Q3_K: [(108, 2)], Q8_K: [(0, 4)], IQ4_XS: [(0, 2)]}


def arbitrary_blocks(t: int, count: int, rng: np.random.Generator) -> np.ndarray:
    """`count` blocks of arbitrary bytes whose header fields are finite and below 2 in magnitude (the top exponent bit cleared)."""
    _, stride = GEOMETRY[t]
    raw = rng.integers(0, 256, size=(count, stride), dtype=np.uint8)
    for at, width in HEADERS[t]:
        raw[:, at + width - 1] &= 0x3F
    return raw.reshape(-1)


def random_blocks(t: int, count: int, rng: np.random.Generator, scale: float = 0.02) -> np.ndarray:
    """`count` format-valid blocks of type t with arbitrary codes and sane fp16 headers (finite, of a
    weight's magnitude): test data for formats that have no encoder here."""
    values, stride = GEOMETRY[t]
    b = rng.integers(0, 256, size=(count, stride), dtype=np.uint8)
    def put_half(col, v):
        b[:, col:col + 2] = np.asarray(v, np.float16).reshape(-1, 1).view(np.uint8)
    mag = np.abs(rng.normal(0, scale, count)) + 1e-2  # large enough that a Q8_0 step of it is a normal fp16
    if t in (Q4_1, Q5_1):
        put_half(0, mag / (15 if t == Q4_1 else 31)); put_half(2, -mag / 2)
    elif t in (Q5_0, Q4_0):
        put_half(0, mag / 16)
    elif t == Q8_0:
        put_half(0, mag / 127)
    elif t == IQ4_NL:
        put_half(0, mag / 127)
    elif t in (Q5_K, Q4_K):
        put_half(0, mag / (63 * (31 if t == Q5_K else 15))); put_half(2, mag / 63 / 2)
    elif t == Q6_K:
        put_half(208, mag / (127 * 32))
    elif t == Q8_1:
        put_half(0, mag / 127); put_half(2, mag)
    elif t == Q2_K:
        put_half(80, mag / (15 * 3)); put_half(82, mag / 15 / 2)
    elif t == Q3_K:
        put_half(108, mag / (32 * 4))
    elif t == Q8_K:
        b[:, 0:4] = (mag / 127).astype(np.float32).reshape(-1, 1).view(np.uint8)
    elif t == IQ4_XS:
        put_half(0, mag / (32 * 127))
    return b.reshape(-1)
THREADS = max(1, os.cpu_count() or 1)


def build() -> Path:
    src = [ORACLE_DIR / "rq_oracle.c", ORACLE_DIR / "rq_oracle.h"]
    if not LIB_PATH.exists() or any(s.stat().st_mtime > LIB_PATH.stat().st_mtime for s in src):
        subprocess.run(["make", "-C", str(ORACLE_DIR), "-s"], check=True)
    return LIB_PATH


class Oracle:
    def __init__(self, lib):
        self.lib = lib
        p, i32, i64 = C.c_void_p, C.c_int, C.c_int64
        lib.rqo_fp16.restype = C.c_uint16
        lib.rqo_fp16.argtypes = [C.c_float]
        lib.rqo_unfp16.restype = C.c_float
        lib.rqo_unfp16.argtypes = [C.c_uint16]
        lib.rqo_qround.restype = C.c_float
        lib.rqo_qround.argtypes = [C.c_float]
        lib.rqo_dequantize.argtypes = [i32, p, i64, p, i32]
        lib.rqo_quantize.argtypes = [i32, p, i64, p, i32]
        lib.rqo_requantize_q8_0.argtypes = [i32, p, i64, p, i32]
        lib.rqo_requantize_q4_1.argtypes = [i32, p, i64, p, i32]
        lib.rqo_quantize_activations.argtypes = [p, i64, i64, i32, p]
        lib.rqo_matvec.argtypes = [i32, p, i64, i64, p, i64, i32, p, i64, i32, i32, i32]
        for name in ("rqo_exp", "rqo_tanh", "rqo_sigmoid", "rqo_silu"):
            getattr(lib, name).restype = C.c_float
            getattr(lib, name).argtypes = [C.c_float]
        lib.rqo_topk.argtypes = [p, i32, i32, i32, i32, i32, p, p]
        lib.rqo_moe_forward.argtypes = [i32, p, p, p, i32, i32, i32, i32, p, p, i32, p, p, p, p, p, i32]
        lib.rqo_moe_forward_ex.argtypes = [i32, p, p, p, i32, i32, i32, i32, p, p, i32, C.c_float, i32, i32, p, p, p, p, p, i32]
        lib.rqo_rmsnorm.argtypes = [p, i64, i64, p, C.c_float, p, i64]
        lib.rqo_rmsnorm.restype = None
        lib.rqo_softcap.argtypes = [p, i64, C.c_double, p]
        lib.rqo_softcap.restype = None
        lib.rqo_glu.argtypes = [p, p, i64, p]
        lib.rqo_glu.restype = None
        lib.rqo_normal.argtypes = [C.c_uint64, C.c_uint64, i64, i64, C.c_double, p]
        lib.rqo_normal.restype = None

    # ---- formats ----
    def quantize(self, t: int, values: np.ndarray) -> np.ndarray:
        v = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
        per, stride = GEOMETRY[t]
        blocks = (v.size + per - 1) // per
        out = np.empty(blocks * stride, dtype=np.uint8)
        assert self.lib.rqo_quantize(t, v.ctypes.data, v.size, out.ctypes.data, THREADS) == 0
        return out

    def dequantize(self, t: int, blocks: np.ndarray) -> np.ndarray:
        b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
        per, stride = GEOMETRY[t]
        count = b.size // stride * per
        out = np.empty(count, dtype=np.float32)
        assert self.lib.rqo_dequantize(t, b.ctypes.data, count, out.ctypes.data, THREADS) == 0
        return out

    def requantize_q8_0(self, t: int, blocks: np.ndarray) -> np.ndarray:
        """The load kernel's Q8_0 re-encode of a tensor stored as type t (what `.int(8)` dots for Q6_K / Q4_0)."""
        b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
        per, stride = GEOMETRY[t]
        count = b.size // stride * per
        out = np.empty(count // 32 * 34, dtype=np.uint8)
        assert self.lib.rqo_requantize_q8_0(t, b.ctypes.data, count, out.ctypes.data, THREADS) == 0
        return out

    def requantize_q4_1(self, t: int, blocks: np.ndarray) -> np.ndarray:
        """The load-time re-encode of `.int(4)`: any stored format -> Q4_1 blocks."""
        b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
        values, stride = GEOMETRY[t]
        count = b.size // stride * values
        out = np.empty((count + 31) // 32 * 20, dtype=np.uint8)
        assert self.lib.rqo_requantize_q4_1(t, b.ctypes.data, count, out.ctypes.data, THREADS) == 0
        return out

    def int4_blocks(self, t: int, blocks: np.ndarray):
        """(type, blocks) that recipe's `.int(4)` dots: kept for Q4_1, re-encoded to Q4_1 otherwise."""
        return (t, blocks) if t == Q4_1 else (Q4_1, self.requantize_q4_1(t, blocks))

    def int8_blocks(self, t: int, blocks: np.ndarray):
        """(type, blocks) that recipe's `.int(8)` dots for a lone tensor: kept for Q8_0 / Q4_K, re-encoded to Q8_0 otherwise."""
        return (t, blocks) if t in (Q8_0, Q4_K) else (Q8_0, self.requantize_q8_0(t, blocks))

    def activation_records(self, x: np.ndarray, step: int) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty((x.size // 32, 36), dtype=np.uint8)
        assert self.lib.rqo_quantize_activations(x.ctypes.data, 1, x.size, step, out.ctypes.data) == 0
        return out

    def matvec(self, t: int, blocks: np.ndarray, rows: int, cols: int, x: np.ndarray, mode: int, step: int = 32, threads: int | None = None) -> np.ndarray:
        """x: [cols] or [tokens, cols] (token-major) -> y [rows] or [tokens, rows]."""
        b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
        x = np.ascontiguousarray(x, dtype=np.float32)
        single = x.ndim == 1
        x2 = x[None, :] if single else x
        tokens = x2.shape[0]
        y = np.empty((tokens, rows), dtype=np.float32)
        # token-major planes: element strides x[k*1 + t*cols] -> the oracle takes x + t and a k stride,
        # so hand it the channel-major transpose
        xc = np.ascontiguousarray(x2.T)  # [cols][tokens]
        yc = np.empty((rows, tokens), dtype=np.float32)
        rc = self.lib.rqo_matvec(t, b.ctypes.data, rows, cols, xc.ctypes.data, tokens, tokens, yc.ctypes.data, tokens, mode, step, threads or THREADS)
        assert rc == 0, rc
        y[:] = yc.T
        return y[0] if single else y

    def topk(self, scores: np.ndarray, top: int, scoring: int = 0, renormalize: bool = True, bias: np.ndarray | None = None) -> np.ndarray:
        """scores [experts, tokens] -> weights [experts, tokens]."""
        s = np.ascontiguousarray(scores, dtype=np.float32)
        experts, tokens = s.shape
        w = np.empty_like(s)
        bp = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32).ctypes.data
        assert self.lib.rqo_topk(s.ctypes.data, experts, tokens, top, scoring, int(renormalize), bp, w.ctypes.data) == 0
        return w

    def moe_forward(self, t, gate, up, down, experts, top, hidden, ffn, x, routing, shared=None, threads=None) -> np.ndarray:
        """x [hidden, tokens], routing [experts, tokens]; shared = (gate, up, down, gate_vector) or None."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        routing = np.ascontiguousarray(routing, dtype=np.float32)
        tokens = x.shape[1]
        y = np.zeros((hidden, tokens), dtype=np.float32)
        g, u, d = (np.ascontiguousarray(a, dtype=np.uint8) for a in (gate, up, down))
        if shared is None:
            sg = su = sd = sw = None
            ptrs = (None, None, None, None)
        else:
            sg, su, sd = (np.ascontiguousarray(a, dtype=np.uint8) for a in shared[:3])
            sw = np.ascontiguousarray(shared[3], dtype=np.float32)
            ptrs = (sg.ctypes.data, su.ctypes.data, sd.ctypes.data, sw.ctypes.data)
        rc = self.lib.rqo_moe_forward(t, g.ctypes.data, u.ctypes.data, d.ctypes.data, experts, top, hidden, ffn,
                                      x.ctypes.data, routing.ctypes.data, tokens, *ptrs, y.ctypes.data, threads or THREADS)
        assert rc == 0, rc
        return y

    def moe_forward_ex(self, t, gate, up, down, experts, top, hidden, ffn, x, routing, routed_scale=1.0, shared_kind=0, shared_count=1, shared=None, threads=None):
        """gguf_moe with a routed scale and an ungated (1) / gated (2) shared expert of shared_count * ffn width."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        routing = np.ascontiguousarray(routing, dtype=np.float32)
        tokens = x.shape[1]
        y = np.zeros((hidden, tokens), dtype=np.float32)
        g, u, d = (np.ascontiguousarray(a, dtype=np.uint8) for a in (gate, up, down))
        ptrs, keep = (None, None, None, None), []
        if shared_kind:
            sg, su, sd = (np.ascontiguousarray(a, dtype=np.uint8) for a in shared[:3])
            keep = [sg, su, sd]
            sw = None
            if shared_kind == 2:
                sw = np.ascontiguousarray(shared[3], dtype=np.float32)
                keep.append(sw)
            ptrs = (sg.ctypes.data, su.ctypes.data, sd.ctypes.data, None if sw is None else sw.ctypes.data)
        rc = self.lib.rqo_moe_forward_ex(t, g.ctypes.data, u.ctypes.data, d.ctypes.data, experts, top, hidden, ffn, x.ctypes.data, routing.ctypes.data, tokens,
                                         routed_scale, shared_kind, shared_count, *ptrs, y.ctypes.data, threads or THREADS)
        assert rc == 0, rc
        return y

    def rmsnorm(self, x: np.ndarray, gain, epsilon: float) -> np.ndarray:
        """x [n] or [tokens, n] -> the RMS-normalised positions."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        x2 = x[None, :] if x.ndim == 1 else x
        y = np.empty_like(x2)
        g = None if gain is None else np.ascontiguousarray(gain, dtype=np.float32)
        for t in range(x2.shape[0]):
            self.lib.rqo_rmsnorm(x2[t].ctypes.data, 1, x2.shape[1], None if g is None else g.ctypes.data, epsilon, y[t].ctypes.data, 1)
        return y[0] if x.ndim == 1 else y

    def softcap(self, x: np.ndarray, cap: float) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        self.lib.rqo_softcap(x.ctypes.data, x.size, cap, y.ctypes.data)
        return y

    def glu(self, gate: np.ndarray, up: np.ndarray) -> np.ndarray:
        g, u = np.ascontiguousarray(gate, dtype=np.float32), np.ascontiguousarray(up, dtype=np.float32)
        y = np.empty_like(g)
        self.lib.rqo_glu(g.ctypes.data, u.ctypes.data, g.size, y.ctypes.data)
        return y

    def normal(self, seed: int, stream: int, count: int, sigma: float = 1.0, first: int = 0) -> np.ndarray:
        out = np.empty(count, dtype=np.float32)
        self.lib.rqo_normal(seed, stream, first, count, sigma, out.ctypes.data)
        return out

    def fp16(self, v: float) -> int:
        return int(self.lib.rqo_fp16(v))

    def unfp16(self, h: int) -> float:
        return float(self.lib.rqo_unfp16(h))


_ORACLE = None


def load() -> Oracle:
    global _ORACLE
    if _ORACLE is None:
        _ORACLE = Oracle(C.CDLL(str(build())))
    return _ORACLE
