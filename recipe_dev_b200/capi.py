"""ctypes binding of the C ABI in include/rq.h.

Device buffers are torch CUDA tensors (torch is the allocator and the stream provider);
every call goes straight to the library. If ``librq_b200.so`` is absent the import of the
library raises: nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

Q4_0, Q8_0, Q4_K, Q6_K = 2, 8, 12, 14
Q4_1, Q5_0, Q5_1, Q5_K, IQ4_NL = 3, 6, 7, 13, 20  # bound, decoded, dotted with fp32 activations, re-encoded under int8
Q8_1, Q2_K, Q3_K, Q8_K, IQ4_XS = 9, 10, 11, 15, 23  # the same
ACT_FLOAT, ACT_INT8 = 0, 1
SCORE_SOFTMAX, SCORE_SIGMOID = 0, 1

_PKG = Path(__file__).resolve().parent
_LIB = None


class RqError(RuntimeError):
    """A call into librq_b200.so returned a negative status."""

    def __init__(self, status: int, text: str):
        super().__init__(f"rq status {status}: {text}")
        self.status = status


def library_path() -> Path:
    return _PKG / "librq_b200.so"


def _declare(lib) -> None:
    p, i32, i64, f32p = C.c_void_p, C.c_int, C.c_int64, C.c_void_p
    sig = {
        "rq_init": (i32, [i32, C.POINTER(p)]),
        "rq_destroy": (None, [p]),
        "rq_last_error": (C.c_char_p, []),
        "rq_check": (i32, [p]),
        "rq_reserve": (i32, [p, i64, i64, i32]),
        "rq_set_wait_limit": (i32, [p, C.c_uint64]),
        "rq_wait_selftest": (i32, [p, p]),
        "rq_block_values": (i32, [i32]),
        "rq_block_bytes": (i32, [i32]),
        "rq_weight_prepare": (i32, [p, i32, p, i64, i64, i64, i64, C.POINTER(p)]),
        "rq_weight_prepare_device": (i32, [p, i32, p, i64, i64, C.POINTER(p), p]),
        "rq_weight_export": (i32, [p, p, p]),
        "rq_weight_requantize": (i32, [p, p, i32, C.POINTER(p), p]),
        "rq_int8_keeps": (i32, [i32]),
        "rq_int4_keeps": (i32, [i32]),
        "rq_weight_free": (None, [p, p]),
        "rq_weight_rows": (i64, [p]),
        "rq_weight_cols": (i64, [p]),
        "rq_weight_type": (i32, [p]),
        "rq_weight_bytes": (i64, [p]),
        "rq_dequant": (i32, [p, p, f32p, p]),
        "rq_quantize": (i32, [p, i32, f32p, i64, p, p]),
        "rq_gather_rows": (i32, [p, p, p, i32, f32p, i64, i64, p]),
        "rq_matvec": (i32, [p, p, f32p, i64, i64, i32, f32p, i64, i64, i32, i32, p]),
        "rq_matmul": (i32, [p, p, f32p, i64, i64, i32, f32p, i64, i64, i32, i32, p]),
        "rq_matvec_glu": (i32, [p, p, p, f32p, i64, i64, i32, f32p, i64, i64, i32, i32, p]),
        "rq_rmsnorm": (i32, [p, f32p, i64, i64, i64, i32, f32p, C.c_float, f32p, i64, i64, p]),
        "rq_add": (i32, [p, f32p, f32p, i64, f32p, p]),
        "rq_softcap": (i32, [p, f32p, i64, C.c_double, f32p, p]),
        "rq_matvec_multi": (i32, [p, i32, p, f32p, i64, i64, i32, p, i64, i64, i32, i32, p]),
        "rq_matvec_host": (i32, [p, p, f32p, i64, i64, i32, f32p, i64, i64, i32, i32]),
        "rq_matvec_multi_host": (i32, [p, i32, p, f32p, i64, i64, i32, p, i64, i64, i32, i32]),
        "rq_quantize_activations": (i32, [p, f32p, i64, i64, i64, i32, i32, p, p]),
        "rq_matvec_int8_static": (i32, [p, p, f32p, f32p, i32, p]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    # optional groups (declared when the library exports them)
    optional = {
        "rq_moe_route": (i32, [p, f32p, i64, i64, i32, i32, i32, i32, f32p, i32, f32p, i64, i64, p]),
        "rq_moe_prepare": (i32, [p, i32, p, p, p, i32, i32, i32, i32, i32, p, p, p, f32p, C.POINTER(p)]),
        "rq_moe_free": (None, [p, p]),
        "rq_moe_set_routed_scale": (i32, [p, C.c_float]),
        "rq_moe_attach_shared": (i32, [p, p, i32, i32, p, p, p, f32p]),
        "rq_moe_bytes": (i64, [p]),
        "rq_moe_forward": (i32, [p, p, f32p, i64, i64, f32p, i64, i64, i32, i32, i32, f32p, i64, i64, p]),
        "rq_moe_route_forward": (i32, [p, p, f32p, i64, i64, i32, i32, i32, f32p, f32p, i64, i64, f32p, i64, i64, i32, i32, f32p, i64, i64, p]),
        "rq_device_alloc": (i32, [p, i64, C.POINTER(p)]),
        "rq_device_free": (None, [p, p]),
        "rq_sequence_begin": (i32, [p, C.POINTER(p)]),
        "rq_sequence_end": (i32, [p, C.POINTER(p)]),
        "rq_sequence_run": (i32, [p, p]),
        "rq_sequence_run_host": (i32, [p, f32p, f32p, i64, f32p, f32p, i64]),
        "rq_sequence_free": (None, [p]),
        "rq_gguf_open": (i32, [C.c_char_p, C.POINTER(p)]),
        "rq_gguf_close": (None, [p]),
        "rq_gguf_tensor_count": (i32, [p]),
        "rq_gguf_find": (i32, [p, C.c_char_p]),
        "rq_gguf_tensor_name": (C.c_char_p, [p, i32]),
        "rq_gguf_tensor_type": (i32, [p, i32]),
        "rq_gguf_tensor_dims": (i32, [p, i32, C.POINTER(i64), i32]),
        "rq_gguf_tensor_bytes": (i64, [p, i32]),
        "rq_gguf_tensor_data": (p, [p, i32]),
        "rq_gguf_meta_count": (i32, [p]),
        "rq_gguf_meta_key": (C.c_char_p, [p, i32]),
        "rq_gguf_meta_kind": (i32, [p, C.c_char_p]),
        "rq_gguf_meta_integer": (i32, [p, C.c_char_p, C.POINTER(C.c_uint64)]),
        "rq_gguf_meta_float": (i32, [p, C.c_char_p, C.POINTER(C.c_double)]),
        "rq_gguf_meta_text": (C.c_char_p, [p, C.c_char_p]),
        "rq_gguf_meta_array_length": (i64, [p, C.c_char_p]),
        "rq_gguf_meta_array_text": (C.c_char_p, [p, C.c_char_p, i64]),
        "rq_gguf_bind": (i32, [p, p, C.c_char_p, i64, i64, C.POINTER(p)]),
        "rq_gguf_bind_experts": (i32, [p, p, C.c_char_p, C.c_char_p, C.c_char_p, i32, i32, C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, C.POINTER(p)]),
        "rq_allgather_rows": (i32, [p, p, f32p, f32p, i64, p]),
        "rq_allreduce_sum": (i32, [p, p, f32p, f32p, i64, p]),
        "rq_nccl_unique_id": (i32, [p]),
        "rq_nccl_comm_create": (i32, [p, p, i32, i32, C.POINTER(p)]),
        "rq_nccl_comm_destroy": (None, [p]),
        "rq_exchange_create": (i32, [p, i32, i32, i64, C.POINTER(p)]),
        "rq_exchange_handle": (i32, [p, p]),
        "rq_exchange_buffer": (p, [p]),
        "rq_exchange_connect": (i32, [p, p, p]),
        "rq_exchange_gather": (i32, [p, f32p, i64, f32p, p]),
        "rq_exchange_reduce": (i32, [p, f32p, i64, f32p, p]),
        "rq_exchange_free": (None, [p]),
    }
    for name, (res, args) in optional.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args


def load_library():
    """Loads librq_b200.so, or raises: the CUDA extension is the only implementation."""
    global _LIB
    if _LIB is None:
        path = library_path()
        if not path.exists():
            raise RqError(-4, f"{path} is missing: build it with `python -m recipe_dev_b200.build` (nvcc, sm_100a); there is no CPU fallback")
        lib = C.CDLL(str(path))
        _declare(lib)
        _LIB = lib
    return _LIB


def block_values(ggml_type: int) -> int:
    return load_library().rq_block_values(ggml_type)


def block_bytes(ggml_type: int) -> int:
    return load_library().rq_block_bytes(ggml_type)


def _check(status: int) -> None:
    if status != 0:
        raise RqError(status, load_library().rq_last_error().decode("utf-8", "replace"))


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _stream(stream) -> int:
    if stream is None:
        import torch

        return torch.cuda.current_stream().cuda_stream
    return stream if isinstance(stream, int) else stream.cuda_stream


class Weight:
    """A stored weight resident in HBM (rq_weight)."""

    def __init__(self, ctx: "Context", handle: int):
        self.ctx, self.handle = ctx, handle

    @property
    def rows(self) -> int:
        return self.ctx.lib.rq_weight_rows(self.handle)

    @property
    def cols(self) -> int:
        return self.ctx.lib.rq_weight_cols(self.handle)

    @property
    def type(self) -> int:
        return self.ctx.lib.rq_weight_type(self.handle)

    @property
    def nbytes(self) -> int:
        return self.ctx.lib.rq_weight_bytes(self.handle)

    def free(self) -> None:
        if self.handle:
            self.ctx.lib.rq_weight_free(self.ctx.handle, self.handle)
            self.handle = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class MoeBank:
    """The expert tables of one gguf_moe block resident in HBM (rq_moe)."""

    def __init__(self, ctx: "Context", handle: int, hidden: int, ffn: int):
        self.ctx, self.handle, self.hidden, self.ffn = ctx, handle, hidden, ffn

    @property
    def nbytes(self) -> int:
        return self.ctx.lib.rq_moe_bytes(self.handle)

    def set_routed_scale(self, scale: float) -> None:
        _check(self.ctx.lib.rq_moe_set_routed_scale(self.handle, scale))

    def attach_shared(self, gate, up, down, count: int = 1, gate_vector=None) -> None:
        """A shared expert of count * ffn width: gated by sigmoid(gate_vector . x) when a vector is given, else at weight one."""
        g, u, d = (np.ascontiguousarray(a, dtype=np.uint8) for a in (gate, up, down))
        v = None if gate_vector is None else np.ascontiguousarray(gate_vector, dtype=np.float32)
        _check(self.ctx.lib.rq_moe_attach_shared(self.ctx.handle, self.handle, int(v is not None), count, g.ctypes.data, u.ctypes.data, d.ctypes.data,
                                                 None if v is None else v.ctypes.data))

    def free(self) -> None:
        if self.handle:
            self.ctx.lib.rq_moe_free(self.ctx.handle, self.handle)
            self.handle = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Context:
    """One device context (rq_ctx)."""

    def __init__(self, device: int = 0):
        self.lib = load_library()
        handle = C.c_void_p()
        _check(self.lib.rq_init(device, C.byref(handle)))
        self.handle = handle.value
        self.device = device

    def close(self) -> None:
        if getattr(self, "handle", 0):
            self.lib.rq_destroy(self.handle)
            self.handle = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self) -> None:
        """Synchronises and raises if a kernel gave up a bounded wait since the last check."""
        _check(self.lib.rq_check(self.handle))

    def reserve(self, max_rows: int, max_cols: int, max_tokens: int) -> None:
        """Sizes the work areas ahead of time, so that no later call within these sizes allocates or synchronises."""
        _check(self.lib.rq_reserve(self.handle, max_rows, max_cols, max_tokens))

    def set_wait_limit(self, nanoseconds: int) -> None:
        _check(self.lib.rq_set_wait_limit(self.handle, nanoseconds))

    def wait_selftest(self, stream=None) -> None:
        _check(self.lib.rq_wait_selftest(self.handle, _stream(stream)))

    # ---- recorded sequences ----
    def sequence_begin(self) -> int:
        """Starts recording; returns the stream (an int) to pass to the calls that are to be recorded."""
        out = C.c_void_p()
        _check(self.lib.rq_sequence_begin(self.handle, C.byref(out)))
        return out.value

    def sequence_end(self) -> "Sequence":
        out = C.c_void_p()
        _check(self.lib.rq_sequence_end(self.handle, C.byref(out)))
        return Sequence(self, out.value)

    # ---- weights ----
    def weight_from_host(self, ggml_type: int, blocks: np.ndarray, rows: int, cols: int, row_first: int = 0, row_count: int | None = None) -> Weight:
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        row_count = rows - row_first if row_count is None else row_count
        out = C.c_void_p()
        _check(self.lib.rq_weight_prepare(self.handle, ggml_type, blocks.ctypes.data, rows, cols, row_first, row_count, C.byref(out)))
        return Weight(self, out.value)

    def weight_from_device(self, ggml_type: int, dev_blocks, rows: int, cols: int, stream=None) -> Weight:
        out = C.c_void_p()
        _check(self.lib.rq_weight_prepare_device(self.handle, ggml_type, _ptr(dev_blocks), rows, cols, C.byref(out), _stream(stream)))
        return Weight(self, out.value)

    def requantize(self, w: Weight, target_type: int = Q8_0, stream=None) -> Weight:
        """The load-time re-encode `.int(8)` applies to a tensor it does not keep (a lone Q6_K / Q4_0 one)."""
        out = C.c_void_p()
        _check(self.lib.rq_weight_requantize(self.handle, w.handle, target_type, C.byref(out), _stream(stream)))
        return Weight(self, out.value)

    def int4_weight(self, w: Weight, stream=None) -> Weight:
        """The weight `.int(4)` dots: `w` itself when it is stored as Q4_1, else its load-time Q4_1 re-encode."""
        return w if self.lib.rq_int4_keeps(w.type) else self.requantize(w, Q4_1, stream)

    def int8_weight(self, w: Weight, stream=None) -> Weight:
        """The weight recipe's `.int(8)` dots: `w` itself when the format is kept, else its Q8_0 re-encode."""
        return w if self.lib.rq_int8_keeps(w.type) else self.requantize(w, Q8_0, stream)

    def export(self, w: Weight) -> np.ndarray:
        n = w.rows * (w.cols // block_values(w.type)) * block_bytes(w.type)
        out = np.empty(n, dtype=np.uint8)
        _check(self.lib.rq_weight_export(self.handle, w.handle, out.ctypes.data))
        return out

    def dequant(self, w: Weight, out=None, stream=None):
        import torch

        if out is None:
            out = torch.empty((w.rows, w.cols), dtype=torch.float32, device=f"cuda:{self.device}")
        _check(self.lib.rq_dequant(self.handle, w.handle, _ptr(out), _stream(stream)))
        return out

    def gather_rows(self, table: Weight, ids, y=None, stream=None):
        """ids: CUDA int32 [tokens] -> y [tokens, cols]: the table's rows ids[t], decoded (embedding lookup)."""
        import torch

        assert ids.is_cuda and ids.dtype == torch.int32 and ids.is_contiguous()
        tokens = ids.numel()
        if y is None:
            y = torch.empty((tokens, table.cols), dtype=torch.float32, device=ids.device)
        _check(self.lib.rq_gather_rows(self.handle, table.handle, _ptr(ids), tokens, _ptr(y), y.stride(1), y.stride(0), _stream(stream)))
        return y

    def quantize(self, ggml_type: int, values, stream=None):
        """fp32 CUDA tensor -> uint8 CUDA tensor of GGUF blocks."""
        import torch

        assert values.is_cuda and values.dtype == torch.float32 and values.is_contiguous()
        n = values.numel()
        per, nbytes = block_values(ggml_type), block_bytes(ggml_type)
        out = torch.empty((n // max(per, 1)) * nbytes if per else 0, dtype=torch.uint8, device=values.device)
        _check(self.lib.rq_quantize(self.handle, ggml_type, _ptr(values), n, _ptr(out), _stream(stream)))
        return out

    # ---- matvec ----
    def matvec(self, w: Weight, x, y=None, act_mode: int = ACT_FLOAT, step: int = 32, stream=None):
        """x: CUDA fp32, [cols] or [tokens, cols] (token-major) -> y [rows] or [tokens, rows]."""
        import torch

        single = x.dim() == 1
        x2 = x.unsqueeze(0) if single else x
        tokens, cols = x2.shape
        if y is None:
            y = torch.empty((tokens, w.rows), dtype=torch.float32, device=x.device)
        y2 = y.unsqueeze(0) if y.dim() == 1 else y
        _check(self.lib.rq_matvec(self.handle, w.handle, _ptr(x2), x2.stride(1), x2.stride(0), tokens,
                                  _ptr(y2), y2.stride(1), y2.stride(0), act_mode, step, _stream(stream)))
        return y2[0] if single else y2

    def matvec_glu(self, gate: Weight, up: Weight, x, y=None, act_mode: int = ACT_FLOAT, step: int = 32, stream=None):
        """silu(gate x) * (up x) in one launch; x [cols] or [tokens, cols] -> y [rows] or [tokens, rows]."""
        import torch

        single = x.dim() == 1
        x2 = x.unsqueeze(0) if single else x
        tokens = x2.shape[0]
        if y is None:
            y = torch.empty((tokens, gate.rows), dtype=torch.float32, device=x.device)
        y2 = y.unsqueeze(0) if y.dim() == 1 else y
        _check(self.lib.rq_matvec_glu(self.handle, gate.handle, up.handle, _ptr(x2), x2.stride(1), x2.stride(0), tokens, _ptr(y2), y2.stride(1), y2.stride(0),
                                      act_mode, step, _stream(stream)))
        return y2[0] if single else y2

    def rmsnorm(self, x, gain=None, epsilon: float = 1e-6, y=None, stream=None):
        """x [n] or [tokens, n] (token-major) -> RMS-normalised, times gain [n] when given."""
        import torch

        x2 = x.unsqueeze(0) if x.dim() == 1 else x
        tokens, n = x2.shape
        if y is None:
            y = torch.empty_like(x2)
        y2 = y.unsqueeze(0) if y.dim() == 1 else y
        _check(self.lib.rq_rmsnorm(self.handle, _ptr(x2), x2.stride(1), x2.stride(0), n, tokens, _ptr(gain), epsilon, _ptr(y2), y2.stride(1), y2.stride(0), _stream(stream)))
        return y2[0] if x.dim() == 1 else y2

    def add(self, a, b, y=None, stream=None):
        import torch

        if y is None:
            y = torch.empty_like(a)
        _check(self.lib.rq_add(self.handle, _ptr(a), _ptr(b), a.numel(), _ptr(y), _stream(stream)))
        return y

    def softcap(self, x, cap: float, y=None, stream=None):
        import torch

        if y is None:
            y = torch.empty_like(x)
        _check(self.lib.rq_softcap(self.handle, _ptr(x), x.numel(), cap, _ptr(y), _stream(stream)))
        return y

    def matmul(self, w: Weight, x, y=None, act_mode: int = ACT_FLOAT, step: int = 32, stream=None):
        """x: CUDA fp32 [tokens, cols] -> y [tokens, rows]; the tensor-core path for RQ_ACT_FLOAT."""
        import torch

        tokens, cols = x.shape
        if y is None:
            y = torch.empty((tokens, w.rows), dtype=torch.float32, device=x.device)
        _check(self.lib.rq_matmul(self.handle, w.handle, _ptr(x), x.stride(1), x.stride(0), tokens, _ptr(y), y.stride(1), y.stride(0), act_mode, step,
                                  _stream(stream)))
        return y

    def matvec_multi(self, ws, x, ys, act_mode: int = ACT_FLOAT, step: int = 32, stream=None):
        """Several weights of one format and width against the same x; ys[i] is [rows_i] or [tokens, rows_i]."""
        x2 = x.unsqueeze(0) if x.dim() == 1 else x
        tokens = x2.shape[0]
        y2 = [y.unsqueeze(0) if y.dim() == 1 else y for y in ys]
        n = len(ws)
        if any(y.stride(1) != y2[0].stride(1) or (tokens > 1 and y.stride(0) != y2[0].stride(0)) for y in y2):
            raise ValueError("matvec_multi: every output must have the same strides (e.g. column slices of one [tokens, all rows] plane)")
        wa = (C.c_void_p * n)(*[w.handle for w in ws])
        ya = (C.c_void_p * n)(*[y.data_ptr() for y in y2])
        _check(self.lib.rq_matvec_multi(self.handle, n, wa, _ptr(x2), x2.stride(1), x2.stride(0), tokens,
                                        ya, y2[0].stride(1), y2[0].stride(0), act_mode, step, _stream(stream)))
        return ys

    def matvec_raw(self, w: Weight, x_ptr: int, sk: int, st: int, tokens: int, y_ptr: int, yn: int, yt: int, act_mode: int, step: int, stream=None) -> int:
        return self.lib.rq_matvec(self.handle, w.handle, x_ptr, sk, st, tokens, y_ptr, yn, yt, act_mode, step, _stream(stream) if stream is not None else 0)

    def matvec_host(self, w: Weight, x: np.ndarray, act_mode: int = ACT_FLOAT, step: int = 32) -> np.ndarray:
        """Host buffers in and out: x [cols] or [tokens, cols] float32."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        single = x.ndim == 1
        x2 = x[None, :] if single else x
        tokens = x2.shape[0]
        y = np.empty((tokens, w.rows), dtype=np.float32)
        _check(self.lib.rq_matvec_host(self.handle, w.handle, x2.ctypes.data, 1, x2.shape[1], tokens, y.ctypes.data, 1, w.rows, act_mode, step))
        return y[0] if single else y

    def matvec_multi_host(self, ws, x: np.ndarray, act_mode: int = ACT_FLOAT, step: int = 32):
        """Host buffers in and out for several weights that read one x ([cols] or [tokens, cols]): a list of outputs."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        single = x.ndim == 1
        x2 = x[None, :] if single else x
        tokens, n = x2.shape[0], len(ws)
        total = sum(w.rows for w in ws)
        plane = np.empty((tokens, total), dtype=np.float32)  # the outputs share one token stride: slices of one plane
        offs = np.cumsum([0] + [w.rows for w in ws])
        wa = (C.c_void_p * n)(*[w.handle for w in ws])
        ya = (C.c_void_p * n)(*[plane.ctypes.data + 4 * int(o) for o in offs[:-1]])
        _check(self.lib.rq_matvec_multi_host(self.handle, n, wa, x2.ctypes.data, 1, x2.shape[1], tokens, ya, 1, total, act_mode, step))
        ys = [plane[:, int(offs[i]):int(offs[i + 1])] for i in range(n)]
        return [y[0] for y in ys] if single else ys

    def matvec_int8_static(self, w: Weight, x, y=None, step: int = 32, stream=None):
        """The INT8 product of one contiguous column through the entry point that allocates nothing
        (its scratch is a fixed array in the library; at most 32768 inputs per row)."""
        import torch

        assert x.dim() == 1 and x.is_contiguous()
        if y is None:
            y = torch.empty(w.rows, dtype=torch.float32, device=x.device)
        _check(self.lib.rq_matvec_int8_static(self.handle, w.handle, _ptr(x), _ptr(y), step, _stream(stream)))
        return y

    # ---- gguf_moe ----
    def moe_route(self, scores, top_k: int, scoring: int = SCORE_SOFTMAX, renormalize: bool = True, bias=None, stream=None):
        """scores: CUDA fp32 [experts, tokens] (the reference's channel-major plane) -> weights of the same shape."""
        import torch

        experts, tokens = scores.shape
        weights = torch.empty_like(scores)
        _check(self.lib.rq_moe_route(self.handle, _ptr(scores), scores.stride(0), scores.stride(1), experts, top_k, scoring, int(renormalize),
                                     _ptr(bias), tokens, _ptr(weights), weights.stride(0), weights.stride(1), _stream(stream)))
        return weights

    def moe_prepare(self, ggml_type: int, gate, up, down, experts: int, hidden: int, ffn: int, expert_first: int = 0, expert_count: int | None = None,
                    shared=None) -> "MoeBank":
        """gate/up/down: host uint8 GGUF blocks of the whole bank; shared = (gate, up, down, gate_vector) or None."""
        expert_count = experts - expert_first if expert_count is None else expert_count
        g, u, d = (np.ascontiguousarray(a, dtype=np.uint8) for a in (gate, up, down))
        keep = [g, u, d]
        sp = [None, None, None, None]
        if shared is not None:
            sg, su, sd = (np.ascontiguousarray(a, dtype=np.uint8) for a in shared[:3])
            sv = np.ascontiguousarray(shared[3], dtype=np.float32)
            keep += [sg, su, sd, sv]
            sp = [sg.ctypes.data, su.ctypes.data, sd.ctypes.data, sv.ctypes.data]
        out = C.c_void_p()
        _check(self.lib.rq_moe_prepare(self.handle, ggml_type, g.ctypes.data, u.ctypes.data, d.ctypes.data, experts, expert_first, expert_count,
                                       hidden, ffn, sp[0], sp[1], sp[2], sp[3], C.byref(out)))
        return MoeBank(self, out.value, hidden, ffn)

    def moe_forward(self, bank: "MoeBank", x, routing, top_k: int, include_shared: bool = True, y=None, stream=None):
        """x: CUDA fp32 [hidden, tokens]; routing: [experts, tokens] -> y [hidden, tokens] (channel-major planes)."""
        import torch

        hidden, tokens = x.shape
        if y is None:
            y = torch.empty((hidden, tokens), dtype=torch.float32, device=x.device)
        _check(self.lib.rq_moe_forward(self.handle, bank.handle, _ptr(x), x.stride(0), x.stride(1), _ptr(routing), routing.stride(0), routing.stride(1),
                                       top_k, tokens, int(include_shared), _ptr(y), y.stride(0), y.stride(1), _stream(stream)))
        return y

    def moe_route_forward(self, bank: "MoeBank", scores, x, top_k: int, scoring: int = SCORE_SOFTMAX, renormalize: bool = True, bias=None, include_shared: bool = True,
                          weights=None, y=None, stream=None):
        """moe_route + moe_forward as one call (three launches instead of four). scores: [experts, tokens]; returns (y, weights)."""
        import torch

        hidden, tokens = x.shape
        if y is None:
            y = torch.empty((hidden, tokens), dtype=torch.float32, device=x.device)
        if weights is None:
            weights = torch.empty_like(scores)
        _check(self.lib.rq_moe_route_forward(self.handle, bank.handle, _ptr(scores), scores.stride(0), scores.stride(1), top_k, scoring, int(renormalize),
                                             _ptr(bias), _ptr(weights), weights.stride(0), weights.stride(1), _ptr(x), x.stride(0),
                                             x.stride(1), tokens, int(include_shared), _ptr(y), y.stride(0), y.stride(1), _stream(stream)))
        return y, weights

    def activation_records(self, x, step: int, stream=None):
        """The 36-byte int8 records of x ([cols] or [tokens, cols]) as a uint8 CUDA tensor."""
        import torch

        x2 = x.unsqueeze(0) if x.dim() == 1 else x
        tokens, cols = x2.shape
        out = torch.empty((tokens, cols // 32, 36), dtype=torch.uint8, device=x.device)
        _check(self.lib.rq_quantize_activations(self.handle, _ptr(x2), x2.stride(1), x2.stride(0), cols, tokens, step, _ptr(out), _stream(stream)))
        return out


class NcclComm:
    """An NCCL communicator made through the library (rq_nccl_comm_create) for hosts that have none of their own."""

    def __init__(self, ctx: "Context", handle: int, rank: int, nranks: int):
        self.ctx, self.handle, self.rank, self.nranks = ctx, handle, rank, nranks

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        _check(load_library().rq_nccl_unique_id(buf))
        return buf.raw

    @classmethod
    def create(cls, ctx: "Context", unique_id: bytes, nranks: int, rank: int) -> "NcclComm":
        out = C.c_void_p()
        _check(ctx.lib.rq_nccl_comm_create(ctx.handle, unique_id, nranks, rank, C.byref(out)))
        return cls(ctx, out.value, rank, nranks)

    def allgather_rows(self, local, gathered, stream=None):
        """local: CUDA fp32 [count]; gathered: [nranks, count]."""
        _check(self.ctx.lib.rq_allgather_rows(self.ctx.handle, self.handle, _ptr(local), _ptr(gathered), local.numel(), _stream(stream)))
        return gathered

    def allreduce_sum(self, local, summed, stream=None):
        _check(self.ctx.lib.rq_allreduce_sum(self.ctx.handle, self.handle, _ptr(local), _ptr(summed), local.numel(), _stream(stream)))
        return summed

    def destroy(self) -> None:
        if self.handle:
            self.ctx.lib.rq_nccl_comm_destroy(self.handle)
            self.handle = 0


class Exchange:
    """The library's own exchange over peer memory (rq_exchange): gather and rank-order sum, one kernel each."""

    def __init__(self, ctx: "Context", rank: int, nranks: int, slot_bytes: int):
        self.ctx, self.rank, self.nranks = ctx, rank, nranks
        out = C.c_void_p()
        _check(ctx.lib.rq_exchange_create(ctx.handle, rank, nranks, slot_bytes, C.byref(out)))
        self.handle = out.value

    def ipc_handle(self) -> bytes:
        buf = C.create_string_buffer(64)
        _check(self.ctx.lib.rq_exchange_handle(self.handle, buf))
        return buf.raw

    def connect(self, handles: list[bytes]) -> None:
        """handles: every rank's 64-byte handle, in rank order."""
        blob = b"".join(handles)
        assert len(blob) == 64 * self.nranks
        _check(self.ctx.lib.rq_exchange_connect(self.handle, blob, None))

    def connect_same_process(self, exchanges: list["Exchange"]) -> None:
        ptrs = (C.c_void_p * self.nranks)(*[e.ctx.lib.rq_exchange_buffer(e.handle) for e in exchanges])
        _check(self.ctx.lib.rq_exchange_connect(self.handle, None, ptrs))

    def gather(self, local, gathered, stream=None):
        """local: CUDA fp32 [count] (contiguous); gathered: [nranks, count]."""
        _check(self.ctx.lib.rq_exchange_gather(self.handle, _ptr(local), local.numel(), _ptr(gathered), _stream(stream)))
        return gathered

    def reduce(self, local, summed, stream=None):
        _check(self.ctx.lib.rq_exchange_reduce(self.handle, _ptr(local), local.numel(), _ptr(summed), _stream(stream)))
        return summed

    def free(self) -> None:
        if self.handle:
            self.ctx.lib.rq_exchange_free(self.handle)
            self.handle = 0


class Gguf:
    """A GGUF v3 file (or split model) mapped read-only: tensor descriptors, metadata, binding to resident weights."""

    def __init__(self, path):
        self.lib = load_library()
        out = C.c_void_p()
        _check(self.lib.rq_gguf_open(str(path).encode(), C.byref(out)))
        self.handle = out.value

    def close(self) -> None:
        if getattr(self, "handle", 0):
            self.lib.rq_gguf_close(self.handle)
            self.handle = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def tensors(self) -> list[dict]:
        out = []
        for i in range(self.lib.rq_gguf_tensor_count(self.handle)):
            dims = (C.c_int64 * 8)()
            n = self.lib.rq_gguf_tensor_dims(self.handle, i, dims, 8)
            out.append({"name": self.lib.rq_gguf_tensor_name(self.handle, i).decode(), "type": self.lib.rq_gguf_tensor_type(self.handle, i),
                        "shape": [int(dims[d]) for d in range(n)], "bytes": int(self.lib.rq_gguf_tensor_bytes(self.handle, i))})
        return out

    def data(self, name: str) -> np.ndarray:
        """The tensor's bytes as the file holds them (a copy of the mapped view)."""
        i = self.lib.rq_gguf_find(self.handle, name.encode())
        if i < 0:
            raise KeyError(name)
        n = int(self.lib.rq_gguf_tensor_bytes(self.handle, i))
        return np.ctypeslib.as_array((C.c_uint8 * n).from_address(self.lib.rq_gguf_tensor_data(self.handle, i))).copy()

    def keys(self) -> list[str]:
        return [self.lib.rq_gguf_meta_key(self.handle, i).decode() for i in range(self.lib.rq_gguf_meta_count(self.handle))]

    def integer(self, key: str) -> int:
        v = C.c_uint64()
        _check(self.lib.rq_gguf_meta_integer(self.handle, key.encode(), C.byref(v)))
        return int(v.value)

    def float(self, key: str) -> float:
        v = C.c_double()
        _check(self.lib.rq_gguf_meta_float(self.handle, key.encode(), C.byref(v)))
        return float(v.value)

    def text(self, key: str):
        v = self.lib.rq_gguf_meta_text(self.handle, key.encode())
        return None if v is None else v.decode()

    def array_text(self, key: str) -> list[str]:
        n = self.lib.rq_gguf_meta_array_length(self.handle, key.encode())
        if n < 0:
            raise KeyError(key)
        return [self.lib.rq_gguf_meta_array_text(self.handle, key.encode(), i).decode() for i in range(n)]

    def bind(self, ctx: "Context", name: str, row_first: int = 0, row_count: int = 0) -> Weight:
        out = C.c_void_p()
        _check(self.lib.rq_gguf_bind(ctx.handle, self.handle, name.encode(), row_first, row_count, C.byref(out)))
        return Weight(ctx, out.value)

    def bind_experts(self, ctx: "Context", gate: str, up: str, down: str, expert_first: int = 0, expert_count: int = 0, shared=None) -> MoeBank:
        """shared = (gate, up, down, gate_vector) tensor names or None."""
        sh = [None] * 4 if shared is None else [s.encode() for s in shared]
        out = C.c_void_p()
        _check(self.lib.rq_gguf_bind_experts(ctx.handle, self.handle, gate.encode(), up.encode(), down.encode(), expert_first, expert_count, *sh, C.byref(out)))
        dims = (C.c_int64 * 8)()
        self.lib.rq_gguf_tensor_dims(self.handle, self.lib.rq_gguf_find(self.handle, gate.encode()), dims, 8)
        return MoeBank(ctx, out.value, int(dims[0]), int(dims[1]))


class Sequence:
    """A recorded list of calls (rq_sequence): replayed as one submission."""

    def __init__(self, ctx: "Context", handle: int):
        self.ctx, self.handle = ctx, handle

    def run(self, stream=None) -> None:
        _check(self.ctx.lib.rq_sequence_run(self.handle, _stream(stream)))

    def run_host(self, host_in: np.ndarray, dev_in, dev_out, host_out: np.ndarray) -> np.ndarray:
        """One copy in (host_in -> dev_in), the recorded calls, one copy out (dev_out -> host_out), one synchronisation."""
        _check(self.ctx.lib.rq_sequence_run_host(self.handle, host_in.ctypes.data, _ptr(dev_in), host_in.size, _ptr(dev_out), host_out.ctypes.data, host_out.size))
        return host_out

    def free(self) -> None:
        if self.handle:
            self.ctx.lib.rq_sequence_free(self.handle)
            self.handle = 0
