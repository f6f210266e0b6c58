"""B200-native GGUF quantised matrix-vector path (Q8_0, Q4_0, Q4_K, Q6_K; ten more stored formats by per-value decode).

The product is ``librq_b200.so``: hand-written CUDA for sm_100a behind the C ABI declared in
``include/rq.h``. This package only binds it (ctypes) and supplies device memory through
torch; there is no CPU path, and loading fails loudly when the library is missing.
"""
from .capi import (  # noqa: F401
    ACT_FLOAT,
    ACT_INT8,
    IQ4_NL,
    IQ4_XS,
    Q2_K,
    Q3_K,
    Q4_0,
    Q4_1,
    Q4_K,
    Q5_0,
    Q5_1,
    Q5_K,
    Q6_K,
    Q8_0,
    Q8_1,
    Q8_K,
    Context,
    Exchange,
    Gguf,
    NcclComm,
    RqError,
    Weight,
    block_bytes,
    block_values,
    library_path,
    load_library,
)

__all__ = [
    "ACT_FLOAT", "ACT_INT8", "IQ4_NL", "IQ4_XS", "Q2_K", "Q3_K", "Q8_1", "Q8_K", "Q4_0", "Q4_1", "Q4_K", "Q5_0", "Q5_1", "Q5_K", "Q6_K", "Q8_0",
    "Context", "Exchange", "Gguf", "NcclComm", "RqError", "Weight", "block_bytes", "block_values", "library_path", "load_library",
]
