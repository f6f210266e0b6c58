"""The C-ABI library loads without a GPU and exports every symbol include/*.h declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    names = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names.update(re.findall(r"\b(rq_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_builds_and_exports_every_declared_symbol():
    from recipe_dev_b200 import build

    lib = ctypes.CDLL(str(build.build()))
    names = declared_symbols()
    assert len(names) >= 18
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_block_geometry_and_error_text_without_gpu():
    import recipe_dev_b200 as rq

    assert [rq.block_values(t) for t in (rq.Q4_0, rq.Q8_0, rq.Q4_K, rq.Q6_K, 99)] == [32, 32, 256, 256, 0]
    assert [rq.block_bytes(t) for t in (rq.Q4_0, rq.Q8_0, rq.Q4_K, rq.Q6_K, 99)] == [18, 34, 144, 210, 0]
    lib = rq.load_library()
    out = ctypes.c_void_p()
    assert lib.rq_init(0, None) == -1 and b"null" in lib.rq_last_error()
    # no device here, or an out-of-range one: a status, never an abort
    assert lib.rq_init(10_000, ctypes.byref(out)) < 0 and out.value is None
    assert len(lib.rq_last_error()) > 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import recipe_dev_b200.capi as capi

    monkeypatch.setattr(capi, "_LIB", None)
    monkeypatch.setattr(capi, "_PKG", tmp_path)
    try:
        capi.load_library()
    except capi.RqError as e:
        assert "no CPU fallback" in str(e)
    else:
        raise AssertionError("loading a missing library must raise")
