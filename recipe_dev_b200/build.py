"""Builds librq_b200.so (hand-written CUDA for sm_100a + the C ABI) in-tree with nvcc.

Run as ``python -m recipe_dev_b200.build``. The library is written next to this file so
that it travels with the source tree; nothing is installed into site-packages.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "librq_b200.so"
OBJ = PKG / "build"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", f"-I{ROOT / 'include'}", f"-I{CSRC}"]
# per-file extras: the weight quantisers must not contract a*b+c into one rounding
EXTRA = {"rq_quantize.cu": ["--fmad=false"]}


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: librq_b200.so cannot be built")
    return found


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def stale() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.glob("*")) + [ROOT / "include" / "rq.h", Path(__file__)])
    return newest > LIB.stat().st_mtime


def _compile(src: Path, verbose: bool) -> Path:
    obj = OBJ / (src.stem + ".o")
    cmd = [nvcc(), *ARCH, *COMMON, *EXTRA.get(src.name, []), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        sys.stderr.write(proc.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    OBJ.mkdir(exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), sources()))
    cmd = [nvcc(), *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
