"""The C++ host mirror of recipe's block API (include/recipe_rq.hpp) built with g++ against
librq_b200.so and the CPU oracle, then run on the GPU."""
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def build(tmp: Path) -> Path:
    from recipe_dev_b200 import build as rq_build
    from tests import oracle_lib

    lib = rq_build.build()
    oracle_lib.build()
    exe = tmp / "host_mirror_test"
    cmd = ["g++", "-std=c++17", "-O1", f"-I{ROOT / 'include'}", f"-I{ROOT / 'oracle'}", "-I/usr/local/cuda/include", str(ROOT / "tests/cpp/host_mirror_test.cpp"),
           "-o", str(exe), f"-L{lib.parent}", "-lrq_b200", f"-L{ROOT / 'oracle'}", "-lrq_oracle", "-L/usr/local/cuda/lib64", "-lcudart",
           f"-Wl,-rpath,{lib.parent}", f"-Wl,-rpath,{ROOT / 'oracle'}", "-Wl,-rpath,/usr/local/cuda/lib64"]
    subprocess.run(cmd, check=True)
    return exe


def test_host_mirror_compiles(tmp_path):
    """No GPU needed: the header and the C ABI agree (it compiles and links)."""
    assert build(tmp_path).exists()


@pytest.mark.gpu
def test_host_mirror_runs(tmp_path):
    out = subprocess.run([str(build(tmp_path))], capture_output=True, text=True, timeout=300)
    sys.stdout.write(out.stdout + out.stderr)
    assert out.returncode == 0 and out.stdout.startswith("ok")
