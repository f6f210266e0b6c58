"""The multi-GPU exchange on real GPUs: one child process per GPU (2, or 4 where the box has them), NVLS off, plain peer
stores in the library's own kernel. Skipped on a single-GPU box; the partition logic is covered on CPU over gloo."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_exchange_across_gpus():
    import torch

    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 4 if n >= 4 else 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", "29517",
           str(ROOT / "tests" / "multi" / "exchange_worker.py")]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + "\n" + proc.stderr[-3000:]
    assert proc.stdout.count("exchange ok") == world


def test_exchange_of_one_rank_on_one_gpu(rq_ctx):
    """The exchange entry points with a single rank (nothing to wait for: no kernel here waits on another launch): the slot
    and call-count bookkeeping, odd and 16-byte-aligned sizes, repeated calls, replay from a CUDA graph, argument checks."""
    import torch

    import recipe_dev_b200 as rq

    two = rq.Exchange(rq_ctx, 0, 2, 4096 * 4)  # a rank of two that never met its peer: the call is refused, nothing is launched
    with pytest.raises(rq.RqError, match="not connected"):
        two.gather(torch.zeros(8, device="cuda"), torch.zeros(2, 8, device="cuda"))
    two.free()
    ex = rq.Exchange(rq_ctx, 0, 1, 4096 * 4)  # a single rank has nobody to connect to
    ex.connect_same_process([ex])
    gen = torch.Generator(device="cuda")
    gen.manual_seed(12)
    for count in (4096, 1001, 3):
        for call in range(3):  # both halves of the buffer, more than once
            src = torch.randn(count, generator=gen, device="cuda")
            out = torch.empty(1, count, device="cuda")
            red = torch.empty(count, device="cuda")
            ex.gather(src, out)
            ex.reduce(src, red)
            torch.cuda.synchronize()
            assert torch.equal(out[0], src) and torch.equal(red, src)
    with pytest.raises(rq.RqError):
        ex.gather(torch.zeros(5000, device="cuda"), torch.zeros(1, 5000, device="cuda"))  # beyond the slot
    src = torch.randn(2048, generator=gen, device="cuda")
    out = torch.empty(1, 2048, device="cuda")
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        ex.gather(src, out, stream=stream.cuda_stream)  # warm: nothing lazy inside the capture
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            ex.gather(src, out, stream=stream.cuda_stream)
            ex.reduce(out[0], src, stream=stream.cuda_stream)
    want = src.clone()
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out[0], want) and torch.equal(src, want)
    rq_ctx.check()
    ex.free()
