"""One rank of the multi-GPU exchange test. Launched by tests/test_gpu_multi.py as
`python -m torch.distributed.run --nproc-per-node N tests/multi/exchange_worker.py`, one process per GPU.

Checks, on real GPUs over NVLink peer memory and over NCCL, through the C ABI:
  * rq_exchange_gather / rq_exchange_reduce against values every rank can compute by itself, over several calls
    (both halves of the double-buffered slots) and replayed from a CUDA graph;
  * rq_allgather_rows / rq_allreduce_sum through a communicator made by rq_nccl_comm_create;
  * the row-split matvec + gather and the expert-parallel bank + rank-order sum against the CPU oracle (rank 0).
A rank leaves only between steps, with nothing in flight."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

import recipe_dev_b200 as rq  # noqa: E402
from recipe_dev_b200 import sharded  # noqa: E402
from tests import oracle_lib as ol  # noqa: E402


def rel_err(y, ref):
    y, ref = np.asarray(y, np.float64), np.asarray(ref, np.float64)
    floor = 1e-3 * np.max(np.abs(ref))
    return float(np.max(np.abs(y - ref) / np.maximum(np.abs(ref), floor)))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")  # the host-side channel: handles and ids travel over it, never tensors of the data path
    dev = f"cuda:{local}"
    ctx = rq.Context(local)
    ctx.set_wait_limit(5_000_000_000)
    oracle = ol.load()

    def share(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    # ---- the library's own exchange
    count = 50_000
    ex = rq.Exchange(ctx, rank, world, count * 4)
    ex.connect(share(ex.ipc_handle()))
    dist.barrier()
    gathered = torch.empty(world, count, device=dev)
    summed = torch.empty(count, device=dev)
    base = torch.arange(count, device=dev, dtype=torch.float32)
    for call in range(5):
        mine = base * (rank + 1) + call
        ex.gather(mine, gathered)
        ex.reduce(mine * 0.5, summed)
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.equal(gathered[r], base * (r + 1) + call), (rank, call, r)
        want = torch.zeros(count, device=dev)
        for r in range(world):  # rank order, as the kernel adds
            want += (base * (r + 1) + call) * 0.5
        assert torch.equal(summed, want), (rank, call)
    ctx.check()
    # odd counts take the scalar path; a CUDA graph of exchanges is replayed
    odd = torch.full((777,), float(rank + 1), device=dev)
    odd_out = torch.empty(world, 777, device=dev)
    ex.gather(odd, odd_out)
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            ex.gather(odd, odd_out, stream=side)
            ex.reduce(odd, summed[:777], stream=side)
            ex.gather(odd * 2, odd_out, stream=side)
    for _ in range(4):
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(odd_out, torch.arange(1, world + 1, device=dev, dtype=torch.float32)[:, None].expand(world, 777) * 2)
    assert torch.equal(summed[:777], torch.full((777,), float(world * (world + 1) // 2), device=dev))
    ctx.check()
    dist.barrier()

    # ---- NCCL through the C ABI
    ids = share(rq.NcclComm.unique_id() if rank == 0 else None)
    comm = rq.NcclComm.create(ctx, ids[0], world, rank)
    mine = base * (rank + 1)
    comm.allgather_rows(mine, gathered)
    comm.allreduce_sum(mine, summed)
    torch.cuda.synchronize()
    for r in range(world):
        assert torch.equal(gathered[r], base * (r + 1))
    assert torch.allclose(summed, base * (world * (world + 1) // 2))
    dist.barrier()

    # ---- row-split matvec + gather against the oracle
    t, rows, cols = ol.Q6_K, 64 * world * 3, 2560
    blocks = oracle.quantize(t, oracle.normal(71, 0, rows * cols, 0.02))  # the same table on every rank
    x = oracle.normal(71, 1, cols, 1.0)
    first, cnt = sharded.shard_range(rows, world, rank)
    w = ctx.weight_from_host(t, blocks, rows, cols, row_first=first, row_count=cnt)
    xd = torch.from_numpy(x).to(dev)
    local_y = ctx.matvec(w, xd, act_mode=rq.ACT_INT8, step=32)
    exh = rq.Exchange(ctx, rank, world, cnt * 4)
    exh.connect(share(exh.ipc_handle()))
    logits = torch.empty(world, cnt, device=dev)
    exh.gather(local_y, logits)
    torch.cuda.synchronize()
    ref = oracle.matvec(t, blocks, rows, cols, x, ol.INT8, 32)
    assert rel_err(logits.reshape(-1).cpu().numpy(), ref) <= 1e-3
    logits2 = torch.empty(world, cnt, device=dev)
    comm.allgather_rows(local_y, logits2)
    torch.cuda.synchronize()
    assert torch.equal(logits, logits2)

    # ---- expert-parallel bank + rank-order sum against the oracle
    experts, top, hidden, ffn, tokens = 8 * world, 4, 512, 256, 3
    tk = ol.Q4_K
    gate = oracle.quantize(tk, oracle.normal(72, 0, experts * ffn * hidden, 0.02))
    up = oracle.quantize(tk, oracle.normal(72, 1, experts * ffn * hidden, 0.02))
    down = oracle.quantize(tk, oracle.normal(72, 2, experts * hidden * ffn, 0.02))
    shared_e = (oracle.quantize(tk, oracle.normal(72, 3, ffn * hidden, 0.02)), oracle.quantize(tk, oracle.normal(72, 4, ffn * hidden, 0.02)),
                oracle.quantize(tk, oracle.normal(72, 5, hidden * ffn, 0.02)), oracle.normal(72, 6, hidden, 0.02))
    scores = oracle.normal(72, 7, experts * tokens, 1.0).reshape(experts, tokens)
    xm = oracle.normal(72, 8, hidden * tokens, 1.0).reshape(hidden, tokens)
    ef, ec = sharded.shard_range(experts, world, rank)
    bank = ctx.moe_prepare(tk, gate, up, down, experts, hidden, ffn, expert_first=ef, expert_count=ec, shared=shared_e if rank == 0 else None)
    routing = ctx.moe_route(torch.from_numpy(scores).to(dev), top)
    part = ctx.moe_forward(bank, torch.from_numpy(xm).to(dev), routing, top, include_shared=(rank == 0))
    exm = rq.Exchange(ctx, rank, world, hidden * tokens * 4)
    exm.connect(share(exm.ipc_handle()))
    total = torch.empty(hidden * tokens, device=dev)
    exm.reduce(part.contiguous().reshape(-1), total)
    torch.cuda.synchronize()
    ref = oracle.moe_forward(tk, gate, up, down, experts, top, hidden, ffn, xm, oracle.topk(scores, top, 0, True), shared=shared_e)
    assert rel_err(total.reshape(hidden, tokens).cpu().numpy(), ref) <= 1e-3
    every = share(total.cpu().numpy().tobytes())
    assert all(e == every[0] for e in every), "the ranks' sums differ in bits"
    ctx.check()
    dist.barrier()
    torch.cuda.synchronize()
    for e in (ex, exh, exm):
        e.free()
    comm.destroy()
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: exchange ok", flush=True)


if __name__ == "__main__":
    main()
