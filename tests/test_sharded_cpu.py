"""The multi-GPU host logic on CPU: two gloo ranks split the LM-head rows and the experts, compute
their shares with the CPU oracle (test infrastructure) and exchange; the results equal the
unsharded oracle. No GPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from recipe_dev_b200 import sharded
from tests import oracle_lib as ol


def test_shard_range_partitions_exactly():
    for total in (1, 7, 256, 262144, 1000):
        for world in (1, 2, 3, 4, 8):
            spans = [sharded.shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == total
            for (a, ca), (b, _) in zip(spans, spans[1:]):
                assert a + ca == b
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        sharded.shard_range(10, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, rows, cols, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        o = ol.load()
        # ---- row-split head: uneven rows on purpose
        t = ol.Q6_K
        blocks = o.quantize(t, o.normal(51, 0, rows * cols, 0.02)).reshape(rows, -1)
        x = o.normal(51, 1, 2 * cols, 1.0).reshape(2, cols)
        first, count = sharded.shard_range(rows, world, rank)

        def head(xin):
            return torch.from_numpy(o.matvec(t, blocks[first:first + count].reshape(-1), count, cols, xin, ol.FLOAT_RUN, threads=2))

        logits = sharded.ShardedHead(rows, head, dist, world, rank)(x).numpy()
        full = o.matvec(t, blocks.reshape(-1), rows, cols, x, ol.FLOAT_RUN, threads=2)
        assert np.array_equal(logits.view(np.uint32), full.view(np.uint32))
        # ---- expert-parallel bank
        experts, top, hidden, ffn, tokens = 6, 2, 256, 256, 3
        te = ol.Q4_K
        gate = o.quantize(te, o.normal(52, 1, experts * ffn * hidden, 0.05)).reshape(experts, -1)
        up = o.quantize(te, o.normal(52, 2, experts * ffn * hidden, 0.05)).reshape(experts, -1)
        down = o.quantize(te, o.normal(52, 3, experts * hidden * ffn, 0.05)).reshape(experts, -1)
        sh = (o.quantize(te, o.normal(52, 4, ffn * hidden, 0.05)), o.quantize(te, o.normal(52, 5, ffn * hidden, 0.05)),
              o.quantize(te, o.normal(52, 6, hidden * ffn, 0.05)), o.normal(52, 7, hidden, 0.05))
        xm = o.normal(52, 8, hidden * tokens, 1.0).reshape(hidden, tokens)
        routing = o.topk(o.normal(52, 9, experts * tokens, 1.0).reshape(experts, tokens), top, 0, True)
        ef, ec = sharded.shard_range(experts, world, rank)

        def bank(xin, r, include_shared):
            local = np.ascontiguousarray(r[ef:ef + ec])
            y = o.moe_forward(te, gate[ef:ef + ec].reshape(-1), up[ef:ef + ec].reshape(-1), down[ef:ef + ec].reshape(-1), ec, top, hidden, ffn, xin, local,
                              shared=sh if include_shared else None, threads=2)
            return torch.from_numpy(y)

        y = sharded.ShardedExperts(experts, bank, dist, world, rank)(xm, routing).numpy()
        want = o.moe_forward(te, gate.reshape(-1), up.reshape(-1), down.reshape(-1), experts, top, hidden, ffn, xm, routing, shared=sh, threads=2)
        assert np.max(np.abs(y - want)) <= 1e-5 * np.max(np.abs(want))
        loads = sharded.routed_bytes_per_rank(routing, experts, world, 1000)
        assert sum(loads) == top * tokens * 1000
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_head_and_experts_over_gloo(tmp_path, world):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, 37, 512, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
