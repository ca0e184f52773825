"""The multi-rank host logic on CPU: two gloo ranks shard rows, each computes its shard,
the shards are gathered, and timings are reduced with max -- as the benchmark does with
NCCL on GPUs.  The per-shard product here is numpy: this test is about the sharding."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hodu_b200.dist import all_gather_rows, shard_range, shard_rows


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, total_rows, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        a = torch.randn(total_rows, 24, generator=g)
        b = torch.randn(24, 10, generator=g)           # replicated on every rank
        local = shard_rows(a, rank, world) @ b          # no collective on the compute path
        lo, hi = shard_range(total_rows, rank, world)
        assert local.shape[0] == hi - lo
        full = all_gather_rows(local, total_rows)
        assert torch.allclose(full, a @ b, atol=1e-5)
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)        # step time = slowest rank
        assert t.item() == float(world)
        units = torch.tensor([float(hi - lo)])
        dist.all_reduce(units, op=dist.ReduceOp.SUM)    # whole-job units
        assert units.item() == float(total_rows)
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total_rows", [16, 17, 1])
def test_two_ranks_shard_gather(tmp_path, total_rows):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), total_rows, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
