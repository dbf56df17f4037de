"""Multi-rank host logic on CPU: shard arithmetic and the exchange protocol over gloo
(world size 2 and 3), with the oracle as the shard-local compute."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fast_dl_b200.sharding import RowSharded, shard_rows


@pytest.mark.parametrize("total,world", [(16384, 1), (16384, 2), (16384, 8), (10, 3), (7, 8), (0, 4)])
def test_shards_tile_the_rows(total, world):
    shards = [shard_rows(total, world, r) for r in range(world)]
    assert sum(s.count for s in shards) == total
    assert shards[0].start == 0
    for a, b in zip(shards, shards[1:]):
        assert a.start + a.count == b.start
    assert max(s.count for s in shards) - min(s.count for s in shards) <= 1


def test_bad_requests_are_rejected():
    for args in [(10, 0, 0), (10, 2, 2), (10, 2, -1), (-1, 2, 0)]:
        with pytest.raises(ValueError):
            shard_rows(*args)


class OracleLocal:
    """CPU stand-in for the CUDA kernels: the oracle, same signatures."""

    def full_sum_f64(self, x):
        from oracle import oracle as orc
        return torch.tensor([orc.full_sum(x.numpy())], dtype=torch.float64)

    def col_sums(self, x2d, global_rows):
        from oracle import oracle as orc
        return torch.from_numpy(orc.reduce_cols(x2d.numpy(), 1, mean_divisor=global_rows))


def _worker(rank, world, port, total, cols, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = np.random.default_rng(42).normal(size=(total, cols)).astype(np.float32)
        sh = shard_rows(total, world, rank)
        mine = torch.from_numpy(full[sh.start:sh.start + sh.count].copy())
        ops = RowSharded(sh, local=OracleLocal())
        s = ops.full_sum(mine)
        m = ops.mean_axis0(mine)
        ok_sum = abs(s.item() - full.astype(np.float64).sum()) <= 1e-9 * np.sqrt((full.astype(np.float64) ** 2).sum())
        ok_mean = np.allclose(m.numpy(), full.astype(np.float64).mean(axis=0), rtol=1e-5, atol=1e-6)
        if rank == 0:
            out.put((bool(ok_sum), bool(ok_mean)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,total", [(2, 1000), (3, 10)])
def test_full_sum_and_axis0_mean_over_gloo(world, total):
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    mp.spawn(_worker, args=(world, _free_port(), total, 33, out), nprocs=world, join=True)
    assert out.get() == (True, True)
