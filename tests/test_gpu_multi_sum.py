"""Two GPUs: the fused sum + exchange kernel against per-GPU sums added on the host.
Skipped on boxes with a single GPU.  Ranks are separate processes (one per GPU); the
64-byte IPC handles travel over a gloo group."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, n, out):
    import torch.distributed as dist
    from fast_dl_b200 import capi
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.cuda.set_device(rank)
        capi.lib()
        capi.use_device(rank)

        def gather(handle):
            handles = [None] * world
            dist.all_gather_object(handles, handle)
            return handles

        ex = capi.Exchange(world, rank, gather)
        dist.barrier()
        rng = np.random.default_rng(100 + rank)
        x = torch.from_numpy(rng.uniform(-1, 1, n).astype(np.float32)).cuda()
        local64 = capi.full_sum(x, want_f64=True)[1].cpu()
        parts = [torch.zeros(1, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(parts, local64)
        want = sum(p.item() for p in parts)  # rank order, like the kernel
        o32 = torch.zeros(1, dtype=torch.float32, device="cuda")
        o64 = torch.zeros(1, dtype=torch.float64, device="cuda")
        results = []
        for _ in range(5):  # consecutive epochs reuse the two parities
            ex.sum(x, o32, o64)
            torch.cuda.synchronize()
            results.append(o64.item())
        capi.take_device_error()
        dist.barrier()
        ex.close()
        ok = all(r == want for r in results) and np.float32(want) == o32.item()
        gathered = [None] * world
        dist.all_gather_object(gathered, (ok, results[0]))
        if rank == 0:
            out.put((all(g[0] for g in gathered), len({g[1] for g in gathered}) == 1))
    finally:
        dist.destroy_process_group()


def test_fused_sum_exchange_two_gpus(cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    mp.spawn(_worker, args=(2, port, (1 << 22) + 3, out), nprocs=2, join=True)
    all_ok, same_bits = out.get()
    assert all_ok and same_bits
