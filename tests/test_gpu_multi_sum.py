"""Two GPUs: the fused sum + exchange and column-reduction + exchange kernels against
per-GPU results combined on the host.
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
        # the same exchange in two halves, with other work on the stream in between, mixed
        # with the one-call form (the epochs and parities are shared)
        other = torch.from_numpy(rng.uniform(-1, 1, n).astype(np.float32)).cuda()
        for k in range(6):
            o64.zero_()
            ex.sum_start(x)
            capi.binary(other, x, capi.ADD)           # overlaps the exchange
            if k == 2:
                try:                                    # a second start before the finish is refused
                    ex.sum_start(x)
                    results.append(float("nan"))
                except capi.FdlError:
                    pass
            ex.sum_finish(o32, o64)
            torch.cuda.synchronize()
            results.append(o64.item())
            if k % 2:
                ex.sum(x, o32, o64)
                torch.cuda.synchronize()
                results.append(o64.item())
        try:                                            # a finish with nothing started is refused
            ex.sum_finish(o32, o64)
            results.append(float("nan"))
        except capi.FdlError:
            pass
        # column reductions with the exchange in the kernel: mean over ALL rows of the stacked
        # [world * rows, cols] matrix, and the column maxima
        cols_ok = True
        for rows, cols in ((300, 256), (1000, 8192), (64, 36), (5000, 65536)):
            shard = torch.from_numpy(rng.normal(size=(rows, cols)).astype(np.float32)).cuda()
            local_sum = shard.double().sum(dim=0).cpu()
            local_max = shard.max(dim=0).values.cpu()
            sums = [torch.zeros(cols, dtype=torch.float64) for _ in range(world)]
            maxs = [torch.zeros(cols, dtype=torch.float32) for _ in range(world)]
            dist.all_gather(sums, local_sum)
            dist.all_gather(maxs, local_max)
            want_mean = (sum(sums) / (world * rows)).numpy()
            want_max = torch.stack(maxs).max(dim=0).values.numpy()
            res = torch.empty(cols, dtype=torch.float32, device="cuda")
            for _ in range(3):
                ex.reduce_cols(shard, capi.REDUCE_MEAN, world * rows, res)
                torch.cuda.synchronize()
                got = res.cpu().numpy()
                good = bool(np.allclose(got, want_mean, rtol=1e-5, atol=1e-6))
                if not good:
                    print(f"rank {rank}: mean [{rows},{cols}] max abs err {np.abs(got - want_mean).max():.3e}", flush=True)
                cols_ok &= good
            ex.reduce_cols(shard, capi.REDUCE_MAX, 1, res)
            torch.cuda.synchronize()
            good = bool(np.array_equal(res.cpu().numpy(), want_max))
            if not good:
                print(f"rank {rank}: max [{rows},{cols}] differs in {(res.cpu().numpy() != want_max).sum()} columns", flush=True)
            cols_ok &= good
            gathered_out = [torch.zeros(cols) for _ in range(world)]
            dist.all_gather(gathered_out, res.cpu())
            good = all(torch.equal(g, gathered_out[0]) for g in gathered_out)   # same bits on every rank
            if not good:
                print(f"rank {rank}: [{rows},{cols}] ranks disagree", flush=True)
            cols_ok &= good
        capi.take_device_error()
        dist.barrier()
        final32 = o32.item()
        # Last, a collective that one rank never joins: rank 1 stays alive but skips the call.
        # Rank 0's kernel waits 50 ms for the missing partial, gives up, writes NaN and raises
        # the device-error flag; an ordinary sum afterwards is correct.  (The contexts' epochs
        # are out of step after this, so they are closed right away.)
        timeout_ok = True
        if rank == 0:
            capi.set_tuning("exchange_wait_ms", 50)
            ex.sum(x, o32, o64)
            torch.cuda.synchronize()
            timeout_ok = bool(np.isnan(o64.item())) and capi.lib().fdl_take_device_error() == -4 \
                and capi.lib().fdl_take_device_error() == 0
            timeout_ok &= capi.full_sum(x, want_f64=True)[1].item() == local64.item()
            capi.set_tuning("exchange_wait_ms", 2000)
            if not timeout_ok:
                print("rank 0: the bounded wait did not report as expected", flush=True)
        dist.barrier()
        ex.close()
        sum_ok = all(r == want for r in results) and np.float32(want) == final32 and timeout_ok
        if not sum_ok:
            print(f"rank {rank}: sum results {results} want {want}", flush=True)
        ok = sum_ok and cols_ok
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
