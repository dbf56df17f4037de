"""A bounded device-side wait that runs out: error status, no hang, the library stays usable.

The fused sum + exchange kernel waits for its peers' partials for a limited time (tuning key
"exchange_wait_ms").  Here nothing ever writes the peer's slot: a two-rank exchange is set up
inside ONE process on one GPU -- the second rank's buffer is simply a second allocation -- and
only rank 0 launches.  Its kernel sends, waits 20 ms, gives up, writes NaN and raises the
device-error flag; the next ordinary call works.  Nothing faults or hangs.
"""
import ctypes as C
import math

import pytest

pytestmark = pytest.mark.gpu


def _two_rank_contexts_on_one_gpu(fdl):
    lib = fdl.lib()
    ctxs = []
    for rank in range(2):
        ctx = C.c_void_p()
        fdl.check(lib.fdl_exchange_create(2, rank, C.byref(ctx)), "fdl_exchange_create")
        ctxs.append(ctx)
    bufs = (C.c_void_p * 2)()
    for rank in range(2):
        p = C.c_void_p()
        fdl.check(lib.fdl_exchange_buffer(ctxs[rank], C.byref(p)), "fdl_exchange_buffer")
        bufs[rank] = p.value
    for rank in range(2):
        fdl.check(lib.fdl_exchange_connect_pointers(ctxs[rank], bufs), "fdl_exchange_connect_pointers")
    return ctxs


def test_exchange_wait_runs_out_and_reports(fdl, cuda):
    lib = fdl.lib()
    cuda.cuda.synchronize()
    fdl.lib().fdl_take_device_error()  # start from a clear flag
    ctxs = _two_rank_contexts_on_one_gpu(fdl)
    x = cuda.ones(1 << 20, dtype=cuda.float32, device="cuda")
    out32 = cuda.zeros(1, dtype=cuda.float32, device="cuda")
    out64 = cuda.zeros(1, dtype=cuda.float64, device="cuda")
    fdl.set_tuning("exchange_wait_ms", 20)
    try:
        fdl.check(lib.fdl_sum_allreduce_f32(x.data_ptr(), x.numel(), out32.data_ptr(), out64.data_ptr(), ctxs[0], None, 0,
                                            None), "fdl_sum_allreduce_f32")
        cuda.cuda.synchronize()  # returns: the wait gave up after ~20 ms
        assert math.isnan(out32.item()) and math.isnan(out64.item())
        assert lib.fdl_take_device_error() == -4          # FDL_ERR_DEVICE_WAIT, reported once
        assert lib.fdl_take_device_error() == 0
        # the arrival counter was left at zero: ordinary sums on the same workspace are correct
        s32, s64 = fdl.full_sum(x, want_f64=True)
        assert s64.item() == float(1 << 20) and s32.item() == float(1 << 20)
        # the column exchange gives up the same way
        m = cuda.ones((4096, 256), dtype=cuda.float32, device="cuda")
        col = cuda.zeros(256, dtype=cuda.float32, device="cuda")
        fdl.check(lib.fdl_reduce_cols_allreduce_f32(m.data_ptr(), 4096, 256, col.data_ptr(), fdl.REDUCE_SUM, 1.0, ctxs[0],
                                                    None, 0, None), "fdl_reduce_cols_allreduce_f32")
        cuda.cuda.synchronize()
        assert bool(cuda.isnan(col).all())
        assert lib.fdl_take_device_error() == -4
        assert to_list(fdl.reduce_cols(m, fdl.REDUCE_SUM)) == [4096.0] * 256
    finally:
        fdl.set_tuning("exchange_wait_ms", 2000)
        for ctx in ctxs:
            lib.fdl_exchange_destroy(ctx)
    assert lib.fdl_take_device_error() == 0


def to_list(t):
    return t.detach().cpu().tolist()


def test_pointer_connection_is_validated(fdl, cuda):
    lib = fdl.lib()
    ctx = C.c_void_p()
    fdl.check(lib.fdl_exchange_create(2, 0, C.byref(ctx)), "fdl_exchange_create")
    try:
        bufs = (C.c_void_p * 2)()
        assert lib.fdl_exchange_connect_pointers(ctx, bufs) == -1          # null entries
        own = C.c_void_p()
        fdl.check(lib.fdl_exchange_buffer(ctx, C.byref(own)), "fdl_exchange_buffer")
        bufs[0], bufs[1] = own.value + 256, own.value
        assert lib.fdl_exchange_connect_pointers(ctx, bufs) == -1          # entry [rank] must be the context's own buffer
        x = cuda.ones(16, dtype=cuda.float32, device="cuda")
        out = cuda.zeros(1, dtype=cuda.float32, device="cuda")
        # not connected yet: the collective is refused on the host
        assert lib.fdl_sum_allreduce_f32(x.data_ptr(), 16, out.data_ptr(), None, ctx, None, 0, None) == -1
    finally:
        lib.fdl_exchange_destroy(ctx)
