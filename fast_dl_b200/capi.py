"""ctypes binding of libfdl_kernels.so -- the same C ABI a cgo/JNI/C++ caller would bind.

This module is harness plumbing for the Python tests and bench: it declares the
prototypes of include/fdl_kernels.h, loads the in-tree library, and offers thin helpers
that take torch CUDA tensors (used only as device-memory handles: `data_ptr()` and the
current stream).  There is no fallback: if the library is missing or a call fails, an
exception is raised.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import build as _build

ADD, SUB, MUL, DIV = 0, 1, 2, 3
RELU, LEAKY_RELU, GELU, SIGMOID, TANH = 0, 1, 2, 3, 4
REDUCE_SUM, REDUCE_MEAN, REDUCE_MAX = 0, 1, 2
TREE_INTERLEAVE, TREE_ADDRESS = 0, 1

_vp, _i64, _int, _f32, _f64, _sz = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_double, C.c_size_t
_pi64 = C.POINTER(C.c_int64)

# name -> (restype, argtypes); must list every symbol include/fdl_kernels.h declares.
PROTOTYPES = {
    "fdl_version": (_int, []),
    "fdl_error_string": (C.c_char_p, [_int]),
    "fdl_device_count": (_int, []),
    "fdl_set_device": (_int, [_int]),
    "fdl_stream_synchronize": (_int, [_vp]),
    "fdl_take_device_error": (_int, []),
    "fdl_set_tuning": (_int, [C.c_char_p, _int]),
    "fdl_debug_sum_trace": (_int, [C.POINTER(C.c_uint64)]),
    "fdl_binary_f32": (_int, [_vp, _vp, _vp, _i64, _int, _vp]),
    "fdl_unary_f32": (_int, [_vp, _vp, _i64, _int, _f32, _vp]),
    "fdl_mul_add_relu_f32": (_int, [_vp, _vp, _vp, _vp, _i64, _vp]),
    "fdl_add_row_bias_f32": (_int, [_vp, _vp, _i64, _i64, _vp]),
    "fdl_add_row_bias_relu_f32": (_int, [_vp, _vp, _i64, _i64, _vp]),
    "fdl_broadcast_binary_f32": (_int, [_vp, _vp, _vp, _int, _pi64, _pi64, _pi64, _int, _vp]),
    "fdl_block_reduce_1024_f32": (_int, [_vp, _vp, _i64, _int, _vp]),
    "fdl_sum_scratch_bytes": (_sz, [_i64]),
    "fdl_reduce_cols_scratch_bytes": (_sz, [_i64, _i64, _i64]),
    "fdl_sum_f32": (_int, [_vp, _i64, _vp, _vp, _vp, _sz, _vp]),
    "fdl_sum_f32_static": (_int, [_vp, _i64, _vp, _vp, _vp]),
    "fdl_debug_split_ticket": (_int, [_i64, _i64, _i64, C.c_uint, C.POINTER(C.c_int64), C.POINTER(C.c_int),
                                      C.POINTER(C.c_int)]),
    "fdl_exchange_create": (_int, [_int, _int, C.POINTER(C.c_void_p)]),
    "fdl_exchange_local_handle": (_int, [_vp, C.c_char_p]),
    "fdl_exchange_connect": (_int, [_vp, C.c_char_p]),
    "fdl_exchange_buffer": (_int, [_vp, C.POINTER(C.c_void_p)]),
    "fdl_exchange_connect_pointers": (_int, [_vp, C.POINTER(C.c_void_p)]),
    "fdl_exchange_destroy": (_int, [_vp]),
    "fdl_sum_allreduce_f32": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _sz, _vp]),
    "fdl_sum_allreduce_start_f32": (_int, [_vp, _i64, _vp, _vp, _sz, _vp]),
    "fdl_sum_allreduce_finish_f32": (_int, [_vp, _vp, _vp, _vp]),
    "fdl_reduce_cols_allreduce_f32": (_int, [_vp, _i64, _i64, _vp, _int, _f64, _vp, _vp, _sz, _vp]),
    "fdl_reduce_rows_f32": (_int, [_vp, _i64, _i64, _vp, _int, _vp]),
    "fdl_argmax_rows_f32": (_int, [_vp, _i64, _i64, _vp, _vp]),
    "fdl_reduce_cols_f32": (_int, [_vp, _i64, _i64, _i64, _vp, _int, _f64, _vp, _sz, _vp]),
    "fdl_softmax_rows_f32": (_int, [_vp, _vp, _i64, _i64, _vp]),
    "fdl_layernorm_rows_f32": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _f32, _vp]),
    "fdl_cross_entropy_f32": (_int, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "fdl_transpose_f32": (_int, [_vp, _vp, _i64, _vp]),
    "fdl_uniform_f32": (_int, [_vp, _i64, _f32, _f32, C.c_uint64, _vp]),
    "fdl_normal_f32": (_int, [_vp, _i64, _f32, _f32, C.c_uint64, _vp]),
    "fdl_host_binary_f32": (_int, [_vp, _vp, _vp, _i64, _int]),
    "fdl_host_unary_f32": (_int, [_vp, _vp, _i64, _int, _f32]),
    "fdl_host_mul_add_relu_f32": (_int, [_vp, _vp, _vp, _vp, _i64]),
    "fdl_host_row_broadcast_f32": (_int, [_vp, _vp, _vp, _i64, _i64, _int]),
    "fdl_host_sum_f32": (_int, [_vp, _i64, C.POINTER(C.c_double)]),
    "fdl_host_sweep_f32": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, C.POINTER(C.c_double)]),
}


class FdlError(RuntimeError):
    def __init__(self, status: int, text: str, where: str):
        super().__init__(f"{where}: {text} (status {status})")
        self.status = status


_lib = None


def library_path() -> Path:
    return _build.kernels_lib_path()


def lib() -> C.CDLL:
    """The loaded library with prototypes attached.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        path = library_path()
        if not path.exists():
            raise FileNotFoundError(
                f"{path} is missing: run `python -m fast_dl_b200.build` (there is no fallback path)")
        handle = C.CDLL(str(path))
        for name, (restype, argtypes) in PROTOTYPES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int, where: str) -> None:
    if status != 0:
        raise FdlError(status, lib().fdl_error_string(status).decode(), where)


# ---- torch-tensor conveniences -------------------------------------------------------------


def _stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


def _require(t, dtype=None):
    import torch
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("expected a contiguous CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"expected dtype {dtype}, got {t.dtype}")
    return t


def set_tuning(key: str, value: int) -> None:
    check(lib().fdl_set_tuning(key.encode(), value), f"fdl_set_tuning({key})")


def use_device(index: int) -> None:
    check(lib().fdl_set_device(index), "fdl_set_device")


def binary(a, b, op, out=None):
    import torch
    _require(a, torch.float32), _require(b, torch.float32)
    if a.numel() != b.numel():
        raise ValueError("binary: operands differ in size")
    out = torch.empty_like(a) if out is None else out
    check(lib().fdl_binary_f32(_ptr(a), _ptr(b), _ptr(out), a.numel(), op, _stream()), "fdl_binary_f32")
    return out


def unary(x, op, alpha=0.01, out=None):
    import torch
    _require(x, torch.float32)
    out = torch.empty_like(x) if out is None else out
    check(lib().fdl_unary_f32(_ptr(x), _ptr(out), x.numel(), op, alpha, _stream()), "fdl_unary_f32")
    return out


def mul_add_relu(a, b, c, out=None):
    import torch
    for t in (a, b, c):
        _require(t, torch.float32)
    out = torch.empty_like(a) if out is None else out
    check(lib().fdl_mul_add_relu_f32(_ptr(a), _ptr(b), _ptr(c), _ptr(out), a.numel(), _stream()),
          "fdl_mul_add_relu_f32")
    return out


def add_row_bias_(out, bias, relu=False):
    rows, cols = out.shape
    fn = lib().fdl_add_row_bias_relu_f32 if relu else lib().fdl_add_row_bias_f32
    check(fn(_ptr(out), _ptr(bias), rows, cols, _stream()), "fdl_add_row_bias_f32")
    return out


def broadcast_strides(shape, out_shape):
    """Element strides of a contiguous tensor of `shape` viewed as `out_shape` (0 = broadcast)."""
    nd = len(out_shape)
    shape = (1,) * (nd - len(shape)) + tuple(shape)
    strides, acc = [0] * nd, 1
    for i in range(nd - 1, -1, -1):
        if shape[i] == 1 and out_shape[i] != 1:
            strides[i] = 0
        elif shape[i] == out_shape[i]:
            strides[i] = acc if shape[i] != 1 else 0
        else:
            raise ValueError(f"shape {shape} does not broadcast to {out_shape}")
        acc *= shape[i]
    return strides


def broadcast_shape(sa, sb):
    nd = max(len(sa), len(sb))
    sa = (1,) * (nd - len(sa)) + tuple(sa)
    sb = (1,) * (nd - len(sb)) + tuple(sb)
    out = []
    for x, y in zip(sa, sb):
        if x != y and x != 1 and y != 1:
            raise ValueError(f"shapes {sa} and {sb} do not broadcast")
        out.append(max(x, y))
    return tuple(out)


def broadcast_binary(a, b, op, out=None):
    import torch
    _require(a, torch.float32), _require(b, torch.float32)
    oshape = broadcast_shape(tuple(a.shape), tuple(b.shape))
    out = torch.empty(oshape, dtype=torch.float32, device=a.device) if out is None else out
    nd = len(oshape)
    arr = C.c_int64 * nd
    check(lib().fdl_broadcast_binary_f32(
        _ptr(a), _ptr(b), _ptr(out), nd, arr(*oshape), arr(*broadcast_strides(a.shape, oshape)),
        arr(*broadcast_strides(b.shape, oshape)), op, _stream()), "fdl_broadcast_binary_f32")
    return out


def block_reduce_1024(x, tree=TREE_ADDRESS):
    import torch
    _require(x, torch.float32)
    out = torch.empty(x.numel() // 1024, dtype=torch.float32, device=x.device)
    check(lib().fdl_block_reduce_1024_f32(_ptr(x), _ptr(out), x.numel(), tree, _stream()),
          "fdl_block_reduce_1024_f32")
    return out


def full_sum(x, want_f64=False, scratch=None):
    import torch
    _require(x, torch.float32)
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    out64 = torch.empty(1, dtype=torch.float64, device=x.device) if want_f64 else None
    check(lib().fdl_sum_f32(_ptr(x), x.numel(), _ptr(out), _ptr(out64), _ptr(scratch),
                            0 if scratch is None else scratch.numel() * scratch.element_size(),
                            _stream()), "fdl_sum_f32")
    return (out, out64) if want_f64 else out


def full_sum_static(x, want_f64=False):
    """fdl_sum_f32_static: the full sum with its scratch in the library's fixed device array."""
    import torch
    _require(x, torch.float32)
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    out64 = torch.empty(1, dtype=torch.float64, device=x.device) if want_f64 else None
    check(lib().fdl_sum_f32_static(_ptr(x), x.numel(), _ptr(out), _ptr(out64), _stream()),
          "fdl_sum_f32_static")
    return (out, out64) if want_f64 else out


def reduce_rows(x, op):
    import torch
    _require(x, torch.float32)
    rows, cols = x.shape
    out = torch.empty(rows, dtype=torch.float32, device=x.device)
    check(lib().fdl_reduce_rows_f32(_ptr(x), rows, cols, _ptr(out), op, _stream()), "fdl_reduce_rows_f32")
    return out


def argmax_rows(x):
    import torch
    _require(x, torch.float32)
    rows, cols = x.shape
    out = torch.empty(rows, dtype=torch.int64, device=x.device)
    check(lib().fdl_argmax_rows_f32(_ptr(x), rows, cols, _ptr(out), _stream()), "fdl_argmax_rows_f32")
    return out


def reduce_cols(x, op, mean_divisor=None, scratch=None):
    """x: [rows, cols] or [batch, rows, cols]; reduces over rows."""
    import torch
    _require(x, torch.float32)
    if x.dim() == 2:
        batch, (rows, cols) = 1, x.shape
        oshape = (cols,)
    else:
        batch, rows, cols = x.shape
        oshape = (batch, cols)
    out = torch.empty(oshape, dtype=torch.float32, device=x.device)
    div = float(rows if mean_divisor is None else mean_divisor)
    check(lib().fdl_reduce_cols_f32(_ptr(x), batch, rows, cols, _ptr(out), op, div, _ptr(scratch),
                                    0 if scratch is None else scratch.numel() * scratch.element_size(),
                                    _stream()), "fdl_reduce_cols_f32")
    return out


def softmax_rows(x, out=None):
    import torch
    _require(x, torch.float32)
    rows, cols = x.shape
    out = torch.empty_like(x) if out is None else out
    check(lib().fdl_softmax_rows_f32(_ptr(x), _ptr(out), rows, cols, _stream()), "fdl_softmax_rows_f32")
    return out


def layernorm_rows(x, gamma=None, beta=None, eps=1e-5, out=None, want_stats=False):
    import torch
    _require(x, torch.float32)
    rows, cols = x.shape
    out = torch.empty_like(x) if out is None else out
    mean = torch.empty(rows, dtype=torch.float32, device=x.device) if want_stats else None
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device) if want_stats else None
    check(lib().fdl_layernorm_rows_f32(_ptr(x), _ptr(gamma), _ptr(beta), _ptr(out), _ptr(mean), _ptr(rstd),
                                       rows, cols, eps, _stream()), "fdl_layernorm_rows_f32")
    return (out, mean, rstd) if want_stats else out


def cross_entropy(logits, labels):
    import torch
    _require(logits, torch.float32), _require(labels, torch.int64)
    batch, classes = logits.shape
    loss = torch.empty(1, dtype=torch.float32, device=logits.device)
    check(lib().fdl_cross_entropy_f32(_ptr(logits), _ptr(labels), _ptr(loss), batch, classes, _stream()),
          "fdl_cross_entropy_f32")
    return loss


def transpose(x):
    import torch
    _require(x, torch.float32)
    out = torch.empty_like(x)
    check(lib().fdl_transpose_f32(_ptr(x), _ptr(out), x.shape[0], _stream()), "fdl_transpose_f32")
    return out


def random_fill(n, normal, p0, p1, seed, device="cuda"):
    import torch
    out = torch.empty(n, dtype=torch.float32, device=device)
    fn = lib().fdl_normal_f32 if normal else lib().fdl_uniform_f32
    check(fn(_ptr(out), n, p0, p1, seed, _stream()), "fdl_random_fill")
    return out


def sum_trace() -> list:
    """The eight words left by the most recent full sum launched with the tuning key sum_trace set."""
    words = (C.c_uint64 * 8)()
    check(lib().fdl_debug_sum_trace(words), "fdl_debug_sum_trace")
    return list(words)


def take_device_error() -> None:
    check(lib().fdl_take_device_error(), "device-side wait")


# ---- host-buffer entry points (torch CPU tensors, ideally pinned) ------------------------------


def host_binary(a, b, out, op):
    check(lib().fdl_host_binary_f32(_ptr(a), _ptr(b), _ptr(out), a.numel(), op), "fdl_host_binary_f32")
    return out


def host_unary(x, out, op, alpha=0.01):
    check(lib().fdl_host_unary_f32(_ptr(x), _ptr(out), x.numel(), op, alpha), "fdl_host_unary_f32")
    return out


def host_mul_add_relu(a, b, c, out):
    check(lib().fdl_host_mul_add_relu_f32(_ptr(a), _ptr(b), _ptr(c), _ptr(out), a.numel()),
          "fdl_host_mul_add_relu_f32")
    return out


def host_row_broadcast(a, row, out, op):
    rows, cols = a.shape
    check(lib().fdl_host_row_broadcast_f32(_ptr(a), _ptr(row), _ptr(out), rows, cols, op),
          "fdl_host_row_broadcast_f32")
    return out


def host_sum(x) -> float:
    res = C.c_double(0.0)
    check(lib().fdl_host_sum_f32(_ptr(x), x.numel(), C.byref(res)), "fdl_host_sum_f32")
    return res.value


def host_sweep(x, y, row, z, w) -> float:
    """z = x + y, w = x + row, returns sum(x); x, y, z, w are [rows, cols] host tensors."""
    rows, cols = x.shape
    res = C.c_double(0.0)
    check(lib().fdl_host_sweep_f32(_ptr(x), _ptr(y), _ptr(row), _ptr(z), _ptr(w), rows, cols, C.byref(res)),
          "fdl_host_sweep_f32")
    return res.value


# ---- cross-GPU exchange for the fused full sum ----------------------------------------------------


class Exchange:
    """Per-process context of fdl_sum_allreduce_f32.  `gather` is a callable that takes this
    rank's 64-byte handle and returns the list of all ranks' handles in rank order (for
    example a wrapper of torch.distributed.all_gather_object)."""

    def __init__(self, world: int, rank: int, gather):
        self.world, self.rank = world, rank
        ctx = C.c_void_p()
        check(lib().fdl_exchange_create(world, rank, C.byref(ctx)), "fdl_exchange_create")
        self.ctx = ctx
        buf = C.create_string_buffer(64)
        check(lib().fdl_exchange_local_handle(self.ctx, buf), "fdl_exchange_local_handle")
        handles = gather(buf.raw)
        if len(handles) != world or any(len(h) != 64 for h in handles):
            raise ValueError("exchange: expected one 64-byte handle per rank")
        check(lib().fdl_exchange_connect(self.ctx, b"".join(handles)), "fdl_exchange_connect")

    def sum(self, x, out32, out64):
        check(lib().fdl_sum_allreduce_f32(_ptr(x), x.numel(), _ptr(out32), _ptr(out64), self.ctx, None, 0,
                                          _stream()), "fdl_sum_allreduce_f32")

    def sum_start(self, x):
        """First half: the sum kernel sends this rank's partial to all ranks and does not wait."""
        check(lib().fdl_sum_allreduce_start_f32(_ptr(x), x.numel(), self.ctx, None, 0, _stream()),
              "fdl_sum_allreduce_start_f32")

    def sum_finish(self, out32, out64):
        """Second half: fold all ranks' partials (rank order) into the outputs."""
        check(lib().fdl_sum_allreduce_finish_f32(_ptr(out32), _ptr(out64), self.ctx, _stream()),
              "fdl_sum_allreduce_finish_f32")

    def reduce_cols(self, x2d, op, mean_divisor, out):
        rows, cols = x2d.shape
        check(lib().fdl_reduce_cols_allreduce_f32(_ptr(x2d), rows, cols, _ptr(out), op, float(mean_divisor),
                                                  self.ctx, None, 0, _stream()), "fdl_reduce_cols_allreduce_f32")
        return out

    def close(self):
        if self.ctx:
            lib().fdl_exchange_destroy(self.ctx)
            self.ctx = None
