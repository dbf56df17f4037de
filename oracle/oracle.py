"""numpy-facing wrapper of oracle/_build/libfdl_oracle.so (test infrastructure only).

Every function takes and returns numpy arrays and calls the scalar C restatement in
oracle/fdl_oracle.c.  The library is built on demand with the flags fixed in
oracle/build_oracle.py.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build_oracle

_lib = None
_fp = C.POINTER(C.c_float)
_dp = C.POINTER(C.c_double)
_ip = C.POINTER(C.c_int64)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build_oracle.build()))
        _lib.orc_sum_f64.restype = C.c_double
        _lib.orc_norm2_f64.restype = C.c_double
        _lib.orc_cross_entropy_f64.restype = C.c_double
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_fp)


def _opt(a):
    if a is None:
        return None, None
    return _f(a)


def binary(a, b, op):
    a, pa = _f(a)
    b, pb = _f(b)
    out = np.empty_like(a)
    lib().orc_binary_f32(pa, pb, out.ctypes.data_as(_fp), C.c_int64(a.size), C.c_int(op))
    return out


def unary(x, op, alpha=0.01):
    x, px = _f(x)
    out = np.empty_like(x)
    lib().orc_unary_f32(px, out.ctypes.data_as(_fp), C.c_int64(x.size), C.c_int(op), C.c_float(alpha))
    return out


def mul_add_relu(a, b, c):
    a, pa = _f(a)
    b, pb = _f(b)
    c, pc = _f(c)
    out = np.empty_like(a)
    lib().orc_mul_add_relu_f32(pa, pb, pc, out.ctypes.data_as(_fp), C.c_int64(a.size))
    return out


def add_row_bias(x, bias, relu=False):
    out = np.array(x, dtype=np.float32, order="C", copy=True)
    bias, pb = _f(bias)
    rows, cols = out.shape
    lib().orc_add_row_bias_f32(out.ctypes.data_as(_fp), pb, C.c_int64(rows), C.c_int64(cols), C.c_int(int(relu)))
    return out


def _bstrides(shape, oshape):
    nd = len(oshape)
    shape = (1,) * (nd - len(shape)) + tuple(shape)
    strides, acc = [0] * nd, 1
    for i in range(nd - 1, -1, -1):
        strides[i] = 0 if shape[i] == 1 else acc
        acc *= shape[i]
    return strides


def broadcast_binary(a, b, op):
    a, pa = _f(a)
    b, pb = _f(b)
    oshape = np.broadcast_shapes(a.shape, b.shape)
    nd = max(len(oshape), 1)
    oshape_l = tuple(oshape) if len(oshape) else (1,)
    out = np.empty(oshape_l, dtype=np.float32)
    arr = C.c_int64 * nd
    lib().orc_broadcast_binary_f32(pa, pb, out.ctypes.data_as(_fp), C.c_int(nd), arr(*oshape_l),
                                   arr(*_bstrides(a.shape, oshape_l)), arr(*_bstrides(b.shape, oshape_l)),
                                   C.c_int(op))
    return out.reshape(oshape)


def block_reduce_1024(x, tree):
    x, px = _f(x)
    out = np.empty(x.size // 1024, dtype=np.float32)
    lib().orc_block_reduce_1024_f32(px, out.ctypes.data_as(_fp), C.c_int64(x.size), C.c_int(tree))
    return out


def full_sum(x) -> float:
    x, px = _f(x)
    return float(lib().orc_sum_f64(px, C.c_int64(x.size)))


def norm2(x) -> float:
    x, px = _f(x)
    return float(lib().orc_norm2_f64(px, C.c_int64(x.size)))


def reduce_rows(x, op):
    x, px = _f(x)
    rows, cols = x.shape
    out = np.empty(rows, dtype=np.float32)
    lib().orc_reduce_rows_f32(px, C.c_int64(rows), C.c_int64(cols), out.ctypes.data_as(_fp), C.c_int(op))
    return out


def argmax_rows(x):
    x, px = _f(x)
    rows, cols = x.shape
    out = np.empty(rows, dtype=np.int64)
    lib().orc_argmax_rows_f32(px, C.c_int64(rows), C.c_int64(cols), out.ctypes.data_as(_ip))
    return out


def reduce_cols(x, op, mean_divisor=None):
    x, px = _f(x)
    if x.ndim == 2:
        batch, (rows, cols) = 1, x.shape
        oshape = (cols,)
    else:
        batch, rows, cols = x.shape
        oshape = (batch, cols)
    out = np.empty(oshape, dtype=np.float32)
    div = float(rows if mean_divisor is None else mean_divisor)
    lib().orc_reduce_cols_f32(px, C.c_int64(batch), C.c_int64(rows), C.c_int64(cols),
                              out.ctypes.data_as(_fp), C.c_int(op), C.c_double(div))
    return out


def softmax_rows(x):
    x, px = _f(x)
    rows, cols = x.shape
    out = np.empty_like(x)
    lib().orc_softmax_rows_f32(px, out.ctypes.data_as(_fp), C.c_int64(rows), C.c_int64(cols))
    return out


def softmax_rows_f64(x):
    x, px = _f(x)
    rows, cols = x.shape
    out = np.empty(x.shape, dtype=np.float64)
    lib().orc_softmax_rows_f64(px, out.ctypes.data_as(_dp), C.c_int64(rows), C.c_int64(cols))
    return out


def layernorm_rows(x, gamma=None, beta=None, eps=1e-5):
    x, px = _f(x)
    g, pg = _opt(gamma)
    b, pb = _opt(beta)
    rows, cols = x.shape
    out = np.empty_like(x)
    lib().orc_layernorm_rows_f32(px, pg, pb, out.ctypes.data_as(_fp), C.c_int64(rows), C.c_int64(cols),
                                 C.c_float(eps))
    return out


def layernorm_rows_f64(x, gamma=None, beta=None, eps=1e-5):
    x, px = _f(x)
    g, pg = _opt(gamma)
    b, pb = _opt(beta)
    rows, cols = x.shape
    out = np.empty(x.shape, dtype=np.float64)
    lib().orc_layernorm_rows_f64(px, pg, pb, out.ctypes.data_as(_dp), C.c_int64(rows), C.c_int64(cols),
                                 C.c_double(eps))
    return out


def ulp_distance(a, b):
    """Distance in units in the last place between two float32 arrays (same sign order)."""
    a = np.ascontiguousarray(a, dtype=np.float32).view(np.int32).astype(np.int64)
    b = np.ascontiguousarray(b, dtype=np.float32).view(np.int32).astype(np.int64)
    a = np.where(a < 0, np.int64(-(2 ** 31)) - a, a)
    b = np.where(b < 0, np.int64(-(2 ** 31)) - b, b)
    return np.abs(a - b)


def cross_entropy(logits, labels) -> float:
    logits, pl = _f(logits)
    labels = np.ascontiguousarray(labels, dtype=np.int64)
    batch, classes = logits.shape
    return float(lib().orc_cross_entropy_f64(pl, labels.ctypes.data_as(_ip), C.c_int64(batch), C.c_int64(classes)))


def transpose(x):
    x, px = _f(x)
    out = np.empty_like(x)
    lib().orc_transpose_f32(px, out.ctypes.data_as(_fp), C.c_int64(x.shape[0]))
    return out
