"""ctypes access to oracle/_ref/libref.so: the reference's own CPU check functions and CUDA
kernels, compiled in place by oracle/build_ref.py.  Test infrastructure only.

CPU functions take numpy arrays.  GPU functions take raw device pointers (ints) and run on
the legacy default stream, exactly as the reference launches them.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build_ref

_lib = None
_fp = C.POINTER(C.c_float)
_sz = C.c_size_t


def available() -> bool:
    return build_ref.lib_path().exists()


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not available():
            raise FileNotFoundError("oracle/_ref/libref.so has not been built (python -m oracle.build_ref)")
        _lib = C.CDLL(str(build_ref.lib_path()))
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_fp)


def hardware_threads() -> int:
    return int(lib().ref_cpu_hardware_threads())


# ---- CPU: the reference's check functions ----------------------------------------------------

def cpu_activation(x, op, alpha=0.01, threads=1, out=None):
    x, px = _f(x)
    out = np.empty_like(x) if out is None else out
    lib().ref_cpu_activation_mt(px, out.ctypes.data_as(_fp), _sz(x.size), C.c_int(op), C.c_float(alpha),
                                C.c_int(threads))
    return out


def cpu_vector_add(a, b, threads=1, out=None):
    a, pa = _f(a)
    b, pb = _f(b)
    out = np.empty_like(a) if out is None else out
    lib().ref_cpu_vector_add_mt(pa, pb, out.ctypes.data_as(_fp), _sz(a.size), C.c_int(threads))
    return out


def cpu_softmax_test(x):
    x, px = _f(x)
    out = np.empty_like(x)
    lib().ref_cpu_softmax_test(px, out.ctypes.data_as(_fp), _sz(x.shape[0]), _sz(x.shape[1]))
    return out


def cpu_softmax(x, threads=1, out=None):
    x, px = _f(x)
    out = np.empty_like(x) if out is None else out
    lib().ref_cpu_softmax_mt(px, out.ctypes.data_as(_fp), _sz(x.shape[0]), _sz(x.shape[1]), C.c_int(threads))
    return out


def cpu_layernorm(x, eps=1e-5, threads=1, out=None):
    x, px = _f(x)
    out = np.empty_like(x) if out is None else out
    lib().ref_cpu_layernorm_mt(px, out.ctypes.data_as(_fp), _sz(x.shape[0]), _sz(x.shape[1]), C.c_float(eps),
                               C.c_int(threads))
    return out


def cpu_block_reduce(x, tree, threads=1):
    x, px = _f(x)
    out = np.empty(x.size // 1024, dtype=np.float32)
    lib().ref_cpu_block_reduce_mt(px, out.ctypes.data_as(_fp), _sz(x.size), C.c_int(tree), C.c_int(threads))
    return out


# ---- GPU: the reference's kernels, raw device pointers ---------------------------------------

def _chk(status, what):
    if status != 0:
        raise RuntimeError(f"reference {what} failed with cudaError {status}")


def gpu_set_device(dev):
    _chk(lib().ref_gpu_set_device(C.c_int(dev)), "cudaSetDevice")


def gpu_sync():
    _chk(lib().ref_gpu_sync(), "cudaDeviceSynchronize")


def gpu_elementwise(a, b, c, n, op):
    _chk(lib().ref_gpu_elementwise(C.c_void_p(a), C.c_void_p(b), C.c_void_p(c), C.c_int(n), C.c_int(op)),
         "elementwise")


def gpu_activation(x, y, n, op, alpha=0.01):
    _chk(lib().ref_gpu_activation(C.c_void_p(x), C.c_void_p(y), C.c_int(n), C.c_int(op), C.c_float(alpha)),
         "activation")


def gpu_vector_add(a, b, c, n):
    _chk(lib().ref_gpu_vector_add(C.c_void_p(a), C.c_void_p(b), C.c_void_p(c), _sz(n)), "vector_add")


def gpu_add_row_bias(out, bias, rows, cols):
    _chk(lib().ref_gpu_add_row_bias(C.c_void_p(out), C.c_void_p(bias), C.c_int(rows), C.c_int(cols)),
         "add_row_bias")


def gpu_reduction(x, out, n, algo):
    _chk(lib().ref_gpu_reduction(C.c_void_p(x), C.c_void_p(out), _sz(n), C.c_int(algo)), "reduction")


def gpu_softmax(x, y, rows, cols, algo=2):
    _chk(lib().ref_gpu_softmax(C.c_void_p(x), C.c_void_p(y), _sz(rows), _sz(cols), C.c_int(algo)), "softmax")


def gpu_layernorm(x, y, rows, cols, eps=1e-5):
    _chk(lib().ref_gpu_layernorm(C.c_void_p(x), C.c_void_p(y), C.c_int(rows), C.c_int(cols), C.c_float(eps)),
         "layernorm")


def gpu_cross_entropy(logits, labels, loss, batch, classes):
    _chk(lib().ref_gpu_cross_entropy(C.c_void_p(logits), C.c_void_p(labels), C.c_void_p(loss), C.c_int(batch),
                                     C.c_int(classes)), "cross_entropy")


def gpu_transpose(x, y, n, algo=2):
    _chk(lib().ref_gpu_transpose(C.c_void_p(x), C.c_void_p(y), _sz(n), C.c_int(algo)), "transpose")


def gpu_uniform(data, n, low, high, seed):
    _chk(lib().ref_gpu_uniform(C.c_void_p(data), C.c_longlong(n), C.c_float(low), C.c_float(high),
                               C.c_ulonglong(seed)), "uniform")


def gpu_normal(data, n, mean, stddev, seed):
    _chk(lib().ref_gpu_normal(C.c_void_p(data), C.c_longlong(n), C.c_float(mean), C.c_float(stddev),
                              C.c_ulonglong(seed)), "normal")
