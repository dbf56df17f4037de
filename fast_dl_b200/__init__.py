"""B200-native (sm_100a) implementation of fast_dl's bandwidth-bound tensor path.

The product is native: CUDA kernels behind the C ABI of include/fdl_kernels.h
(csrc/ -> lib/libfdl_kernels.so) and a C++ host library with fast_dl's `dl::` API on top
(host/ -> lib/libdl_core.so).  The Python modules here only build those libraries
(`build`) and bind the C ABI for the tests and the bench (`capi`).
"""
__all__ = ["build", "capi"]
