"""blackriver_b200: B200-native (sm_100a) implementation of BlackRiver's BLOOM decoder hot path.

The product is two native libraries built in-tree:

* ``lib/libbrk.so``   -- hand-written CUDA kernels behind the C ABI declared in ``include/brk.h``
* ``lib/libbr_host.so`` -- the C++ host side: operator interface, tensor facade, words VM

This Python package only loads them (ctypes) for tests and benchmarks; there is no Python or
CPU fallback for any operator: a missing library raises at import of the binding.
"""
from . import brk  # noqa: F401

__all__ = ["brk"]
