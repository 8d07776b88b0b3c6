"""cgadimpl_b200 -- cgadimpl's RMSNorm forward / VJP / JVP path for NVIDIA B200.

The product is libagb_cuda.so (C ABI in include/agb/agb.h) and the C++ `ag::` graph API
in cgadimpl_b200/host.  This Python package is plumbing for tests and benchmarks: it loads
the library with ctypes and passes torch device pointers and streams through.
"""
from . import _lib  # noqa: F401
from ._lib import AgbError  # noqa: F401

__all__ = ["ops", "AgbError"]
