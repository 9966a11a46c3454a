"""ter_b200: B200 (sm_100a) implementation of the reference's packed-trit matmul fabric
and decode forward, behind the C ABI declared in ``include/ter_b200.h``.

This package is a thin ctypes binding over ``libter_b200.so`` for tests and benchmarks;
the product is the shared library.  There is no CPU fallback: if the CUDA library
cannot be loaded, importing :mod:`ter_b200.api` raises.
"""
from .api import TerB200, lib, load, TerB200Error, FMT_V11, FMT_ROWMAJOR, FMT_I32  # noqa: F401
