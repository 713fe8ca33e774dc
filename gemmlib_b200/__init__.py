"""B200-native blockwise-int4 weight-only GEMM/GEMV (W4A16).

The product is the C-ABI shared library ``libms_blkq4gemm.so`` (entry points
declared in ``include/ms_blkq4gemm.h``) built from the CUDA sources in
``csrc/``.  The Python modules are the host-side mirror of the reference's
PyTorch surface (``ms_blkq4linear_ext`` / ``BlkQ4Linear``) and a thin ctypes
binding used by the tests and the benchmark.  There is no CPU fallback: every
operation fails loudly when the library or a CUDA device is missing.
"""
from . import capi  # noqa: F401

__all__ = ["capi"]
