"""B200-native blockwise-int4 weight-only GEMM/GEMV (W4A16).

The product is the C-ABI shared library ``libms_blkq4gemm.so`` (entry points
declared in ``include/ms_blkq4gemm.h``) built from the CUDA sources in
``csrc/`` by ``python -m gemmlib_b200.build``.  The Python modules are the
host-side mirror of the reference's PyTorch surface (``ms_blkq4linear_ext`` /
``BlkQ4Linear``) and a thin ctypes binding (``capi``) used by the tests and the
benchmark.  There is no CPU fallback: every operation fails loudly when the
library or a CUDA device is missing.

Submodules are imported on first use so that ``gemmlib_b200.build`` can run
before the library exists.
"""
import importlib

__all__ = ["capi", "build", "ms_blkq4linear", "ms_blkq4linear_ext", "sharded"]


def __getattr__(name):
    if name in __all__:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
