"""Loader of the compiled PyTorch extension ``ms_blkq4linear_ext`` (built in-tree by
``gemmlib_b200.build.build_ext`` from ``csrc/ms_blkq4linear_ext.cpp``).

Exposes the reference extension's functions (python/ms_blkq4linear_ext/
ms_blkq4linear.cpp:120-123): ``quant(block_size, col_wise, has_offsets, weights)``
and ``forward(block_size, col_wise, in_features, out_features, input, q_weights,
q_scales, q_zp)``, plus ``forward_out(..., output, bias=None, flags=0)``.  There is no Python or CPU fallback: a
missing binary is an ImportError.
"""
import importlib.util
import os
import sys

import torch  # noqa: F401  (libtorch must be loaded before the extension)

from . import build as _build

_path = _build.ext_path()
if not os.path.exists(_path):
    raise ImportError(
        f"{_path} is missing: build it with `python -m gemmlib_b200.build --ext` (no fallback exists)"
    )
_spec = importlib.util.spec_from_file_location("ms_blkq4linear_ext", _path)
_mod = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_mod)
sys.modules.setdefault("ms_blkq4linear_ext", _mod)

quant = _mod.quant
forward = _mod.forward
forward_out = _mod.forward_out
library_version = _mod.library_version
EARLY_WEIGHT_FETCH = _mod.EARLY_WEIGHT_FETCH
gemm_workspace_size = _mod.gemm_workspace_size
