"""Helpers shared by the parity tests."""
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden", "prepack_golden.npz")

# The 26 calls of the reference GEMM test (test/blkq4_fp16_gemm_sm80_test.cu:480-518)
# as (block, colwise, has_zp, M, N, K); its duplicated line is listed once.
REF_GEMM_CASES = [
    (32, False, False, 32, 32, 64), (32, False, True, 32, 32, 64),
    (32, False, False, 32, 96, 64), (32, False, True, 32, 96, 64),
    (32, False, False, 32, 96, 192), (32, False, True, 32, 96, 192),
    (32, False, False, 256, 672, 576), (32, False, True, 256, 672, 576),
    (32, False, False, 512, 2080, 960),
    (16, False, False, 256, 672, 576), (16, False, True, 256, 672, 576),
    (64, False, False, 256, 1024, 576), (64, False, True, 256, 1024, 576),
    (16, True, False, 256, 672, 576), (16, True, True, 256, 672, 576),
    (64, True, False, 256, 1024, 576), (64, True, True, 256, 1024, 576),
    (16, False, False, 16, 704, 576), (16, False, True, 16, 704, 576),
    (64, False, False, 16, 1024, 576), (64, False, True, 16, 1024, 576),
    (16, True, False, 16, 672, 576), (16, True, True, 16, 672, 576),
    (64, True, False, 16, 1024, 576), (64, True, True, 16, 1024, 576),
]

# Shapes of the reference prepack tests (test/blkq4_fp16_quant_sm80_test.cu:313-347).
REF_PREPACK_SHAPES = [(64, 32), (64, 64), (64, 128), (64, 256), (128, 32), (256, 32), (256, 256)]


def golden_key(block, colwise, K, N, has_zp):
    return f"b{block}_{'col' if colwise else 'row'}_{K}x{N}_{'zp' if has_zp else 'sym'}"


def golden_cases():
    z = np.load(GOLDEN)
    keys = sorted({k.split("/")[0] for k in z.files})
    out = []
    for k in keys:
        b, o, shape, zp = k.split("_")
        K, N = map(int, shape.split("x"))
        out.append((int(b[1:]), o == "col", K, N, zp == "zp"))
    return out


def gaussian_weight(N, K, sigma=0.02, seed=0):
    """fp16 [N, K] ~ N(0, sigma), torch CPU generator (the benchmark's inputs)."""
    import torch

    g = torch.Generator().manual_seed(seed)
    return (torch.randn(N, K, generator=g) * sigma).to(torch.float16)


def gaussian_act(M, K, seed=1):
    import torch

    g = torch.Generator().manual_seed(seed)
    return torch.randn(M, K, generator=g).to(torch.float16)


def bits(a):
    """Bit pattern view for exact comparisons of fp16 arrays (keeps -0 != +0)."""
    a = np.ascontiguousarray(a)
    return a.view(np.uint16) if a.dtype == np.float16 else a
