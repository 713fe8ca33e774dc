"""Generate tests/golden/prepack_golden.npz from the reference's own host code.

Run in a container that has the reference tree (it is not needed afterwards):

    make -C oracle ref_host        # compiles <reference>/test/blkq4_fp16_gemm_sm80.h
    python tests/golden/make_golden.py

For every shape of the reference's prepack tests
(test/blkq4_fp16_quant_sm80_test.cu:313-347, block 32) plus a few shapes at the
other block sizes, the known-answer weights / scales / zero points (plain
layout) are pushed through the reference's prepack_weights_ref,
prepack_quant_scales_ref and prepack_quant_offsets_ref, and the outputs are
stored.  The fixtures pin the CPU oracle, which the CUDA path is then compared
with.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import blkq4_oracle as O  # noqa: E402

# (block, colwise, K, N, has_zp)
REF_TEST_SHAPES = [(64, 32), (64, 64), (64, 128), (64, 256), (128, 32), (256, 32), (256, 256)]
REF_TEST_SHAPES_NOZP = [(64, 128), (128, 32), (256, 256)]


def cases():
    out = []
    for colwise in (False, True):
        for K, N in REF_TEST_SHAPES:
            out.append((32, colwise, K, N, True))
        for K, N in REF_TEST_SHAPES_NOZP:
            out.append((32, colwise, K, N, False))
        out.append((32, True, 64, 32, False))  # ColblockSmall's second call
    for block in (16, 64, 128):
        for colwise in (False, True):
            for has_zp in (True, False):
                out.append((block, colwise, 128, 128, has_zp))
    return sorted(set(out))


def key(block, colwise, K, N, has_zp):
    return f"b{block}_{'col' if colwise else 'row'}_{K}x{N}_{'zp' if has_zp else 'sym'}"


def main():
    assert O.have_ref_host(), "build oracle/_ref first: make -C oracle ref_host"
    data = {}
    for c in cases():
        block, colwise, K, N, has_zp = c
        q, s, z = O.kat_generate(block, colwise, K, N, has_zp)
        pw, ps, pz = O.ref_host_prepack(block, colwise, K, N, q, s, z)
        k = key(*c)
        data[k + "/q_plain"] = q
        data[k + "/scales_cm"] = s.view(np.uint16)
        data[k + "/packed"] = pw
        data[k + "/packed_scales"] = ps.view(np.uint16)
        if has_zp:
            data[k + "/zp_cm"] = z
            data[k + "/packed_zp"] = pz
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "prepack_golden.npz")
    np.savez_compressed(path, **data)
    print(path, len(cases()), "cases", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
