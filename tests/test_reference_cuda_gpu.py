"""This library against the reference's own CUDA code on the same GPU.

The reference library (src/blkq4_f16_gemm_sm80.cu and src/mickey, compiled for sm_100a by
`make -C oracle ref_gpu` into oracle/_ref/) is loaded with ctypes and given the same device
buffers as this library.  On the reference test's 26 known-answer GEMM calls
(test/blkq4_fp16_gemm_sm80_test.cu:475-519) both must produce equal bits; on the quantizer's
corner values (sign of zero, ties, saturation) the packed bytes, scales and zero points must
be equal too.  Skipped where the reference build is absent."""
import ctypes

import numpy as np
import pytest

from oracle import blkq4_oracle as O
from tests._util import REF_GEMM_CASES, bits

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not O.have_ref_gpu(), reason="reference CUDA library not built")]

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def ref():
    lib = ctypes.CDLL(O.ref_gpu_path())
    vp, sz = ctypes.c_void_p, ctypes.c_size_t
    lib.blkq4_fp16_gemm_sm80.argtypes = [ctypes.c_int, ctypes.c_bool] + [ctypes.c_int] * 3 + [vp] + [vp, sz] * 5 + [vp]
    lib.blkq4_fp16_gemm_sm80.restype = ctypes.c_int
    lib.blkq4_fp16_quant_sm80.argtypes = [ctypes.c_int, ctypes.c_bool] + [ctypes.c_int] * 3 + [vp] + [vp, sz] * 4 + [vp]
    lib.blkq4_fp16_quant_sm80.restype = ctypes.c_int
    return lib


def cuda(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("case", REF_GEMM_CASES, ids=lambda c: "-".join(map(str, c)))
def test_gemm_equals_reference_cuda_gemm_on_known_answers(ref, case):
    from gemmlib_b200 import capi

    block, colwise, has_zp, M, N, K = case
    q, s, z = O.kat_generate(block, colwise, K, N, has_zp)
    pw = cuda(O.prepack_weights(K, N, q))
    ps, pz = (cuda(x) for x in O.prepack_meta(block, colwise, K, N, s, z))
    a = cuda(O.kat_activations(M, K))
    ours = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    theirs = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    capi.gemm(block, colwise, M, N, K, a, pw, ps, pz, ours)
    rc = ref.blkq4_fp16_gemm_sm80(block, colwise, M, N, K, None, a.data_ptr(), a.numel() * 2, pw.data_ptr(), pw.numel(),
                                  ps.data_ptr(), ps.numel() * 2, pz.data_ptr() if pz is not None else None,
                                  pz.numel() if pz is not None else 0, theirs.data_ptr(), theirs.numel() * 2, None)
    torch.cuda.synchronize()
    assert rc == 0
    assert torch.equal(ours.view(torch.int16), theirs.view(torch.int16)), int((ours.view(torch.int16) != theirs.view(torch.int16)).sum())


def edge_weights(N, K, block):
    """fp16 [N, K] built from the values where two quantizers could part ways: all-zero blocks of
    either sign, a block whose extremes tie in magnitude, values that round half-way between two
    levels, the largest and smallest normal halves, subnormals."""
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float16)
    w[0, :block] = 0.0
    w[1, :block] = np.float16(-0.0)
    w[2, :block] = np.float16(-0.0)
    w[2, 1] = 0.0
    w[3, :block] = np.linspace(-1, 1, block).astype(np.float16)           # |min| == |max|
    w[4, :block] = (np.arange(block) % 16).astype(np.float16) * np.float16(0.5) + np.float16(0.25)  # ties
    w[5, :block] = np.float16(65504.0)
    w[5, 1] = np.float16(-65504.0)
    w[6, :block] = np.float16(6.1e-5)
    w[7, :block] = np.float16(6e-8)
    w[8, :block] = np.float16(-6e-8)
    w[9, :block] = 0.0
    w[9, 3] = np.float16(1.0)
    return w


@pytest.mark.parametrize("colwise", [True, False])
@pytest.mark.parametrize("has_zp", [True, False])
@pytest.mark.parametrize("block", [16, 32, 64])
def test_quantizer_edge_values_equal_reference_cuda(ref, block, colwise, has_zp):
    from gemmlib_b200 import capi

    K, N = 256, 128
    w_np = edge_weights(N, K, block)
    if not colwise:
        # row-wise blocks run along N: put the corner rows along that direction as well
        w_np = np.ascontiguousarray(edge_weights(K, N, block).T) if N >= block else w_np
    w = torch.from_numpy(w_np).cuda()
    wb, me = capi.quant_size(block, colwise, K, N)
    out = []
    for which in ("ours", "theirs"):
        qw = torch.zeros(wb, dtype=torch.uint8, device="cuda")
        qs = torch.zeros(me, dtype=torch.float16, device="cuda")
        qz = torch.zeros(me, dtype=torch.uint8, device="cuda")
        if which == "ours":
            capi.quant(block, colwise, K, N, K, w, qw, qs, qz if has_zp else None)
        else:
            rc = ref.blkq4_fp16_quant_sm80(block, colwise, K, N, K, None, w.data_ptr(), N * K * 2, qw.data_ptr(), wb,
                                           qs.data_ptr(), me * 2, qz.data_ptr() if has_zp else None, me if has_zp else 0, None)
            assert rc == 0
        torch.cuda.synchronize()
        out.append((qw.cpu().numpy(), qs.cpu().numpy(), qz.cpu().numpy()))
    (ow, os_, oz), (tw, ts, tz) = out
    assert (ow == tw).all(), int((ow != tw).sum())
    assert (bits(os_) == bits(ts)).all(), int((bits(os_) != bits(ts)).sum())
    if has_zp:
        assert (oz == tz).all()
    # and the CPU oracle agrees with both
    pw, ps, pz = O.quant_prepack(block, colwise, w_np, has_zp)
    assert (pw == tw).all() and (bits(ps) == bits(ts)).all() and (not has_zp or (pz == tz).all())
