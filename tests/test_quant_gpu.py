"""GPU parity of the fused quantize + prepack kernel, through the C ABI.

Bar: bit-exact packed bytes, scales and zero points against the CPU oracle (which
is pinned to the reference's own host code) and, when it has been built, against
the reference's CUDA quantizer run on the same device."""
import ctypes

import numpy as np
import pytest

from oracle import blkq4_oracle as O
from tests._util import REF_PREPACK_SHAPES, bits, gaussian_weight

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def gpu_quant(block, colwise, w_nk_cuda, has_zp, ld=None):
    from gemmlib_b200 import capi

    N, K = w_nk_cuda.shape
    ld = ld or w_nk_cuda.stride(0)
    wb, me = capi.quant_size(block, colwise, K, N)
    qw = torch.full((wb,), 0xAB, dtype=torch.uint8, device="cuda")
    qs = torch.full((me,), float("nan"), dtype=torch.float16, device="cuda")
    qz = torch.full((me,), 0xCD, dtype=torch.uint8, device="cuda") if has_zp else None
    nbytes = (N - 1) * ld * 2 + K * 2 if ld != K else N * K * 2
    capi.quant(block, colwise, K, N, ld, (w_nk_cuda.data_ptr(), max(nbytes, N * ld * 2)), qw, qs, qz)
    torch.cuda.synchronize()
    return qw.cpu().numpy(), qs.cpu().numpy(), (qz.cpu().numpy() if has_zp else None)


def assert_same(got, want, what=""):
    (gw, gs, gz), (ww, ws, wz) = got, want
    assert (gw == ww).all(), f"packed weights differ {what}: {(gw != ww).sum()} bytes"
    assert (bits(gs) == bits(ws)).all(), f"scales differ {what}: {(bits(gs) != bits(ws)).sum()}"
    if wz is not None:
        assert (gz == wz).all(), f"zero points differ {what}"


@pytest.mark.parametrize("colwise", [True, False])
@pytest.mark.parametrize("has_zp", [True, False])
@pytest.mark.parametrize("block", [16, 32, 64, 128])
def test_known_answer_round_trip(block, colwise, has_zp):
    """The reference's testPrepack: dequantize known nibbles/scales/zps on the host,
    quantize on the device, expect the prepacked originals back exactly."""
    # (960, 2080) is a reference GEMM-test shape, used there row-wise only: column-wise its
    # generator's int arithmetic overflows (c * v with v > 5e6) and the identity is lost.
    shapes = (REF_PREPACK_SHAPES + [(576, 672)] + ([] if colwise else [(960, 2080)])) if block <= 32 \
        else [(128, 128), (576, 1024), (256, 384)]
    for K, N in shapes:
        try:
            O.quant_size(block, colwise, K, N)
        except ValueError:
            continue
        q, s, z = O.kat_generate(block, colwise, K, N, has_zp)
        w = O.dequant_plain(block, colwise, K, N, q, s, z)
        want = (O.prepack_weights(K, N, q),) + O.prepack_meta(block, colwise, K, N, s, z)
        got = gpu_quant(block, colwise, torch.from_numpy(w).cuda(), has_zp)
        assert_same(got, want, f"K={K} N={N}")


@pytest.mark.parametrize("colwise", [True, False])
@pytest.mark.parametrize("has_zp", [True, False])
@pytest.mark.parametrize("block", [16, 32, 64, 128])
def test_gaussian_bit_exact_vs_oracle(block, colwise, has_zp):
    K, N = 512, 384
    w = gaussian_weight(N, K, seed=block)
    want = O.quant_prepack(block, colwise, w.numpy(), has_zp)
    got = gpu_quant(block, colwise, w.cuda(), has_zp)
    assert_same(got, want)


def test_edge_values_bit_exact_vs_oracle():
    """Zero blocks (both signs of zero), constant blocks, fp16 extremes, subnormals,
    ties at .5 steps: the places where rounding and the sign of zero can differ."""
    K, N = 128, 64
    rng = np.random.default_rng(7)
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float16)
    w[0] = 0.0
    w[1] = -0.0
    w[2, ::2] = 0.0
    w[2, 1::2] = -0.0
    w[3] = 0.125
    w[4] = -0.125
    w[5, :64] = 65504.0
    w[5, 64:] = -65504.0
    w[6] = np.float16(6e-8)  # subnormal
    w[7] = (np.arange(K) % 16 - 8).astype(np.float16) * 0.5  # exact half steps
    w[8, :16] = np.linspace(0, 15, 16).astype(np.float16)
    w[9] = np.abs(w[9])
    w[10] = -np.abs(w[10])
    w[11:14] = (rng.integers(-3, 4, (3, K)) * 0.0625).astype(np.float16)
    for block in (16, 32, 64, 128):
        for colwise in (True, False):
            for has_zp in (True, False):
                if block == 128 and not colwise:
                    continue  # N = 64 < 128
                want = O.quant_prepack(block, colwise, w, has_zp)
                got = gpu_quant(block, colwise, torch.from_numpy(w).cuda(), has_zp)
                assert_same(got, want, f"block={block} colwise={colwise} zp={has_zp}")


def test_leading_dimension_and_unaligned_source():
    """ld > K, and a source whose rows are not 16-byte aligned (scalar-load path)."""
    K, N = 128, 64
    for ld, off in [(K + 8, 0), (K + 3, 0), (K, 1)]:
        base = torch.zeros(N * ld + 8, dtype=torch.float16)
        view = base[off : off + N * ld].view(N, ld)
        view[:, :K] = gaussian_weight(N, K, seed=3)
        w_np = np.ascontiguousarray(view[:, :K].numpy())
        dev = base.cuda()
        dview = dev[off : off + N * ld].view(N, ld)[:, :K]
        want = O.quant_prepack(32, True, w_np, True)
        got = gpu_quant(32, True, dview, True, ld=ld)
        assert_same(got, want, f"ld={ld} off={off}")


@pytest.mark.parametrize("cfg", [(32, True, True, 4096, 4096), (64, True, False, 4096, 11008)])
def test_benchmark_shapes_bit_exact(cfg):
    """Full-size benchmark shapes (c3 / c2 weights) against the oracle."""
    block, colwise, has_zp, K, N = cfg
    w = gaussian_weight(N, K, seed=0)
    want = O.quant_prepack(block, colwise, w.numpy(), has_zp)
    got = gpu_quant(block, colwise, w.cuda(), has_zp)
    assert_same(got, want)


def test_shard_of_quantized_equals_quantized_shard():
    """Size-independent property behind N-sharding: quantizing columns [n0, n1) alone
    gives the same bytes as slicing the full result (packed weight: a contiguous
    byte range; column-wise meta: a column slice)."""
    K, N, g = 8192, 3584, 4
    block = 128
    w = gaussian_weight(N, K, sigma=0.015, seed=5).cuda()
    fw, fs, _ = gpu_quant(block, True, w, False)
    ns = N // g
    for r in range(g):
        sw, ss, _ = gpu_quant(block, True, w[r * ns : (r + 1) * ns].contiguous(), False)
        assert (sw == fw[r * ns // 2 * K : (r + 1) * ns // 2 * K]).all()
        assert (bits(ss.reshape(K // block, ns)) == bits(fs.reshape(K // block, N)[:, r * ns : (r + 1) * ns])).all()


@pytest.mark.skipif(not O.have_ref_gpu(), reason="reference CUDA library not built")
@pytest.mark.parametrize("colwise", [True, False])
@pytest.mark.parametrize("has_zp", [True, False])
@pytest.mark.parametrize("block", [16, 32, 64])
def test_bit_exact_vs_reference_cuda_quantizer(block, colwise, has_zp):
    """The reference's own CUDA quantizer (compiled for sm_100a from its sources) on
    the same Gaussian input: the authority for bit-exactness on real-valued data."""
    ref = ctypes.CDLL(O.ref_gpu_path())
    K, N = 1024, 768
    w = gaussian_weight(N, K, seed=11 + block).cuda()
    wb, me = O.quant_size(block, colwise, K, N)
    qw = torch.zeros(wb, dtype=torch.uint8, device="cuda")
    qs = torch.zeros(me, dtype=torch.float16, device="cuda")
    qz = torch.zeros(me, dtype=torch.uint8, device="cuda")
    vp, sz = ctypes.c_void_p, ctypes.c_size_t
    ref.blkq4_fp16_quant_sm80.argtypes = [ctypes.c_int, ctypes.c_bool] + [ctypes.c_int] * 3 + [vp] + [vp, sz] * 4 + [vp]
    rc = ref.blkq4_fp16_quant_sm80(
        block, colwise, K, N, K, None, w.data_ptr(), N * K * 2, qw.data_ptr(), wb, qs.data_ptr(), me * 2,
        qz.data_ptr() if has_zp else None, me if has_zp else 0, None)
    torch.cuda.synchronize()
    assert rc == 0
    want = (qw.cpu().numpy(), qs.cpu().numpy(), qz.cpu().numpy() if has_zp else None)
    got = gpu_quant(block, colwise, w, has_zp)
    assert_same(got, want, "vs reference CUDA")
    # and the CPU oracle agrees with the reference's device code as well
    assert_same(O.quant_prepack(block, colwise, w.cpu().numpy(), has_zp), want, "oracle vs reference CUDA")
