"""GPU parity of the W4A16 GEMM / GEMV kernels, through the C ABI.

Two bars.  (1) On the reference tests' known-answer family every product and
partial sum is exact, and the result must EQUAL the naive fp32-accumulate GEMM on
the host-dequantized weights (the reference's TensorEquals criterion).  (2) On
Gaussian inputs: max |delta| <= 1e-2 * sqrt(K) * max|a| * max|w| against the oracle's
dequantize-then-GEMM (fp32 accumulate), plus a much tighter relative check that
catches layout mistakes the loose bound would hide."""
import numpy as np
import pytest

from oracle import blkq4_oracle as O
from tests._util import REF_GEMM_CASES, bits, gaussian_act, gaussian_weight

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def to_cuda(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def gpu_gemm(block, colwise, a_mk, N, packed, scales, zp, flags=0, workspace=None):
    from gemmlib_b200 import capi

    M, K = a_mk.shape
    a, pw, ps, pz = to_cuda(a_mk), to_cuda(packed), to_cuda(scales), to_cuda(zp)
    out = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    capi.gemm(block, colwise, M, N, K, a, pw, ps, pz, out, flags=flags, workspace=workspace)
    torch.cuda.synchronize()
    assert capi.last_kernel_status() == 0
    return out.cpu().numpy()


def kat_problem(block, colwise, has_zp, M, N, K):
    q, s, z = O.kat_generate(block, colwise, K, N, has_zp)
    pw = O.prepack_weights(K, N, q)
    ps, pz = O.prepack_meta(block, colwise, K, N, s, z)
    a = O.kat_activations(M, K)
    return a, pw, ps, pz


@pytest.mark.parametrize("case", REF_GEMM_CASES, ids=lambda c: "-".join(map(str, c)))
def test_reference_gemm_cases_exact(case):
    """The reference's BlkQ4Fp16Gemm.Sm80Test list (test/blkq4_fp16_gemm_sm80_test.cu:480-518)."""
    block, colwise, has_zp, M, N, K = case
    a, pw, ps, pz = kat_problem(block, colwise, has_zp, M, N, K)
    want = O.dequant_gemm(block, colwise, a, N, pw, ps, pz)
    got = gpu_gemm(block, colwise, a, N, pw, ps, pz)
    assert (bits(got) == bits(want)).all(), f"{(bits(got) != bits(want)).sum()} of {got.size} differ"


@pytest.mark.parametrize("M", [1, 2, 3, 7, 8, 9, 15, 16, 17, 33, 64, 100, 128, 129, 255, 256, 300])
def test_every_m_class_exact(M):
    """Row counts around the kernel boundaries (skinny <= 8, <= 16, tensor-core tiles),
    block 128 included, on exact known-answer data."""
    for block, colwise, has_zp, N, K in [(64, True, True, 352, 256), (128, True, False, 256, 384),
                                         (32, False, True, 96, 192), (16, True, False, 2080, 64)]:
        a, pw, ps, pz = kat_problem(block, colwise, has_zp, M, N, K)
        want = O.dequant_gemm(block, colwise, a, N, pw, ps, pz)
        got = gpu_gemm(block, colwise, a, N, pw, ps, pz)
        assert (bits(got) == bits(want)).all(), (M, block, colwise, has_zp, N, K)


def check_gaussian(block, colwise, has_zp, M, N, K, sigma=0.02, flags=0, workspace=None):
    w = gaussian_weight(N, K, sigma=sigma, seed=K + N)
    a = gaussian_act(M, K, seed=M).numpy()
    pw, ps, pz = O.quant_prepack(block, colwise, w.numpy(), has_zp)
    got = gpu_gemm(block, colwise, a, N, pw, ps, pz, flags=flags, workspace=workspace).astype(np.float64)
    assert np.isfinite(got).all()
    wdq = O.dequant(block, colwise, K, N, pw, ps, pz)
    want = O.gemm(a, wdq).astype(np.float64)
    tol = 1e-2 * np.sqrt(K) * np.abs(a.astype(np.float32)).max() * np.abs(wdq.astype(np.float32)).max()
    err = np.abs(got - want).max()
    assert err <= tol, (err, tol)
    # Tight check.  The tensor-core kernel and the generic skinny kernel dequantize to fp16
    # with the reference kernel's two-rounding formula; the fast skinny path scales fp32
    # partial sums instead (no fp16 rounding of scale * q).  The result must sit next to
    # one of the two: what remains is fp32 summation order and one fp16 output rounding.
    wk = O.dequant(block, colwise, K, N, pw, ps, pz, kernel_formula=True)
    a64 = a.astype(np.float64)
    exact_kernel = a64 @ wk.astype(np.float64).T
    exact_ideal = a64 @ O.dequant_ideal(block, colwise, K, N, pw, ps, pz).T
    dist = min(np.abs(got - exact_kernel).max(), np.abs(got - exact_ideal).max())
    assert dist <= 2.0 ** -10 * max(1.0, np.abs(exact_ideal).max()), dist


@pytest.mark.parametrize("colwise", [True, False])
@pytest.mark.parametrize("has_zp", [True, False])
@pytest.mark.parametrize("block", [16, 32, 64, 128])
@pytest.mark.parametrize("M", [1, 5, 16, 48, 512])
def test_gaussian_tolerance(block, colwise, has_zp, M):
    check_gaussian(block, colwise, has_zp, M, 384, 512)


# Shapes that walk the streaming skinny kernel's corners: more tiles than SMs, fewer tiles than
# SMs, K not a multiple of 1024, fewer units per tile than consumer warps (K < 8192), 9..16
# rows, very long K.
STREAM_CASES = [
    (64, False, 1, 4736, 1024), (64, True, 3, 2400, 1280), (128, False, 8, 160, 3072),
    (128, True, 16, 4768, 2048), (64, True, 9, 2432, 5120), (64, False, 2, 1600, 16384),
    (128, True, 16, 64, 32768),  # per-step terms would not fit in shared memory: generic kernel
    (64, True, 1, 4096, 11008), (128, False, 5, 512, 1664),  # K not a multiple of 512: partial last unit
]


@pytest.mark.parametrize("flags", [0, 1], ids=["plain", "early_fetch"])
@pytest.mark.parametrize("case", STREAM_CASES, ids=lambda c: "-".join(map(str, c)))
def test_streaming_skinny_kernel_shapes(case, flags):
    block, has_zp, M, N, K = case
    check_gaussian(block, True, has_zp, M, N, K, flags=flags)


@pytest.mark.parametrize("M", [1, 64, 300])
def test_early_weight_fetch_keeps_stream_order_for_activations(M):
    """A chain of layers on one stream, each consuming the previous output.  With
    BLKQ4_GEMM_EARLY_WEIGHT_FETCH a launch may fetch (and, in the tensor-core kernel, dequantize)
    weights while its predecessor still runs, but must not read activations (or write its
    output) before the predecessor is done: the chain's result must match the plainly
    serialized chain.  M = 1: skinny kernel; 64 and 300: tensor-core kernel."""
    from gemmlib_b200 import capi

    K = N = 4096
    layers = []
    for i in range(6):
        w = gaussian_weight(N, K, sigma=0.015, seed=100 + i)
        layers.append(tuple(to_cuda(x) for x in O.quant_prepack(64, True, w.numpy(), False)))
    a0 = to_cuda(gaussian_act(M, K, seed=3).numpy())

    def chain(flags):
        bufs = [a0] + [torch.zeros(M, N, dtype=torch.float16, device="cuda") for _ in layers]
        for _ in range(3):  # repeat: later rounds run with everything warm
            for i, (pw, ps, pz) in enumerate(layers):
                capi.gemm(64, True, M, N, K, bufs[i], pw, ps, pz, bufs[i + 1], flags=flags)
        torch.cuda.synchronize()
        assert capi.last_kernel_status() == 0
        return [b.float().cpu().numpy() for b in bufs[1:]]

    plain, early = chain(0), chain(capi.EARLY_WEIGHT_FETCH)
    for i, (x, y) in enumerate(zip(plain, early)):
        assert np.isfinite(y).all()
        assert (x == y).all(), i  # both kernels add their partial sums in a fixed order


@pytest.mark.parametrize("case", [(64, True, False, 1, 2048, 1024), (64, True, True, 12, 352, 256),
                                  (32, False, True, 5, 96, 192), (32, True, True, 300, 384, 512),
                                  (128, True, False, 64, 256, 384)], ids=lambda c: "-".join(map(str, c)))
def test_fused_bias_equals_separate_add(case):
    """The bias of blkq4_fp16_gemm_sm100 is added in fp16 to the rounded result: bit-identical
    to the reference module's `output += bias` on the fp16 output (every kernel family)."""
    from gemmlib_b200 import capi

    block, colwise, has_zp, M, N, K = case
    w = gaussian_weight(N, K, seed=7)
    a = to_cuda(gaussian_act(M, K, seed=8).numpy())
    pw, ps, pz = (to_cuda(x) for x in O.quant_prepack(block, colwise, w.numpy(), has_zp))
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(9)) * 0.5).to(torch.float16).cuda()
    plain = torch.empty(M, N, dtype=torch.float16, device="cuda")
    fused = torch.empty_like(plain)
    capi.gemm(block, colwise, M, N, K, a, pw, ps, pz, plain)
    capi.gemm(block, colwise, M, N, K, a, pw, ps, pz, fused, bias=bias)
    torch.cuda.synchronize()
    plain += bias
    assert torch.equal(plain.view(torch.int16), fused.view(torch.int16))
    with pytest.raises(capi.BlkQ4Error, match="bias"):
        capi.gemm(block, colwise, M, N, K, a, pw, ps, pz, fused, bias=bias[:-2])


@pytest.mark.parametrize("case", [(64, True, True, 512, 512, 2048), (32, False, False, 300, 384, 1024),
                                  (128, True, False, 48, 1024, 4096), (16, True, True, 700, 256, 1024)],
                         ids=lambda c: "-".join(map(str, c)))
def test_split_k_with_workspace(case):
    """blkq4_fp16_gemm_ws_sm100: few output tiles, so K is split over several SMs through the
    caller's workspace.  Same parity bars as the unsplit kernel; the flags part of the workspace
    is back to zero afterwards; two runs agree bit for bit (partials are added in part order)."""
    from gemmlib_b200 import capi

    block, colwise, has_zp, M, N, K = case
    need = capi.gemm_workspace_size(M, N, K)
    assert need > 0, "the shape is meant to split"
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    check_gaussian(block, colwise, has_zp, M, N, K, workspace=ws)
    tiles = -(-M // min(256, -(-M // 16) * 16)) * -(-N // 128)
    assert int(ws[: 4 * tiles].view(torch.int32).abs().sum()) == 0
    w = gaussian_weight(N, K, seed=K + N)
    a = gaussian_act(M, K, seed=M).numpy()
    pw, ps, pz = O.quant_prepack(block, colwise, w.numpy(), has_zp)
    r1 = gpu_gemm(block, colwise, a, N, pw, ps, pz, workspace=ws)
    r2 = gpu_gemm(block, colwise, a, N, pw, ps, pz, workspace=ws)
    assert (bits(r1) == bits(r2)).all()
    # a workspace that is too small is ignored, not an error
    small = torch.zeros(256, dtype=torch.uint8, device="cuda")
    r3 = gpu_gemm(block, colwise, a, N, pw, ps, pz, workspace=small)
    plain = gpu_gemm(block, colwise, a, N, pw, ps, pz)
    assert (bits(r3) == bits(plain)).all()


@pytest.mark.parametrize("case", [(64, True, True, 48, 28672, 1024), (128, True, False, 300, 11008, 4096),
                                  (32, False, True, 100, 22528, 4096), (64, True, True, 512, 11008, 4096),
                                  (32, False, False, 257, 28672, 2048)],
                         ids=lambda c: "-".join(map(str, c)))
def test_balanced_ranges_with_workspace(case):
    """More output tiles than SMs, but far from a whole number of rounds: with a workspace every CTA
    takes one contiguous range of k steps and a tile cut by a range boundary is finished through an
    fp32 partial tile.  Same parity bars; flag words back to zero; runs agree bit for bit; without
    the workspace the kernel runs in whole rounds."""
    from gemmlib_b200 import capi

    block, colwise, has_zp, M, N, K = case
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    tiles = -(-M // min(256, -(-M // 16) * 16)) * -(-N // 128)
    units = sms
    if M >= 256 and -(-M // 256) * -(-(-(-N // 128)) // 2) >= sms // 2:
        # the CTA-pair kernel: 256-column pair tiles on sms / 2 pairs
        tiles, units = -(-M // 256) * -(-(-(-N // 128)) // 2), sms // 2
    if not (tiles > units and tiles < 0.8 * -(-tiles // units) * units and tiles * (K // 64) // units >= K // 64 + 8):
        pytest.skip(f"{tiles} tiles on {units} units: not a balanced plan on this device")
    need = capi.gemm_workspace_size(M, N, K)
    assert need > 4 * sms
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    check_gaussian(block, colwise, has_zp, M, N, K, workspace=ws)
    assert int(ws[: 4 * sms].view(torch.int32).abs().sum()) == 0
    w = gaussian_weight(N, K, seed=K + N)
    a = gaussian_act(M, K, seed=M).numpy()
    pw, ps, pz = O.quant_prepack(block, colwise, w.numpy(), has_zp)
    r1 = gpu_gemm(block, colwise, a, N, pw, ps, pz, workspace=ws)
    r2 = gpu_gemm(block, colwise, a, N, pw, ps, pz, workspace=ws)
    assert (bits(r1) == bits(r2)).all()
    assert capi.last_kernel_status() == 0
    # whole rounds (no workspace) sum every tile in one accumulator: equal up to fp32 summation order
    plain = gpu_gemm(block, colwise, a, N, pw, ps, pz)
    assert np.abs(r1.astype(np.float32) - plain.astype(np.float32)).max() <= 2e-3 * max(1.0, float(np.abs(plain).max()))


def test_workspace_plans():
    from gemmlib_b200 import capi

    assert capi.gemm_workspace_size(2048, 4096, 4096) == 0   # 128 pair tiles on 74 CTA pairs: 86 % busy, left alone
    assert capi.gemm_workspace_size(16, 4096, 4096) == 0     # skinny kernel
    assert capi.gemm_workspace_size(512, 4096, 4096) > 0     # 64 tiles: split-K over single CTAs
    assert capi.gemm_workspace_size(512, 11008, 4096) > 0    # 86 pair tiles: balanced ranges


def test_config_c1_cpu_reference_case():
    """configs[0]: M16 K4096 N4096 b32 column-wise with zero points."""
    check_gaussian(32, True, True, 16, 4096, 4096)


def test_config_c2_decode_gemv():
    """configs[1]: M1 K4096 N11008 b64 column-wise symmetric."""
    check_gaussian(64, True, False, 1, 11008, 4096)


def test_config_c3_prefill_gemm_rows_sample():
    """configs[2]: M2048 K4096 N4096 b32 zp.  The oracle GEMM at full M is slow; the GPU
    runs the full problem and 64 sampled rows are checked, together with linearity
    in A (a size-independent property): f(2a) == 2 f(a) exactly in fp16
    (outside the subnormal range)."""
    block, colwise, has_zp, M, N, K = 32, True, True, 2048, 4096, 4096
    w = gaussian_weight(N, K, seed=0)
    a = gaussian_act(M, K, seed=1).numpy()
    pw, ps, pz = O.quant_prepack(block, colwise, w.numpy(), has_zp)
    got = gpu_gemm(block, colwise, a, N, pw, ps, pz)
    rows = np.random.default_rng(0).choice(M, 64, replace=False)
    wdq = O.dequant(block, colwise, K, N, pw, ps, pz)
    want = O.gemm(a[rows], wdq).astype(np.float64)
    tol = 1e-2 * np.sqrt(K) * np.abs(a.astype(np.float32)).max() * np.abs(wdq.astype(np.float32)).max()
    assert np.abs(got[rows].astype(np.float64) - want).max() <= tol
    assert np.abs(got[rows].astype(np.float64) - want).max() <= 0.02  # outputs are O(1)
    got2 = gpu_gemm(block, colwise, (a * np.float16(2)).astype(np.float16), N, pw, ps, pz)
    # doubling is exact except where the fp16 result is subnormal
    normal = np.abs(got.astype(np.float32)) >= 2.0 ** -13
    assert (bits(got2)[normal] == bits((got * np.float16(2)).astype(np.float16))[normal]).all()
    assert np.abs(got2.astype(np.float32) - 2 * got.astype(np.float32))[~normal].max(initial=0) <= 2.0 ** -23


def test_config_c4_sweep_shape_block128():
    """configs[3] shapes (K8192 N28672 b128 symmetric), one shard of 8 (N=3584)."""
    for M in (1, 4, 16, 64, 256):
        check_gaussian(128, True, False, M, 3584, 8192, sigma=0.015)


def test_output_canaries_untouched():
    """The kernels write exactly M*N outputs: guard bytes around the buffer survive."""
    from gemmlib_b200 import capi

    for M in (1, 16, 40):
        block, colwise, N, K = 32, True, 96, 128
        a, pw, ps, pz = kat_problem(block, colwise, True, M, N, K)
        buf = torch.full((M * N + 512,), 7.0, dtype=torch.float16, device="cuda")
        out = buf[256 : 256 + M * N]
        capi.gemm(block, colwise, M, N, K, to_cuda(a), to_cuda(pw), to_cuda(ps), to_cuda(pz), out)
        torch.cuda.synchronize()
        h = buf.cpu().numpy()
        assert (h[:256] == 7).all() and (h[256 + M * N :] == 7).all()
        want = O.dequant_gemm(block, colwise, a, N, pw, ps, pz)
        assert (bits(h[256 : 256 + M * N].reshape(M, N)) == bits(want)).all()
