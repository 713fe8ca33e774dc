"""CPU tests of the oracle: golden vectors from the reference's own host code,
the reference tests' known-answer round trip, and internal consistency."""
import numpy as np
import pytest

from oracle import blkq4_oracle as O
from tests._util import GOLDEN, REF_PREPACK_SHAPES, bits, gaussian_act, gaussian_weight, golden_cases

GOLD = np.load(GOLDEN)


@pytest.mark.parametrize("case", golden_cases(), ids=lambda c: "-".join(map(str, c)))
def test_prepack_matches_reference_golden(case):
    """Oracle prepack == outputs of the reference's prepack_*_ref (committed fixtures)."""
    from tests._util import golden_key

    block, colwise, K, N, has_zp = case
    k = golden_key(*case)
    q, s, z = O.kat_generate(block, colwise, K, N, has_zp)
    assert (q == GOLD[k + "/q_plain"]).all()
    assert (bits(s) == GOLD[k + "/scales_cm"]).all()
    pw = O.prepack_weights(K, N, q)
    ps, pz = O.prepack_meta(block, colwise, K, N, s, z)
    assert (pw == GOLD[k + "/packed"]).all()
    assert (bits(ps) == GOLD[k + "/packed_scales"]).all()
    if has_zp:
        assert (z == GOLD[k + "/zp_cm"]).all()
        assert (pz == GOLD[k + "/packed_zp"]).all()


@pytest.mark.skipif(not O.have_ref_host(), reason="reference host helpers not built here")
@pytest.mark.parametrize("block", [16, 32, 64, 128])
@pytest.mark.parametrize("colwise", [True, False])
def test_prepack_matches_reference_live(block, colwise):
    """Same comparison against the reference code run live, on random nibbles."""
    K, N = 256, 384
    rng = np.random.default_rng(block + colwise)
    wb, me = O.quant_size(block, colwise, K, N)
    q = rng.integers(0, 256, wb, dtype=np.uint8)
    s = rng.standard_normal(me).astype(np.float16)
    z = rng.integers(0, 16, me, dtype=np.uint8)
    pw, ps, pz = O.ref_host_prepack(block, colwise, K, N, q, s, z)
    assert (pw == O.prepack_weights(K, N, q)).all()
    os_, oz = O.prepack_meta(block, colwise, K, N, s, z)
    assert (bits(ps) == bits(os_)).all() and (pz == oz).all()


@pytest.mark.parametrize("colwise", [True, False])
@pytest.mark.parametrize("has_zp", [True, False])
@pytest.mark.parametrize("block", [16, 32, 64, 128])
def test_kat_round_trip(block, colwise, has_zp):
    """quantize(dequantize(q, s, z)) == (q, s, z): the identity the reference's
    testPrepack relies on (test/blkq4_fp16_quant_sm80_test.cu:53-67)."""
    shapes = REF_PREPACK_SHAPES if block == 32 else [(128, 128), (256, 384)]
    for K, N in shapes:
        try:
            O.quant_size(block, colwise, K, N)
        except ValueError:
            continue
        q, s, z = O.kat_generate(block, colwise, K, N, has_zp)
        w = O.dequant_plain(block, colwise, K, N, q, s, z)
        q2, s2, z2 = O.quantize_plain(block, colwise, w, has_zp)
        assert (q2 == q).all() and (bits(s2) == bits(s)).all()
        if has_zp:
            assert (z2 == z).all()


@pytest.mark.parametrize("colwise", [True, False])
@pytest.mark.parametrize("block", [16, 64])
def test_dequant_inverts_prepack(block, colwise):
    """Reading the packed form back gives the plain-form dequantization, and on
    known-answer data the kernel's two-rounding formula gives the same bits."""
    K, N = 128, 96 if block == 16 else 128
    q, s, z = O.kat_generate(block, colwise, K, N, True)
    w = O.dequant_plain(block, colwise, K, N, q, s, z)
    pw = O.prepack_weights(K, N, q)
    ps, pz = O.prepack_meta(block, colwise, K, N, s, z)
    for formula in (False, True):
        d = O.dequant(block, colwise, K, N, pw, ps, pz, formula)
        assert (bits(d) == bits(w)).all()


def test_quantize_properties_gaussian():
    """On Gaussian weights: nibble range, zero-point range, reconstruction error
    within half a quantization step (plus fp16 rounding)."""
    K, N = 256, 128
    w = gaussian_weight(N, K).numpy()
    for block, colwise, has_zp in [(32, True, True), (64, True, False), (16, False, True), (128, False, False)]:
        pw, ps, pz = O.quant_prepack(block, colwise, w, has_zp)
        if has_zp:
            assert pz.min() >= 0 and pz.max() <= 15
        d = O.dequant(block, colwise, K, N, pw, ps, pz).astype(np.float32)
        bk, bn = O.blocking(block, colwise)
        # per-element scale, from the plain (column-major) meta
        q, s, z = O.quantize_plain(block, colwise, w, has_zp)
        smat = np.abs(s.astype(np.float32).reshape(N // bn, K // bk))
        sfull = np.repeat(np.repeat(smat, bn, axis=0), bk, axis=1)
        err = np.abs(d - w.astype(np.float32))
        # symmetric: range [-8s, 7s] clips the positive extreme by up to one step
        bound = (0.5 if has_zp else 1.0) * sfull * 1.01 + 1e-4
        assert (err <= bound).all()


def test_symmetric_scale_sign_and_zero_block():
    """Symmetric scale = extreme / -8 keeps the extreme's sign (negative scale for a
    positive extreme); an all-zero block gives a zero scale and nibbles of 8."""
    K, N = 64, 32
    w = np.zeros((N, K), np.float16)
    w[0, :16] = np.linspace(-1, 2, 16).astype(np.float16)  # extreme +2 -> scale -0.25
    w[1, :16] = np.linspace(-2, 1, 16).astype(np.float16)  # extreme -2 -> scale +0.25
    q, s, z = O.quantize_plain(16, True, w, False)
    smat = s.reshape(N, K // 16)
    assert smat[0, 0] == np.float16(-0.25) and smat[1, 0] == np.float16(0.25)
    assert smat[2, 0] == 0
    assert (q.reshape(N, K // 2)[2] == 0x88).all()


def test_shape_rules():
    assert O.quant_size(32, True, 4096, 4096) == (4096 * 4096 // 2, 4096 * 4096 // 32)
    assert O.quant_size(64, True, 4096, 11008) == (22544384, 704512)
    assert O.quant_size(128, True, 8192, 28672) == (117440512, 1835008)
    for bad in [(32, True, 96, 32), (32, True, 64, 48), (64, False, 64, 96), (128, True, 64, 128), (8, True, 64, 32)]:
        with pytest.raises(ValueError):
            O.quant_size(*bad)


def test_gemm_oracle_against_numpy():
    M, K, N = 5, 128, 48
    a = gaussian_act(M, K).numpy()
    w = gaussian_weight(N, K).numpy()
    c = O.gemm(a, w).astype(np.float32)
    ref = a.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(c - ref).max() <= 2e-3 * np.abs(ref).max() + 1e-3
