"""GPU parity at the full sizes of the benchmark configurations, through the C ABI.

configs[3] (K=8192, N=28672, block 128 symmetric) at its FULL width for M from decode to
prefill, and the layer shapes of configs[4] (Llama-2-7B: 4096->4096, 4096->11008,
11008->4096, block 64 with zero points) at M=1 and M=512.  The oracle dequantizes the whole
weight once per shape; the GEMM is then checked on sampled rows and on sampled 128-column
tiles (first, a middle one, last), which bounds the CPU time without leaving a region of
the output unsampled in either direction.  Bars as everywhere: max |delta| <= 1e-2 *
sqrt(K) * max|a| * max|w| against the oracle's fp32-accumulate GEMM, plus the tight check
against the exact product."""
import numpy as np
import pytest

from oracle import blkq4_oracle as O
from tests._util import gaussian_act, gaussian_weight

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


class Problem:
    """One quantized weight on the device and its oracle dequantization on the host."""

    def __init__(self, block, has_zp, N, K, sigma, seed):
        from gemmlib_b200 import capi

        self.block, self.has_zp, self.N, self.K = block, has_zp, N, K
        w = gaussian_weight(N, K, sigma=sigma, seed=seed).cuda()
        wb, me = capi.quant_size(block, True, K, N)
        self.qw = torch.empty(wb, dtype=torch.uint8, device="cuda")
        self.qs = torch.empty(me, dtype=torch.float16, device="cuda")
        self.qz = torch.empty(me, dtype=torch.uint8, device="cuda") if has_zp else None
        capi.quant(block, True, K, N, K, w, self.qw, self.qs, self.qz)
        torch.cuda.synchronize()
        del w
        pw, ps = self.qw.cpu().numpy(), self.qs.cpu().numpy()
        pz = self.qz.cpu().numpy() if has_zp else None
        # fp16 [N, K]: what the reference's tests dequantize on the host; and the unrounded scale * (q - zp)
        self.wdq = O.dequant(block, True, K, N, pw, ps, pz)
        self.wmax = float(np.abs(self.wdq.astype(np.float32)).max())
        self._packed = (pw, ps, pz)

    def tile(self, t):
        """The packed tensors of the 128-column tile t (a column shard is a contiguous byte range of the
        weights and a column slice of the meta)."""
        pw, ps, pz = self._packed
        K, N, block = self.K, self.N, self.block
        w_t = pw[t * 64 * K:(t + 1) * 64 * K]
        s_t = np.ascontiguousarray(ps.reshape(K // block, N)[:, t * 128:(t + 1) * 128]).reshape(-1)
        z_t = None if pz is None else np.ascontiguousarray(pz.reshape(K // block, N)[:, t * 128:(t + 1) * 128]).reshape(-1)
        return w_t, s_t, z_t

    def ideal_tile(self, t):
        """float64 [128, K] of scale * (q - zp), no fp16 rounding."""
        return O.dequant_ideal(self.block, True, self.K, 128, *self.tile(t))

    def kernel_tile(self, t):
        """float64 [128, K] of the kernels' two-rounding fp16 dequantization."""
        return O.dequant(self.block, True, self.K, 128, *self.tile(t), kernel_formula=True).astype(np.float64)

    def run(self, a, workspace=None, flags=0):
        from gemmlib_b200 import capi

        M = a.shape[0]
        out = torch.full((M, self.N), float("nan"), dtype=torch.float16, device="cuda")
        capi.gemm(self.block, True, M, self.N, self.K, a.cuda(), self.qw, self.qs, self.qz, out, flags=flags,
                  workspace=workspace)
        torch.cuda.synchronize()
        assert capi.last_kernel_status() == 0
        return out.cpu().numpy()

    def check(self, M, seed, workspace=None, max_rows=8):
        a = gaussian_act(M, self.K, seed=seed)
        got = self.run(a, workspace=workspace)
        assert np.isfinite(got.astype(np.float32)).all()
        a_np = a.numpy()
        amax = float(np.abs(a_np.astype(np.float32)).max())
        tol = 1e-2 * np.sqrt(self.K) * amax * self.wmax
        rng = np.random.default_rng(seed)
        rows = np.arange(M) if M <= max_rows else np.sort(rng.choice(M, max_rows, replace=False))
        tiles = sorted({0, (self.N // 128) // 2, self.N // 128 - 1})
        cols = np.concatenate([np.arange(t * 128, (t + 1) * 128) for t in tiles])
        # sampled rows over ALL columns, and all rows over the sampled column tiles
        want_rows = O.gemm(a_np[rows], self.wdq).astype(np.float64)
        assert np.abs(got[rows].astype(np.float64) - want_rows).max() <= tol
        row_chunks = [np.arange(M)] if M <= 512 else [np.arange(0, 256), np.arange(M // 2, M // 2 + 256), np.arange(M - 256, M)]
        for rc in row_chunks:
            want_cols = O.gemm(a_np[rc], np.ascontiguousarray(self.wdq[cols])).astype(np.float64)
            assert np.abs(got[np.ix_(rc, cols)].astype(np.float64) - want_cols).max() <= tol
        # tight: next to the exact product with either dequantization formula
        exact_ideal = a_np[rows].astype(np.float64) @ np.concatenate([self.ideal_tile(t) for t in tiles]).T
        exact_kernel = a_np[rows].astype(np.float64) @ np.concatenate([self.kernel_tile(t) for t in tiles]).T
        g = got[np.ix_(rows, cols)].astype(np.float64)
        # the tensor-core and generic kernels dequantize to fp16 with the reference kernel's formula, the
        # decode kernels scale fp32 partial sums: the result sits next to one of the two exact products
        dist = min(np.abs(g - exact_ideal).max(), np.abs(g - exact_kernel).max())
        assert dist <= 2.0 ** -10 * max(1.0, np.abs(exact_ideal).max()), dist
        return got


@pytest.fixture(scope="module")
def c4_full():
    return Problem(128, False, 28672, 8192, sigma=0.015, seed=4)


@pytest.mark.parametrize("M", [1, 16, 64, 1024, 4096])
def test_config_c4_full_width(c4_full, M):
    """configs[3] at N = 28672: decode kernel (M=1), TMA skinny kernel (16), tensor-core kernel (64 and up)."""
    c4_full.check(M, seed=40 + M)


@pytest.fixture(scope="module", params=[(4096, 4096), (11008, 4096), (4096, 11008)], ids=lambda p: f"{p[1]}to{p[0]}")
def c5_layer(request):
    N, K = request.param
    return Problem(64, True, N, K, sigma=0.02, seed=5 + N % 7)


def test_config_c5_decode(c5_layer):
    """configs[4] at M = 1: the decode kernel with zero points, K = 4096 and K = 11008."""
    c5_layer.check(1, seed=51)


def test_config_c5_prefill(c5_layer):
    """configs[4] at M = 512, with the workspace BlkQ4Linear passes.  4096-wide outputs (64 tiles) split
    K (K = 11008 is 172 k-steps cut in two or four parts); the 11008-wide one (172 tiles) runs as
    balanced ranges."""
    from gemmlib_b200 import capi

    need = capi.gemm_workspace_size(512, c5_layer.N, c5_layer.K)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda") if need else None
    if c5_layer.N == 4096:
        assert need > 0, "a 64-tile prefill is meant to split K"
    got = c5_layer.check(512, seed=52, workspace=ws)
    if ws is not None:
        # the split result is reproducible and the workspace's flags are back to zero
        again = c5_layer.run(gaussian_act(512, c5_layer.K, seed=52), workspace=ws)
        assert (got.view(np.uint16) == again.view(np.uint16)).all()
        # one flag word per 256-row x 128-column output tile (split-K) or per CTA (balanced ranges)
        words = min(2 * (c5_layer.N // 128), torch.cuda.get_device_properties(0).multi_processor_count)
        assert int(ws[:4 * words].view(torch.int32).abs().sum()) == 0


@pytest.mark.parametrize("M", [1, 2, 3, 5, 8, 9, 12, 16])
@pytest.mark.parametrize("shape", [(64, True, 352, 2048), (128, False, 256, 4096), (64, False, 4736, 2304),
                                   (128, True, 160, 3072)], ids=lambda s: "-".join(map(str, s)))
def test_decode_kernel_exact_on_known_answers(shape, M):
    """The decode kernel (M <= 8, K >= 2048 in whole groups of 256) and, for M 9..16, the generic skinny
    kernel on the reference tests' known-answer family, where every product and partial sum is exact:
    equal bits.  (The family stops being exact near K = 8192 - its sums leave the fp16 range - so the
    kernel with two row groups, which takes M 9..16 from K = 8192 on, is covered by the Gaussian
    full-width case of configs[3] at M = 16 instead.)"""
    from gemmlib_b200 import capi

    block, has_zp, N, K = shape
    q, s, z = O.kat_generate(block, True, K, N, has_zp)
    pw = O.prepack_weights(K, N, q)
    ps, pz = O.prepack_meta(block, True, K, N, s, z)
    a = O.kat_activations(M, K)
    want = O.dequant_gemm(block, True, a, N, pw, ps, pz)
    out = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    for flags in (0, capi.EARLY_WEIGHT_FETCH):
        capi.gemm(block, True, M, N, K, torch.from_numpy(a).cuda(), torch.from_numpy(pw).cuda(),
                  torch.from_numpy(ps).cuda(), None if pz is None else torch.from_numpy(pz).cuda(), out, flags=flags)
        torch.cuda.synchronize()
        assert capi.last_kernel_status() == 0
        got = out.cpu().numpy()
        assert (got.view(np.uint16) == want.view(np.uint16)).all(), (flags, int((got.view(np.uint16) != want.view(np.uint16)).sum()))
