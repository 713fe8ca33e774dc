"""blkq4_fp16_gemm_static_ws_sm100: the split-K GEMM on the library's own device scratch array.

Collected last (file name); needs no state from other tests and leaves none: the scratch's flag
words return to zero after every call, so it passes alone and after the rest of the suite."""
import numpy as np
import pytest

from oracle import blkq4_oracle as O
from tests._util import gaussian_act, gaussian_weight

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _problem(block, has_zp, M, N, K):
    w = gaussian_weight(N, K, seed=41)
    pw, ps, pz = O.quant_prepack(block, True, w.numpy(), has_zp)
    cu = lambda x: None if x is None else torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return cu(gaussian_act(M, K, seed=42).numpy()), cu(pw), cu(ps), cu(pz)


@pytest.mark.parametrize("case", [(64, True, 512, 1024, 2048), (128, False, 300, 512, 4096)],
                         ids=lambda c: "-".join(map(str, c)))
def test_two_calls_in_a_row_match_the_workspace_entry_point(case):
    from gemmlib_b200 import capi

    block, has_zp, M, N, K = case
    a, pw, ps, pz = _problem(block, has_zp, M, N, K)
    need = capi.gemm_workspace_size(M, N, K)
    assert 0 < need <= capi.static_scratch_size()
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    want = torch.empty(M, N, dtype=torch.float16, device="cuda")
    capi.gemm(block, True, M, N, K, a, pw, ps, pz, want, workspace=ws)          # the existing entry point
    outs = [torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda") for _ in range(2)]
    capi.gemm_static_ws(block, True, M, N, K, a, pw, ps, pz, outs[0])            # first call on this device: set-up
    torch.cuda.synchronize()
    # nothing is allocated by a call: neither through torch's allocator nor behind its back
    free_before, _ = torch.cuda.mem_get_info()
    torch_before = torch.cuda.memory_allocated()
    for o in outs:                                                               # two calls in a row
        capi.gemm_static_ws(block, True, M, N, K, a, pw, ps, pz, o)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == torch_before
    assert torch.cuda.mem_get_info()[0] == free_before
    assert capi.last_kernel_status() == 0
    for o in outs:
        assert torch.equal(o.view(torch.int16), want.view(torch.int16))
    # and against the oracle, at the reference's tolerance
    wdq = O.dequant(block, True, K, N, pw.cpu().numpy(), ps.cpu().numpy(), None if pz is None else pz.cpu().numpy())
    ref = O.gemm(a.cpu().numpy(), wdq).astype(np.float64)
    tol = 1e-2 * np.sqrt(K) * float(a.abs().max()) * float(np.abs(wdq.astype(np.float32)).max())
    assert np.abs(outs[0].cpu().numpy().astype(np.float64) - ref).max() <= tol


def test_a_plan_beyond_the_scratch_is_refused():
    from gemmlib_b200 import capi

    M, N, K = 256, 4096, 4096   # four-way split: 32 tiles x 3 partial tiles of 128 KB + flags
    assert capi.gemm_workspace_size(M, N, K) > capi.static_scratch_size()
    a, pw, ps, pz = _problem(64, False, M, N, K)
    out = torch.empty(M, N, dtype=torch.float16, device="cuda")
    with pytest.raises(capi.BlkQ4Error, match="exceeds the static scratch"):
        capi.gemm_static_ws(64, True, M, N, K, a, pw, ps, pz, out)
    # a shape that needs no workspace at all runs as the plain kernel
    M2 = 16
    a2 = torch.from_numpy(gaussian_act(M2, K, seed=43).numpy()).cuda()
    o1 = torch.empty(M2, N, dtype=torch.float16, device="cuda")
    o2 = torch.empty_like(o1)
    capi.gemm_static_ws(64, True, M2, N, K, a2, pw, ps, pz, o1)
    capi.gemm(64, True, M2, N, K, a2, pw, ps, pz, o2)
    torch.cuda.synchronize()
    assert torch.equal(o1.view(torch.int16), o2.view(torch.int16))


def test_reset_clears_the_scratch_flags_and_status_words():
    """blkq4_reset: the recovery a caller runs after a non-zero kernel status.  Here nothing has
    expired; the call must be harmless (enqueued on the stream, allocating nothing) and leave the
    entry point working."""
    from gemmlib_b200 import capi

    block, has_zp, M, N, K = 64, True, 512, 1024, 2048
    a, pw, ps, pz = _problem(block, has_zp, M, N, K)
    o1 = torch.empty(M, N, dtype=torch.float16, device="cuda")
    o2 = torch.empty_like(o1)
    capi.gemm_static_ws(block, True, M, N, K, a, pw, ps, pz, o1)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    capi.reset()
    capi.gemm_static_ws(block, True, M, N, K, a, pw, ps, pz, o2)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert capi.last_kernel_status() == 0
    assert torch.equal(o1.view(torch.int16), o2.view(torch.int16))
