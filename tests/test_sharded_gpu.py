"""GPU tests of the fused GEMM + all-gather (``blkq4_gather_*``).

With one GPU the exchange degenerates to world size 1 (the kernel still stores into the
exchange buffer, raises its flag, and the second kernel waits and copies out), which covers
the epoch / slot / flag protocol, CUDA-graph replay included.  With two or more GPUs a
torchrun job of two ranks checks the gathered result against the unsharded layer on both
ranks.  Ranks never share a GPU: kernels that wait on one another must run on different
devices."""
import os
import subprocess
import sys

import numpy as np
import pytest

from tests._util import ROOT, gaussian_act, gaussian_weight

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.mark.parametrize("M,has_zp,block,N", [(1, False, 64, 1536), (4, True, 64, 1536), (7, True, 128, 1536),
                                              (8, False, 64, 1536), (16, False, 128, 1536),
                                              (16, True, 64, 8192),    # 256 KB result: copied out by the full-width kernel
                                              (12, False, 64, 6144)])
def test_world_size_one_fused_gather_matches_plain(M, has_zp, block, N):
    from gemmlib_b200.ms_blkq4linear import BlkQ4Linear
    from gemmlib_b200.sharded import PeerGather

    K = 2048
    layer = BlkQ4Linear(block, True, not has_zp, gaussian_weight(N, K, seed=5).cuda())
    x = gaussian_act(M, K, seed=6).cuda()
    want = layer(x)
    pg = PeerGather(16, N)
    assert pg.supports(layer, M)
    outs = []
    for _ in range(5):  # epochs 1..5: both slots, flags compared against a moving epoch
        full = torch.zeros(M, N, dtype=torch.float16, device="cuda")
        pg.forward(layer, x, full)
        outs.append(full)
    # replay from a CUDA graph: the epoch lives in device memory, not in the captured launch
    full_g = torch.zeros(M, N, dtype=torch.float16, device="cuda")
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        pg.forward(layer, x, full_g)
    for _ in range(3):
        full_g.zero_()
        g.replay()
    torch.cuda.synchronize()
    assert pg.status() == 0
    for full in outs + [full_g]:
        assert torch.allclose(full.float(), want.float(), rtol=0, atol=2.0 ** -8 * max(1.0, float(want.abs().max())))
    pg.close()


@pytest.mark.parametrize("M,has_zp,block,colwise", [(300, True, 64, True), (512, False, 32, False)])
def test_world_size_one_fused_gather_on_the_tensor_core_path(M, has_zp, block, colwise):
    """Prefill shapes: the CTA-pair GEMM kernel stores its tiles into the exchange buffer and publishes,
    the wait kernel waits, the copy kernel copies out.  World size 1 exercises the whole protocol - both
    buffer parities, a moving epoch, CUDA-graph replay - and the result must be the plain kernel's, bit
    for bit (same kernel, same tiles; only the destination differs)."""
    from gemmlib_b200 import capi
    from gemmlib_b200.ms_blkq4linear import BlkQ4Linear
    from gemmlib_b200.sharded import PeerGather

    sms = torch.cuda.get_device_properties(0).multi_processor_count
    K = 1024
    N = 256 * -(-(sms // 2) // -(-M // 256))     # enough 256-column pair tiles for one round of the SM pairs
    layer = BlkQ4Linear(block, colwise, not has_zp, gaussian_weight(N, K, seed=5).cuda())
    x = gaussian_act(M, K, seed=6).cuda()
    want = torch.empty(M, N, dtype=torch.float16, device="cuda")
    capi.gemm(block, colwise, M, N, K, x, layer.q_weights, layer.q_scales, layer.q_zp if has_zp else None, want)
    pg = PeerGather(M, N)
    assert pg.supports(layer, M)
    assert not pg.supports(layer, 64)            # between the skinny and the pair kernel: not fused
    outs = []
    for _ in range(3):
        full = torch.zeros(M, N, dtype=torch.float16, device="cuda")
        pg.forward(layer, x, full)
        outs.append(full)
    full_g = torch.zeros(M, N, dtype=torch.float16, device="cuda")
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        pg.forward(layer, x, full_g)
    for _ in range(3):
        full_g.zero_()
        g.replay()
    torch.cuda.synchronize()
    assert pg.status() == 0 and capi.last_kernel_status() == 0
    for full in outs + [full_g]:
        assert torch.equal(full.view(torch.int16), want.view(torch.int16))
    # a skinny call on the same context afterwards: the protocols share epochs and tickets
    x1 = gaussian_act(1, K, seed=7).cuda()
    one = torch.zeros(1, N, dtype=torch.float16, device="cuda")
    if pg.supports(layer, 1):
        pg.forward(layer, x1, one)
        torch.cuda.synchronize()
        assert pg.status() == 0
        ref1 = layer(x1)
        assert torch.allclose(one.float(), ref1.float(), rtol=0, atol=2.0 ** -8 * max(1.0, float(ref1.abs().max())))
    pg.close()


def test_unsupported_shape_is_refused_not_miscomputed():
    from gemmlib_b200 import capi
    from gemmlib_b200.ms_blkq4linear import BlkQ4Linear
    from gemmlib_b200.sharded import PeerGather

    layer = BlkQ4Linear(32, True, True, gaussian_weight(256, 512, seed=1).cuda())  # block 32: generic kernel
    pg = PeerGather(16, 256)
    assert not pg.supports(layer, 1)
    with pytest.raises(capi.BlkQ4Error, match="unsupported"):
        pg.forward(layer, gaussian_act(1, 512).cuda(), torch.empty(1, 256, dtype=torch.float16, device="cuda"))
    pg.close()


@pytest.mark.parametrize("K", [1024, 2048])  # two-kernel protocol (TMA skinny kernel) / one-kernel (decode kernel)
def test_missing_peer_expires_the_bounded_wait_and_reports_it(K):
    """Failure detection without a GPU fault: rank 0 of a two-rank exchange runs, rank 1 never
    does (its flag / arrival counter is a word nothing sets).  The wait gives up after its ~1 s
    limit, records (0x400 | rank 1), and the context, the stream and the device stay usable."""
    from gemmlib_b200 import capi
    from gemmlib_b200.ms_blkq4linear import BlkQ4Linear

    ns = 256
    layer = BlkQ4Linear(64, True, True, gaussian_weight(ns, K, seed=2).cuda())
    x = gaussian_act(1, K, seed=3).cuda()
    a = capi.GatherContext(2, 0, 16 * 2 * ns * 2)
    b = capi.GatherContext(2, 1, 16 * 2 * ns * 2)   # exists, is mapped, never runs
    blocks = [a.local_block(), b.local_block()]
    a.connect_pointers(blocks)
    b.connect_pointers(blocks)
    out = torch.zeros(1, 2 * ns, dtype=torch.float16, device="cuda")
    a.gemm(64, True, 1, ns, K, x, layer.q_weights, layer.q_scales, None, out)
    assert a.status() == (0x400 | 1)
    # rank 0's own half arrived in its buffer and was copied out; the device still works
    want = layer(x)
    torch.cuda.synchronize()
    assert torch.allclose(out[:, :ns].float(), want.float(), atol=2.0 ** -8 * max(1.0, float(want.abs().max())), rtol=0)
    assert capi.last_kernel_status() == 0
    # the context keeps working: the next call of the same (still lonely) rank expires the same way
    out.zero_()
    a.gemm(64, True, 1, ns, K, x, layer.q_weights, layer.q_scales, None, out)
    assert a.status() == (0x400 | 1)
    assert torch.allclose(out[:, :ns].float(), want.float(), atol=2.0 ** -8 * max(1.0, float(want.abs().max())), rtol=0)
    a.close()
    b.close()


def _rank_counts():
    """2, and every further power of two the box offers (4, 8): one rank per GPU."""
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return [w for w in (2, 4, 8) if w <= n] or [2]


@pytest.mark.parametrize("world", _rank_counts())
def test_ranks_fused_gather_matches_unsharded(world):
    """One torchrun rank per GPU (2, and 4 / 8 where the box has them): the fused GEMM + all-gather of an
    N-sharded layer equals the unsharded layer on every rank - eagerly, over many epochs, from a CUDA graph -
    and the unfused paths write the caller's buffer."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(29533 + world),
           os.path.join(ROOT, "tests", "sharded_gpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("RANK_OK") == world, r.stdout[-2000:] + r.stderr[-2000:]
