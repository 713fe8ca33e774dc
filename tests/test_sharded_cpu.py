"""CPU tests of the N-sharding host logic: shard arithmetic, the property that a
shard of the quantized weight is the quantized shard (oracle), and the all-gather at the
layer boundary with two gloo ranks."""
import os
import socket

import numpy as np
import pytest

from oracle import blkq4_oracle as O
from tests._util import bits, gaussian_act, gaussian_weight

torch = pytest.importorskip("torch")


def test_shard_bounds_and_multiples():
    from gemmlib_b200.sharded import shard_bounds, shard_multiple

    assert shard_multiple(64, True) == 32 and shard_multiple(128, False) == 128 and shard_multiple(16, False) == 32
    assert shard_bounds(28672, 8, 3, 128, True) == (3 * 3584, 4 * 3584)
    assert shard_bounds(11008, 4, 0, 64, True) == (0, 2752)
    with pytest.raises(ValueError):
        shard_bounds(11008, 3, 0, 64, True)       # uneven split


def test_shard_bounds_rowwise_rule():
    from gemmlib_b200.sharded import shard_bounds

    assert shard_bounds(4096, 8, 1, 128, False) == (512, 1024)
    with pytest.raises(ValueError):
        shard_bounds(1536, 8, 0, 128, False)      # 192 is not a multiple of 128
    with pytest.raises(ValueError):
        shard_bounds(1104, 2, 0, 16, True)        # 552 is not a multiple of 32


@pytest.mark.parametrize("block,colwise,has_zp", [(128, True, False), (32, True, True), (64, False, True)])
def test_quantized_shard_equals_shard_of_quantized(block, colwise, has_zp):
    """Oracle-level statement of why N-sharding needs no requantization or repacking."""
    K, N, g = 256, 512, 4
    w = gaussian_weight(N, K, seed=3).numpy()
    fw, fs, fz = O.quant_prepack(block, colwise, w, has_zp)
    ns = N // g
    for r in range(g):
        sw, ss, sz = O.quant_prepack(block, colwise, np.ascontiguousarray(w[r * ns:(r + 1) * ns]), has_zp)
        assert (sw == fw[r * ns // 2 * K:(r + 1) * ns // 2 * K]).all()  # contiguous byte range
        if colwise:   # meta row-major [K/block, N]: a column slice
            assert (bits(ss.reshape(K // block, ns)) == bits(fs.reshape(K // block, N)[:, r * ns:(r + 1) * ns])).all()
            if has_zp:
                assert (sz.reshape(K // block, ns) == fz.reshape(K // block, N)[:, r * ns:(r + 1) * ns]).all()
        else:         # meta column-major [K, N/block]: a contiguous range
            nb = ns // block
            assert (bits(ss) == bits(fs[r * nb * K:(r + 1) * nb * K])).all()
            if has_zp:
                assert (sz == fz[r * nb * K:(r + 1) * nb * K]).all()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _gather_worker(rank, world, port, M, N, K, q):
    import torch.distributed as dist

    from gemmlib_b200.sharded import gather_columns, shard_bounds

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        block, colwise = 64, True
        w = gaussian_weight(N, K, seed=9).numpy()
        a = gaussian_act(M, K, seed=2).numpy()
        n0, n1 = shard_bounds(N, world, rank, block, colwise)
        pw, ps, pz = O.quant_prepack(block, colwise, np.ascontiguousarray(w[n0:n1]), False)
        local = O.dequant_gemm(block, colwise, a, n1 - n0, pw, ps, pz)   # CPU stand-in for the shard's GEMM
        full = gather_columns(torch.from_numpy(local))
        q.put((rank, full.numpy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M", [1, 5])
def test_all_gather_of_shards_equals_unsharded(M):
    """Two gloo ranks: each computes its column shard (oracle arithmetic), the gather gives
    every rank the unsharded layer's output, bit for bit."""
    import torch.multiprocessing as mp

    world, N, K = 2, 256, 128
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gather_worker, args=(r, world, port, M, N, K, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    w = gaussian_weight(N, K, seed=9).numpy()
    a = gaussian_act(M, K, seed=2).numpy()
    pw, ps, pz = O.quant_prepack(64, True, w, False)
    want = O.dequant_gemm(64, True, a, N, pw, ps, pz)
    for r in range(world):
        assert results[r].shape == (M, N)
        assert (bits(results[r]) == bits(want)).all()
