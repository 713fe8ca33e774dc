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


class _OracleShard(torch.nn.Module):
    """CPU stand-in for the rank-local BlkQ4Linear: oracle arithmetic, same call signature."""

    def __init__(self, block, colwise, w_shard):
        super().__init__()
        self.block, self.colwise = block, colwise
        self.out_features, self.in_features = w_shard.shape
        self.packed = O.quant_prepack(block, colwise, np.ascontiguousarray(w_shard), False)

    def forward(self, x, out=None):
        res = torch.from_numpy(O.dequant_gemm(self.block, self.colwise, x.numpy(), self.out_features, *self.packed))
        if out is not None:
            out.copy_(res)
            return out
        return res


def _out_worker(rank, world, port, M, N, K, q):
    import torch.distributed as dist

    from gemmlib_b200.sharded import ShardedBlkQ4Linear, shard_bounds

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        block, colwise = 64, True
        w = gaussian_weight(N, K, seed=9).numpy()
        a = gaussian_act(M, K, seed=2)
        n0, n1 = shard_bounds(N, world, rank, block, colwise)
        # the module without its CUDA-only constructor: the partition and out= logic is what is under test
        layer = ShardedBlkQ4Linear.__new__(ShardedBlkQ4Linear)
        torch.nn.Module.__init__(layer)
        layer.group, layer.world_size, layer.rank = None, world, rank
        layer.gather_output, layer.out_features, layer.in_features, layer.n0 = True, N, K, n0
        layer.local = _OracleShard(block, colwise, w[n0:n1])
        layer.bias = torch.arange(N, dtype=torch.float16) / 64
        layer.peer_gather = None
        mine = torch.full((M, N), float("nan"), dtype=torch.float16)
        ret = layer(a, out=mine)                      # unfused path: the caller's buffer must hold the result
        same_buffer = ret.data_ptr() == mine.data_ptr()
        fresh = layer(a)
        layer.gather_output = False
        layer.bias = None
        part = torch.full((M, n1 - n0), float("nan"), dtype=torch.float16)
        layer(a, out=part)                            # no gather: the buffer receives this rank's columns
        q.put((rank, mine.numpy(), fresh.numpy(), part.numpy(), same_buffer, (n0, n1)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M", [3, 40])
def test_forward_out_writes_the_callers_buffer_on_the_unfused_path(M):
    """ShardedBlkQ4Linear.forward(x, out=buf) without a fused exchange (any M, here also M > 16): the
    gathered result, bias included, lands in `buf`; with gather_output=False `buf` receives the rank's
    own columns.  Two gloo ranks, oracle arithmetic for the rank-local GEMM."""
    import torch.multiprocessing as mp

    world, N, K = 2, 256, 128
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_out_worker, args=(r, world, port, M, N, K, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    w = gaussian_weight(N, K, seed=9).numpy()
    a = gaussian_act(M, K, seed=2).numpy()
    pw, ps, pz = O.quant_prepack(64, True, w, False)
    plain = torch.from_numpy(O.dequant_gemm(64, True, a, N, pw, ps, pz))
    want = (plain + torch.arange(N, dtype=torch.float16) / 64).numpy()
    for rank, mine, fresh, part, same_buffer, (n0, n1) in results:
        assert same_buffer
        assert (bits(mine) == bits(want)).all()
        assert (bits(fresh) == bits(want)).all()
        assert (bits(part) == bits(plain.numpy()[:, n0:n1])).all()
