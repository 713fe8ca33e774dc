"""Worker of tests/test_sharded_gpu.py (one rank per GPU, launched by torch.distributed.run):
the fused GEMM + all-gather of an N-sharded layer must equal the unsharded layer on every
rank, eagerly, over many epochs, and from a CUDA graph."""
import os
import sys
import threading

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    from gemmlib_b200.ms_blkq4linear import BlkQ4Linear
    from gemmlib_b200.sharded import PeerGather, ShardedBlkQ4Linear

    K, N = 4096, 2048 * world
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(N, K, generator=g) * 0.02).half().to(dev)
    pg = PeerGather(16, N)
    ok = True
    for M, scale_only in [(1, True), (5, False), (16, True)]:
        x = torch.randn(M, K, generator=g).half().to(dev)
        full_layer = BlkQ4Linear(64, True, scale_only, w)
        want = full_layer(x).float()
        sharded = ShardedBlkQ4Linear(64, True, scale_only, w, peer_gather=pg)
        tol = 2.0 ** -8 * max(1.0, float(want.abs().max()))
        for it in range(6):
            got = sharded(x)
            torch.cuda.synchronize()
            ok &= bool((got.float() - want).abs().max() <= tol)
        out = torch.zeros(M, N, dtype=torch.float16, device=dev)
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            sharded(x, out=out)
        for it in range(4):
            out.zero_()
            graph.replay()
            torch.cuda.synchronize()
            ok &= bool((out.float() - want).abs().max() <= tol)
        del graph
    # prefill on the CTA-pair kernel: its epilogue stores straight into every rank's exchange buffer
    Mp, Kp = 512, 1024
    Np = 256 * 40 * world                      # 80 pair tiles per rank: at least one round of 74 pairs
    wp = (torch.randn(Np, Kp, generator=g) * 0.02).half().to(dev)
    xp = torch.randn(Mp, Kp, generator=g).half().to(dev)
    pgp = PeerGather(Mp, Np)
    full_p = BlkQ4Linear(64, True, False, wp)
    want_p = full_p(xp).float()
    tol_p = 2.0 ** -8 * max(1.0, float(want_p.abs().max()))
    sharded_p = ShardedBlkQ4Linear(64, True, False, wp, peer_gather=pgp)
    ok &= pgp.supports(sharded_p.local, Mp) == (world <= 4)   # beyond four ranks: kernel + NCCL all-gather
    for it in range(4):
        got = sharded_p(xp)
        torch.cuda.synchronize()
        ok &= bool((got.float() - want_p).abs().max() <= tol_p)
    ok &= pgp.status() == 0
    dist.barrier()
    pgp.close()
    # unfused paths (M > 16: kernel + NCCL all-gather): the caller's buffer receives the result too
    x = torch.randn(40, K, generator=g).half().to(dev)
    full_layer = BlkQ4Linear(64, True, True, w)
    want = full_layer(x).float()
    tol = 2.0 ** -8 * max(1.0, float(want.abs().max()))
    sharded = ShardedBlkQ4Linear(64, True, True, w, peer_gather=pg)
    out = torch.full((40, N), float("nan"), dtype=torch.float16, device=dev)
    ret = sharded(x, out=out)
    torch.cuda.synchronize()
    ok &= ret.data_ptr() == out.data_ptr() and bool((out.float() - want).abs().max() <= tol)
    local_only = ShardedBlkQ4Linear(64, True, True, w, gather_output=False)
    part = torch.full((40, N // world), float("nan"), dtype=torch.float16, device=dev)
    local_only(x, out=part)
    torch.cuda.synchronize()
    ok &= bool((part.float() - want[:, rank * (N // world):(rank + 1) * (N // world)]).abs().max() <= tol)
    ok &= pg.status() == 0
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    torch.cuda.synchronize()
    if int(flag.item()) == 1:
        print("RANK_OK", rank, flush=True)
    dist.barrier()
    pg.close()
    t = threading.Thread(target=dist.destroy_process_group, daemon=True)
    t.start()
    t.join(timeout=20)
    sys.stdout.flush()
    os._exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
