"""N-sharded ``BlkQ4Linear`` for one box of B200s: one process per GPU.

The weight [out_features, in_features] is split along out_features (N); rank r owns
rows [r*N/g, (r+1)*N/g), quantizes and prepacks its shard locally, and computes
``out_r = input @ W_r^T`` for the replicated input.  The only exchange is an
all-gather of the outputs along the last dimension at the layer boundary.  On GPUs
and for M <= 16 on the skinny kernels' fast paths that exchange is FUSED into the
kernel (``PeerGather``, C ABI ``blkq4_gather_*``): the decode kernel (M <= 8) stores
its results into every rank's buffer over NVLink as flagged 8-byte words, waits for
the peers' words and copies the gathered rows out, all in one launch; for M 9..16 the
epilogue stores plain fp16 and a small second kernel waits for the peers' flags.
Everything else all-gathers with ``torch.distributed`` (NCCL on GPUs; gloo in the CPU
tests of the partitioning logic).  The reference has no
multi-GPU path; this module is the partition the W4A16 path shards along.

Quantization blocks never straddle a shard when the shard width is a multiple of
``shard_multiple(block, col_wise)``; quantizing a shard then yields exactly the
bytes of the corresponding slice of the full quantized weight.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist
from torch import nn


def shard_multiple(block_size: int, col_wise: bool) -> int:
    """Shard widths must be multiples of this: 32 (the quantizer's column rule; also
    covers the 16-column prepack tile) and, row-wise, the block size."""
    return 32 if col_wise else max(32, block_size)


def shard_bounds(out_features: int, world_size: int, rank: int, block_size: int, col_wise: bool):
    """[n0, n1) of `rank`.  Requires an even split into legal shard widths."""
    if out_features % world_size != 0:
        raise ValueError(f"out_features {out_features} does not split evenly over {world_size} ranks")
    ns = out_features // world_size
    mult = shard_multiple(block_size, col_wise)
    if ns % mult != 0:
        raise ValueError(f"shard width {ns} is not a multiple of {mult} (block {block_size}, col_wise={col_wise})")
    return rank * ns, (rank + 1) * ns


def gather_columns(local_out: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather [M, N/g] shards into [M, N] (concatenation along the last dim)."""
    g = dist.get_world_size(group)
    if g == 1:
        return local_out
    M, ns = local_out.shape
    # rank r's [M, ns] block lands at rows [r*M, (r+1)*M) of the gather buffer
    stacked = torch.empty((g * M, ns), dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(stacked, local_out.contiguous(), group=group)
    if M == 1:
        return stacked.view(1, g * ns)
    return stacked.view(g, M, ns).permute(1, 0, 2).reshape(M, g * ns)


class PeerGather:
    """This rank's exchange block for the fused GEMM + all-gather, connected to all peers.

    Collective: every rank of ``group`` must construct it at the same point.  The 64-byte IPC
    handles travel through ``all_gather_object`` on the group; after that the data path uses no
    collective library.
    """

    def __init__(self, max_rows: int, out_features: int, group=None):
        from . import capi

        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.max_rows, self.out_features = int(max_rows), int(out_features)
        self.ctx = capi.GatherContext(self.world, self.rank, self.max_rows * self.out_features * 2)
        handles = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, self.ctx.handle, group=group)
        else:
            handles[0] = self.ctx.handle
        error = None
        try:
            self.ctx.connect(handles)
        except Exception as exc:  # noqa: BLE001  (reported on every rank below)
            error = exc
        if self.world > 1:
            # Doubles as the barrier "nobody stores into a block before everybody has mapped it";
            # a rank that could not map its peers must not leave the others waiting in a collective.
            flags = [None] * self.world
            dist.all_gather_object(flags, error is None, group=group)
            if not all(flags):
                self.ctx.close()
                raise RuntimeError("PeerGather: mapping the peers' exchange blocks failed on rank(s) "
                                   + ", ".join(str(r) for r, ok in enumerate(flags) if not ok)
                                   + (f" (here: {error})" if error is not None else ""))
        elif error is not None:
            raise error

    def supports(self, layer, rows: int) -> bool:
        """Shapes the fused kernels take (the library refuses the others): decode and skinny shapes
        up to 16 rows, and prefill shapes on the CTA-pair tensor-core kernel."""
        from . import capi

        if rows > self.max_rows or layer.out_features * self.world != self.out_features:
            return False
        if rows > 16 and self.world > int(os.environ.get("BLKQ4_GATHER_PREFILL_MAX_RANKS", "4")):
            return False  # the prefill path's peer stores do not scale to eight destinations (measured)
        return capi.gather_supported(layer.block_size, layer.col_wise, rows, layer.out_features, layer.in_features)

    def forward(self, layer, x, out_full, flags=0):
        """``out_full[M, N] = x[M, K] @ W^T`` with this rank computing its ``layer``'s columns."""
        from . import capi

        stream = torch.cuda.current_stream(x.device).cuda_stream
        self.ctx.gemm(layer.block_size, layer.col_wise, x.size(0), layer.out_features, layer.in_features,
                      x, layer.q_weights, layer.q_scales, layer.q_zp if layer.has_offsets else None,
                      out_full, stream=stream, flags=flags)
        return out_full

    def status(self) -> int:
        return self.ctx.status()

    def close(self):
        """Collective: every rank drains its device, then all meet at a barrier, and only then are the
        exchange blocks unmapped and freed - a peer's kernel may store into this rank's block until
        that peer has drained.  Safe to call twice."""
        if getattr(self, "ctx", None) is None:
            return
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        if self.world > 1 and dist.is_initialized():
            dist.barrier(self.group)
        self.ctx.close()
        self.ctx = None


class ShardedBlkQ4Linear(nn.Module):
    """``BlkQ4Linear`` whose out_features are split over the ranks of ``process_group``.

    ``weights`` is either the full [N, K] weight (each rank slices its rows) or,
    with ``weights_are_local=True``, this rank's [N/g, K] shard.
    """

    def __init__(self, block_size, col_wise, scale_only, weights, bias_tensor=None, process_group=None,
                 weights_are_local=False, gather_output=True, peer_gather=None):
        super().__init__()
        from .ms_blkq4linear import BlkQ4Linear

        self.group = process_group
        self.world_size = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        self.gather_output = gather_output
        if weights_are_local:
            local = weights
            self.out_features = weights.size(0) * self.world_size
            self.n0 = self.rank * weights.size(0)
        else:
            self.out_features = weights.size(0)
            self.n0, n1 = shard_bounds(self.out_features, self.world_size, self.rank, block_size, col_wise)
            local = weights[self.n0:n1].contiguous()
        self.in_features = weights.size(1)
        self.local = BlkQ4Linear(block_size, col_wise, scale_only, local)
        self.bias = bias_tensor  # full-width bias, added after the gather
        # A PeerGather shared by the layers of a model (its buffers serve one call at a time):
        # skinny inputs on CUDA then take the fused kernel instead of compute + NCCL all-gather.
        self.peer_gather = peer_gather

    def forward(self, input, out=None):
        lead = input.shape[:-1]
        x = input.reshape(-1, self.in_features)
        pg = self.peer_gather
        if (self.gather_output and pg is not None and x.is_cuda and pg.supports(self.local, x.size(0))):
            full = out if out is not None else torch.empty(x.size(0), self.out_features, dtype=torch.float16,
                                                           device=x.device)
            lyr = self.local
            flags = 1 if (lyr.early_weight_fetch and lyr._settled) else 0
            pg.forward(lyr, x, full.view(-1, self.out_features), flags)
            lyr._settled = True
            if self.bias is not None:
                full += self.bias
            return full.view(*lead, self.out_features)
        if not self.gather_output:
            # the caller's buffer, if any, receives this rank's columns
            local_out = None if out is None else out.view(-1, self.local.out_features)
            res = self.local(x, out=local_out)
            return res.view(*lead, -1)
        res = gather_columns(self.local(x), self.group)
        if self.bias is not None:
            res += self.bias
        if out is not None:
            # a caller that reads its own buffer (a captured graph, a LinearStack) must find the result there
            out.view(-1, self.out_features).copy_(res)
            return out.view(*lead, self.out_features)
        return res.view(*lead, self.out_features)
