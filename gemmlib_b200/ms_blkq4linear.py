"""``BlkQ4Linear``: blockwise-int4 weight-only linear layer.

Mirror of the reference module python/ms_blkq4linear.py:10-28: same class name,
constructor arguments ``(block_size, col_wise, scale_only, weights,
bias_tensor=None)``, attributes and ``forward(input)``.  Quantization and prepack
happen in the constructor (on the device the weights live on); ``forward`` runs the
W4A16 GEMM/GEMV and adds the bias.

Additive differences: the packed tensors are registered as buffers, so they travel
with ``state_dict()`` / ``.to()``; the constructor's diagnostic prints are gone;
``from_packed`` rebuilds a layer from already-quantized tensors; inputs with leading
batch dimensions are flattened to 2-D and restored; ``forward(input, out=...)`` writes
into a caller's tensor; a float16 bias on the layer's device is added inside the kernel's
epilogue (bit-identical to the reference's separate ``output += bias``, one pass over the
output less); and, from the second call on, the skinny kernel is launched with
``BLKQ4_GEMM_EARLY_WEIGHT_FETCH`` (set ``early_weight_fetch = False`` on a layer whose
packed tensors are rewritten by work queued on the same stream as ``forward``); prefill
shapes with too few output tiles to fill the GPU split K through a workspace shared per
(device, stream) (``split_k = False`` turns that off).
"""
from __future__ import annotations

import torch
from torch import nn

from . import ms_blkq4linear_ext


# Split-K workspaces: one zero-initialised buffer per (device, stream), shared by all layers (calls
# on one stream run one at a time; the kernel leaves the buffer's flags zeroed).  Grown on demand.
_WORKSPACES = {}


def split_k_workspace(device, nbytes: int):
    if nbytes <= 0:
        return None
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 16 << 20), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


class BlkQ4Linear(nn.Module):
    def __init__(self, block_size, col_wise, scale_only, weights, bias_tensor=None):
        super().__init__()
        self.block_size = int(block_size)
        self.col_wise = bool(col_wise)
        self.has_offsets = not scale_only
        self.in_features = weights.size(1)
        self.out_features = weights.size(0)
        q_weights, q_scales, q_zp = ms_blkq4linear_ext.quant(
            self.block_size, self.col_wise, self.has_offsets, weights
        )
        self.register_buffer("q_weights", q_weights)
        self.register_buffer("q_scales", q_scales)
        self.register_buffer("q_zp", q_zp)
        self.bias = bias_tensor
        self.early_weight_fetch = True
        self.split_k = True  # prefill shapes with few output tiles split K through a shared workspace
        self._settled = False  # the first forward is a plain launch, ordered after the quantizer

    @classmethod
    def from_packed(cls, block_size, col_wise, in_features, out_features, q_weights, q_scales, q_zp=None,
                    bias_tensor=None):
        """Build a layer from tensors produced earlier by ``quant`` (no requantization)."""
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        self.block_size, self.col_wise = int(block_size), bool(col_wise)
        self.in_features, self.out_features = int(in_features), int(out_features)
        if q_zp is None:
            q_zp = torch.empty(0, dtype=torch.uint8, device=q_weights.device)
        self.has_offsets = q_zp.numel() > 0
        self.register_buffer("q_weights", q_weights)
        self.register_buffer("q_scales", q_scales)
        self.register_buffer("q_zp", q_zp)
        self.bias = bias_tensor
        self.early_weight_fetch = True
        self.split_k = True  # prefill shapes with few output tiles split K through a shared workspace
        self._settled = False
        return self

    def _load_from_state_dict(self, *args, **kwargs):
        self._settled = False  # the buffers are about to be overwritten by a copy on some stream
        return super()._load_from_state_dict(*args, **kwargs)

    def _fusable_bias(self, x):
        b = self.bias
        if (b is not None and b.dtype == torch.float16 and b.device == x.device and b.dim() == 1
                and b.numel() == self.out_features and b.is_contiguous()):
            return b
        return None

    def forward(self, input, out=None):
        lead = input.shape[:-1]
        x = input.reshape(-1, self.in_features)
        if out is None:
            output = torch.empty(x.size(0), self.out_features, dtype=torch.float16, device=x.device)
        else:
            output = out.view(-1, self.out_features)
        fused = self._fusable_bias(x)
        flags = ms_blkq4linear_ext.EARLY_WEIGHT_FETCH if (self.early_weight_fetch and self._settled) else 0
        ws = None
        if x.size(0) > 16 and self.split_k:
            ws = split_k_workspace(x.device, ms_blkq4linear_ext.gemm_workspace_size(
                x.size(0), self.out_features, self.in_features))
        ms_blkq4linear_ext.forward_out(
            self.block_size, self.col_wise, self.in_features, self.out_features,
            x, self.q_weights, self.q_scales, self.q_zp, output, fused, flags, ws)
        self._settled = True
        if self.bias is not None and fused is None:
            output += self.bias
        return output.view(*lead, self.out_features)

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.out_features}, block_size={self.block_size}, "
                f"col_wise={self.col_wise}, has_offsets={self.has_offsets}, bias={self.bias is not None}")
