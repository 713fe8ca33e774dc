"""On-disk format for quantized + prepacked layers, so that quantization is paid once.

The reference has no serialization (its module re-quantizes from fp16 in the
constructor, python/ms_blkq4linear.py:11-22).  A file holds one or more layers:

    magic   8 bytes  b"BLKQ4PK1"
    count   uint32   number of layers
    per layer:
        name_len uint32, name utf-8
        block uint32, col_wise uint8, has_zp uint8, has_bias uint8, pad uint8
        K uint64 (in_features), N uint64 (out_features)
        q_weights  K*N/2 bytes         packed int4, the layout blkq4_fp16_gemm_sm80 consumes
        q_scales   2*meta bytes        fp16, meta = (K/bk)*(N/bn)
        q_zp       meta bytes          only if has_zp
        bias       2*N bytes (fp16)    only if has_bias

All integers little-endian.  The arrays are exactly what ``blkq4_fp16_quant_sm80`` wrote,
so a file written on one machine loads on another without touching the quantizer, and a
C caller can read it with three ``fread`` calls per layer.  Sizes are checked on load
against the header (the same formulas as ``blkq4_fp16_quant_size_sm80``).
"""
from __future__ import annotations

import struct
from typing import BinaryIO, Dict, Iterable, Tuple

import torch

MAGIC = b"BLKQ4PK1"


def expected_sizes(block: int, col_wise: bool, K: int, N: int) -> Tuple[int, int]:
    """(packed weight bytes, meta entries): include/ms_blkq4gemm.h, blkq4_fp16_quant_size_sm80."""
    bk, bn = (block, 1) if col_wise else (1, block)
    if K % bk or N % bn or K % 2:
        raise ValueError(f"shape {K}x{N} does not hold whole blocks of {block}")
    return (K // 2) * N, (K // bk) * (N // bn)


def _write_tensor(f: BinaryIO, t: torch.Tensor):
    f.write(t.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes())


def _read_exact(f: BinaryIO, n: int) -> bytes:
    b = f.read(n)
    if len(b) != n:
        raise ValueError("truncated file")
    return b


def save_packed(path, layers: Dict[str, "object"] | Iterable[Tuple[str, "object"]]):
    """Write ``{name: BlkQ4Linear}`` (anything with block_size, col_wise, in_features,
    out_features, q_weights, q_scales, q_zp, bias) to ``path``."""
    items = list(layers.items()) if isinstance(layers, dict) else list(layers)
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<I", len(items)))
        for name, lyr in items:
            K, N = int(lyr.in_features), int(lyr.out_features)
            wb, meta = expected_sizes(lyr.block_size, lyr.col_wise, K, N)
            has_zp = lyr.q_zp is not None and lyr.q_zp.numel() > 0
            bias = getattr(lyr, "bias", None)
            if lyr.q_weights.numel() != wb or lyr.q_scales.numel() != meta or (has_zp and lyr.q_zp.numel() != meta):
                raise ValueError(f"layer {name!r}: tensor sizes do not match its shape")
            nb = name.encode()
            f.write(struct.pack("<I", len(nb)) + nb)
            f.write(struct.pack("<IBBBBQQ", lyr.block_size, int(lyr.col_wise), int(has_zp), int(bias is not None), 0, K, N))
            _write_tensor(f, lyr.q_weights)
            _write_tensor(f, lyr.q_scales.to(torch.float16))
            if has_zp:
                _write_tensor(f, lyr.q_zp)
            if bias is not None:
                if bias.numel() != N:
                    raise ValueError(f"layer {name!r}: bias has {bias.numel()} entries, expected {N}")
                _write_tensor(f, bias.to(torch.float16))


def load_packed_tensors(path):
    """-> ``{name: dict(block_size, col_wise, in_features, out_features, q_weights, q_scales,
    q_zp, bias)}`` with CPU tensors.  No device, no quantizer involved."""
    out = {}
    with open(path, "rb") as f:
        if _read_exact(f, 8) != MAGIC:
            raise ValueError("not a BLKQ4PK1 file")
        (count,) = struct.unpack("<I", _read_exact(f, 4))
        for _ in range(count):
            (nl,) = struct.unpack("<I", _read_exact(f, 4))
            name = _read_exact(f, nl).decode()
            block, cw, has_zp, has_bias, _pad, K, N = struct.unpack("<IBBBBQQ", _read_exact(f, 24))
            if block not in (16, 32, 64, 128):
                raise ValueError(f"layer {name!r}: unsupported block size {block}")
            wb, meta = expected_sizes(block, bool(cw), K, N)
            qw = torch.frombuffer(bytearray(_read_exact(f, wb)), dtype=torch.uint8)
            qs = torch.frombuffer(bytearray(_read_exact(f, 2 * meta)), dtype=torch.float16)
            qz = torch.frombuffer(bytearray(_read_exact(f, meta)), dtype=torch.uint8) if has_zp \
                else torch.empty(0, dtype=torch.uint8)
            bias = torch.frombuffer(bytearray(_read_exact(f, 2 * N)), dtype=torch.float16) if has_bias else None
            out[name] = dict(block_size=block, col_wise=bool(cw), in_features=K, out_features=N,
                             q_weights=qw, q_scales=qs, q_zp=qz, bias=bias)
        if f.read(1):
            raise ValueError("trailing bytes after the last layer")
    return out


def load_packed(path, device="cuda"):
    """-> ``{name: BlkQ4Linear}`` on ``device``, rebuilt with ``BlkQ4Linear.from_packed``."""
    from .ms_blkq4linear import BlkQ4Linear

    layers = {}
    for name, d in load_packed_tensors(path).items():
        bias = d["bias"].to(device) if d["bias"] is not None else None
        layers[name] = BlkQ4Linear.from_packed(
            d["block_size"], d["col_wise"], d["in_features"], d["out_features"],
            d["q_weights"].to(device), d["q_scales"].to(device), d["q_zp"].to(device), bias)
    return layers
