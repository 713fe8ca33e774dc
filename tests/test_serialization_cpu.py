"""The packed-layer file format: round trip, size checks, corruption handling (CPU only:
the format is bytes in, bytes out; the oracle provides quantized tensors to store)."""
import types

import numpy as np
import pytest

from oracle import blkq4_oracle as O
from tests._util import gaussian_weight

torch = pytest.importorskip("torch")


def fake_layer(block, colwise, has_zp, N, K, bias=False, seed=0):
    w = gaussian_weight(N, K, seed=seed)
    pw, ps, pz = O.quant_prepack(block, colwise, w.numpy(), has_zp)
    return types.SimpleNamespace(
        block_size=block, col_wise=colwise, in_features=K, out_features=N,
        q_weights=torch.from_numpy(pw.copy()), q_scales=torch.from_numpy(ps.copy()),
        q_zp=torch.from_numpy(pz.copy()) if pz is not None else torch.empty(0, dtype=torch.uint8),
        bias=torch.linspace(-1, 1, N).half() if bias else None)


def test_round_trip_is_bit_exact(tmp_path):
    from gemmlib_b200 import serialization as S

    layers = {
        "blocks.0.q": fake_layer(64, True, False, 128, 256, seed=1),
        "blocks.0.down": fake_layer(32, False, True, 96, 192, bias=True, seed=2),
        "odd name/ü": fake_layer(128, True, True, 64, 256, seed=3),
    }
    p = tmp_path / "m.blkq4"
    S.save_packed(p, layers)
    got = S.load_packed_tensors(p)
    assert list(got) == list(layers)
    for name, lyr in layers.items():
        g = got[name]
        assert (g["block_size"], g["col_wise"], g["in_features"], g["out_features"]) == \
            (lyr.block_size, lyr.col_wise, lyr.in_features, lyr.out_features)
        assert torch.equal(g["q_weights"], lyr.q_weights)
        assert torch.equal(g["q_scales"].view(torch.int16), lyr.q_scales.view(torch.int16))
        assert torch.equal(g["q_zp"], lyr.q_zp)
        assert (g["bias"] is None) == (lyr.bias is None)
        if lyr.bias is not None:
            assert torch.equal(g["bias"], lyr.bias)
    # header sizes follow the library's own size query
    wb, meta = S.expected_sizes(64, True, 256, 128)
    assert (wb, meta) == O.quant_size(64, True, 256, 128)


def test_rejects_bad_files(tmp_path):
    from gemmlib_b200 import serialization as S

    p = tmp_path / "m.blkq4"
    S.save_packed(p, {"a": fake_layer(64, True, True, 64, 128)})
    raw = p.read_bytes()
    (tmp_path / "trunc").write_bytes(raw[:-5])
    with pytest.raises(ValueError, match="truncated"):
        S.load_packed_tensors(tmp_path / "trunc")
    (tmp_path / "magic").write_bytes(b"NOTBLKQ4" + raw[8:])
    with pytest.raises(ValueError, match="BLKQ4PK1"):
        S.load_packed_tensors(tmp_path / "magic")
    (tmp_path / "extra").write_bytes(raw + b"x")
    with pytest.raises(ValueError, match="trailing"):
        S.load_packed_tensors(tmp_path / "extra")
    bad = fake_layer(64, True, True, 64, 128)
    bad.q_scales = bad.q_scales[:-1]
    with pytest.raises(ValueError, match="sizes"):
        S.save_packed(tmp_path / "bad", {"a": bad})
