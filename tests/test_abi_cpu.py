"""CPU checks of the drop-in boundary: the library loads, exports every symbol the
header declares, and its host-side validation answers like the reference's."""
import ctypes
import os
import re

import pytest

from tests._util import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "ms_blkq4gemm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    return sorted(set(re.findall(r"\b(blkq4_\w+)\s*\(", text)))


def test_header_declares_the_reference_entry_points():
    syms = _declared_symbols()
    for s in ("blkq4_fp16_gemm_sm80", "blkq4_fp16_quant_sm80", "blkq4_fp16_quant_size_sm80"):
        assert s in syms


def test_library_exports_every_declared_symbol(lib_built):
    lib = ctypes.CDLL(lib_built)
    for s in _declared_symbols():
        assert hasattr(lib, s), f"{s} declared in include/ms_blkq4gemm.h but not exported"


def test_capi_symbol_list_matches_header(lib_built):
    from gemmlib_b200 import capi

    assert sorted(capi.SYMBOLS) == _declared_symbols()
    assert "sm_100a" in capi.version()


def test_quant_size_values(lib_built):
    from gemmlib_b200 import capi

    # reference get_quant_weights_shape / get_quant_meta_shape (f16_quant_sm80.cuh:190-198)
    assert capi.quant_size(32, True, 4096, 4096) == (8388608, 524288)
    assert capi.quant_size(64, True, 4096, 11008) == (22544384, 704512)
    assert capi.quant_size(32, False, 64, 32) == (1024, 64)
    assert capi.quant_size(128, True, 8192, 28672) == (117440512, 1835008)


@pytest.mark.parametrize(
    "args,msg",
    [
        ((8, True, 64, 32), "Unsupported block size: 8"),
        ((32, True, 0, 32), "Empty problem size: 0x32"),
        ((32, True, 96, 32), "Cannot block quantize matrix with rows: 96"),
        ((32, True, 64, 48), "Cannot block quantize matrix with columns: 48"),
        ((64, False, 64, 96), "Cannot block quantize matrix with columns: 96"),
        ((128, True, 192, 32), "Cannot block quantize matrix with rows: 192"),
    ],
)
def test_quant_size_errors(lib_built, args, msg):
    """Error texts of the reference dispatcher (src/blkq4_f16_gemm_sm80.cu:166,189,195,460)."""
    from gemmlib_b200 import capi

    with pytest.raises(capi.BlkQ4Error) as e:
        capi.quant_size(*args)
    assert str(e.value) == msg


def test_gemm_and_quant_reject_bad_sizes_before_touching_the_device(lib_built):
    """Size validation is host-side and comes first, so it can be checked without a GPU
    (pointers are never dereferenced on these paths)."""
    from gemmlib_b200 import capi

    M, N, K = 4, 32, 64
    fake = lambda nbytes: (0x1000, nbytes)  # noqa: E731  (pointer, byte size)
    with pytest.raises(capi.BlkQ4Error, match="Empty problem size: 0x32x64"):
        capi.gemm(32, True, 0, N, K, fake(0), fake(K * N // 2), fake(2 * 2 * N), None, fake(0))
    with pytest.raises(capi.BlkQ4Error, match="Unexpected activation tensor size: 10 expected: 512"):
        capi.gemm(32, True, M, N, K, fake(10), fake(K * N // 2), fake(2 * 2 * N), None, fake(2 * M * N))
    with pytest.raises(capi.BlkQ4Error, match="Unexpected weight tensor size"):
        capi.gemm(32, True, M, N, K, fake(2 * M * K), fake(7), fake(2 * 2 * N), None, fake(2 * M * N))
    with pytest.raises(capi.BlkQ4Error, match="Unexpected scale tensor size"):
        capi.gemm(32, True, M, N, K, fake(2 * M * K), fake(K * N // 2), fake(2), None, fake(2 * M * N))
    with pytest.raises(capi.BlkQ4Error, match="Unexpected output tensor size"):
        capi.gemm(32, True, M, N, K, fake(2 * M * K), fake(K * N // 2), fake(2 * 2 * N), None, fake(2))
    with pytest.raises(capi.BlkQ4Error, match="Unexpected offsets tensor size"):
        capi.gemm(32, True, M, N, K, fake(2 * M * K), fake(K * N // 2), fake(2 * 2 * N), fake(3), fake(2 * M * N))
    with pytest.raises(capi.BlkQ4Error, match="Unsupported block size: 48"):
        capi.gemm(48, True, M, N, K, fake(2 * M * K), fake(K * N // 2), fake(2 * 2 * N), None, fake(2 * M * N))
    with pytest.raises(capi.BlkQ4Error, match="Unexpected quantized weight tensor size: 5 expected: 1024"):
        capi.quant(32, True, K, N, K, fake(2 * K * N), fake(5), fake(2 * 2 * N), None)
    with pytest.raises(capi.BlkQ4Error, match="Unexpected scale tensor size"):
        capi.quant(32, True, K, N, K, fake(2 * K * N), fake(K * N // 2), fake(2), None)
    with pytest.raises(capi.BlkQ4Error, match="Unexpected offset tensor size"):
        capi.quant(32, True, K, N, K, fake(2 * K * N), fake(K * N // 2), fake(2 * 2 * N), fake(1))
    with pytest.raises(capi.BlkQ4Error, match="Unexpected weight tensor size"):
        capi.quant(32, True, K, N, K, fake(10), fake(K * N // 2), fake(2 * 2 * N), None)


def test_extension_entry_points_validate_on_the_host(lib_built):
    """The entry points without a reference counterpart check their extra arguments before any
    device work too: bias size, workspace planning, static scratch limit, gather arguments."""
    import ctypes as C

    from gemmlib_b200 import capi

    M, N, K = 4, 32, 64
    fake = lambda nbytes: (0x1000, nbytes)  # noqa: E731
    with pytest.raises(capi.BlkQ4Error, match="Unexpected bias tensor size: 6 expected: 64"):
        capi.gemm(32, True, M, N, K, fake(2 * M * K), fake(K * N // 2), fake(2 * 2 * N), None, fake(2 * M * N),
                  bias=fake(6))
    with pytest.raises(capi.BlkQ4Error, match="Bias tensor must be 4-byte aligned"):
        capi.gemm(32, True, M, N, K, fake(2 * M * K), fake(K * N // 2), fake(2 * 2 * N), None, fake(2 * M * N),
                  bias=(0x1002, 2 * N))
    # split-K planning is a pure host function (it falls back to 148 SMs without a device)
    assert capi.gemm_workspace_size(512, 4096, 4096) == 256 + 64 * 256 * 128 * 4
    assert capi.gemm_workspace_size(2048, 4096, 4096) == 0
    assert capi.gemm_workspace_size(16, 4096, 4096) == 0
    assert capi.gemm_workspace_size(512, 4096, 512) == 0           # too few k steps per part
    assert capi.gemm_workspace_size(512, 4096, 100) == 0           # not a GEMM shape
    assert capi.static_scratch_size() == 12 << 20
    with pytest.raises(capi.BlkQ4Error, match="exceeds the static scratch"):
        capi.gemm_static_ws(64, True, 256, 4096, 4096, fake(2 * 256 * 4096), fake(4096 * 4096 // 2),
                            fake(2 * 64 * 4096), None, fake(2 * 256 * 4096))
    # gather: argument checks that come before any allocation
    ctx, handle = C.c_void_p(), C.create_string_buffer(64)
    err = capi.lib.blkq4_errmsg_create()
    try:
        assert capi.lib.blkq4_gather_create(9, 0, 1024, C.byref(ctx), handle, err) == -1
        assert b"Unsupported world size" in capi.lib.blkq4_errmsg_cstr(err)
        assert capi.lib.blkq4_gather_create(2, 2, 1024, C.byref(ctx), handle, err) == -1
        assert capi.lib.blkq4_gather_create(2, 0, 0, C.byref(ctx), handle, err) == -1
        assert capi.lib.blkq4_fp16_gemm_gather_sm100(None, 64, True, 1, 32, 512, None, None, 0, None, 0, None, 0,
                                                     None, 0, None, 0, 0, err) == -1
        assert b"Null gather context" in capi.lib.blkq4_errmsg_cstr(err)
    finally:
        capi.lib.blkq4_errmsg_destroy(err)
