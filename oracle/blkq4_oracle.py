"""ctypes binding of the CPU oracle (oracle/blkq4_oracle.c).  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this module.  It exists for the test
suite, the smoke check and the benchmark's CPU-baseline leg, as the checker the
CUDA path is compared with.

All arrays are numpy; fp16 data travels as ``np.float16`` (viewed as uint16 at
the C boundary).  Layout names follow the C file's header comment.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libblkq4_oracle.so")
_REF_HOST_PATH = os.path.join(_HERE, "_ref", "libblkq4_ref_host.so")
_REF_GPU_PATH = os.path.join(_HERE, "_ref", "libms_blkq4gemm_ref.so")

_u8p = ctypes.POINTER(ctypes.c_uint8)
_u16p = ctypes.POINTER(ctypes.c_uint16)


def build(targets=("oracle",)) -> None:
    """Run the oracle Makefile for the given targets (gcc / g++ / nvcc only)."""
    subprocess.check_call(["make", "-s", "-C", _HERE, *targets])


def _load():
    if not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(
        os.path.join(_HERE, "blkq4_oracle.c")
    ):
        build(("oracle",))
    return ctypes.CDLL(_LIB_PATH)


_lib = _load()


def _p8(a):
    return None if a is None else a.ctypes.data_as(_u8p)


def _p16(a):
    return None if a is None else a.view(np.uint16).ctypes.data_as(_u16p)


def num_threads() -> int:
    return int(_lib.blkq4_oracle_num_threads())


def set_num_threads(n: int) -> int:
    """Set the OpenMP thread count of the oracle's loops (launchers may have exported
    OMP_NUM_THREADS=1); returns the count now in effect."""
    _lib.blkq4_oracle_set_num_threads(int(n))
    return num_threads()


def host_cores() -> int:
    """Cores this process may run on."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def blocking(block: int, colwise: bool):
    return (block, 1) if colwise else (1, block)


def quant_size(block: int, colwise: bool, K: int, N: int):
    """(packed weight bytes, meta element count), or raises ValueError."""
    w, m = ctypes.c_int64(0), ctypes.c_int64(0)
    rc = _lib.blkq4_oracle_quant_size(block, int(colwise), K, N, ctypes.byref(w), ctypes.byref(m))
    if rc != 0:
        raise ValueError(f"cannot block quantize {K}x{N} with block {block}")
    return w.value, m.value


def quantize_plain(block, colwise, w_nk: np.ndarray, has_zp: bool):
    """Stage 1.  ``w_nk``: fp16 [N, K] C-contiguous (PyTorch Linear.weight layout).

    Returns (q_plain u8 [K/2*N], scales fp16 [meta] column-major, zp u8 or None).
    """
    assert w_nk.dtype == np.float16 and w_nk.ndim == 2 and w_nk.strides[1] == 2
    N, K = w_nk.shape
    ld = w_nk.strides[0] // 2
    wb, me = quant_size(block, colwise, K, N)
    q = np.empty(wb, np.uint8)
    s = np.empty(me, np.float16)
    z = np.empty(me, np.uint8) if has_zp else None
    _lib.blkq4_oracle_quantize_plain(block, int(colwise), K, N, ld, _p16(w_nk), _p8(q), _p16(s), _p8(z))
    return q, s, z


def prepack_weights(K, N, q_plain):
    out = np.empty_like(q_plain)
    _lib.blkq4_oracle_prepack_weights(K, N, _p8(q_plain), _p8(out))
    return out


def prepack_meta(block, colwise, K, N, scales_cm, zp_cm):
    s = np.empty_like(scales_cm)
    z = np.empty_like(zp_cm) if zp_cm is not None else None
    _lib.blkq4_oracle_prepack_meta(block, int(colwise), K, N, _p16(scales_cm), _p8(zp_cm), _p16(s), _p8(z))
    return s, z


def quant_prepack(block, colwise, w_nk: np.ndarray, has_zp: bool):
    """Quantize + prepack: what ``blkq4_fp16_quant_sm80`` hands its caller.

    Returns (packed u8 [K*N/2], scales fp16 [meta], zp u8 [meta] or None).
    """
    N, K = w_nk.shape
    q, s, z = quantize_plain(block, colwise, w_nk, has_zp)
    ps, pz = prepack_meta(block, colwise, K, N, s, z)
    return prepack_weights(K, N, q), ps, pz


def dequant(block, colwise, K, N, packed, scales, zp, kernel_formula: bool = False):
    """Packed form -> fp16 [N, K] (i.e. column-major K x N)."""
    out = np.empty((N, K), np.float16)
    _lib.blkq4_oracle_dequant(
        block, int(colwise), K, N, _p8(packed), _p16(scales), _p8(zp), int(kernel_formula), _p16(out)
    )
    return out


def dequant_ideal(block, colwise, K, N, packed, scales, zp):
    """Packed form -> float64 [N, K] of scale * (q - zp) with no fp16 rounding at all:
    the value both fp16 dequantization formulas approximate."""
    bk, bn = blocking(block, colwise)
    k = np.arange(K)
    n = np.arange(N)
    kk, nn = k % 16, n % 16
    kp = 16 * (k // 16) + 4 * ((kk % 8) // 2) + 2 * (kk & 1)          # + nhi
    np_ = 8 * (n // 16) + nn % 8
    byte = packed.reshape(N // 2, K)[np_[:, None], kp[None, :] + (nn // 8)[:, None]]
    q = np.where((kk // 8)[None, :] == 1, byte >> 4, byte & 0xF).astype(np.int64)
    if colwise:
        mi = (k // block)[None, :] * N + n[:, None]
        mi_z = mi
    else:
        r = k % 16
        t, hi, odd = (r % 8) // 2, r // 8, r & 1
        base = (n // block)[:, None] * K + (k // 16 * 16)[None, :]
        mi = base + (4 * t + 2 * hi + odd)[None, :]
        mi_z = base + (4 * t + 2 * odd + hi)[None, :]
    s = scales.astype(np.float64)[mi]
    z = zp.astype(np.int64)[mi_z] if zp is not None else 8
    return s * (q - z)


def gemm(a_mk: np.ndarray, wdq_nk: np.ndarray):
    """fp16 [M,K] x fp16 [N,K]^T -> fp16 [M,N], fp32 accumulation."""
    M, K = a_mk.shape
    N = wdq_nk.shape[0]
    a_mk = np.ascontiguousarray(a_mk)
    wdq_nk = np.ascontiguousarray(wdq_nk)
    c = np.empty((M, N), np.float16)
    _lib.blkq4_oracle_gemm(M, N, K, _p16(a_mk), _p16(wdq_nk), _p16(c))
    return c


def dequant_gemm(block, colwise, a_mk, N, packed, scales, zp, kernel_formula: bool = False):
    M, K = a_mk.shape
    return gemm(a_mk, dequant(block, colwise, K, N, packed, scales, zp, kernel_formula))


def kat_generate(block, colwise, K, N, has_zp: bool = True):
    """The reference tests' known-answer weights: (q_plain, scales_cm, zp_cm)."""
    wb, me = quant_size(block, colwise, K, N)
    q = np.empty(wb, np.uint8)
    s = np.empty(me, np.float16)
    z = np.empty(me, np.uint8) if has_zp else None
    _lib.blkq4_oracle_kat_generate(block, int(colwise), K, N, _p8(q), _p16(s), _p8(z))
    return q, s, z


def dequant_plain(block, colwise, K, N, q_plain, scales_cm, zp_cm):
    out = np.empty((N, K), np.float16)
    _lib.blkq4_oracle_dequant_plain(block, int(colwise), K, N, _p8(q_plain), _p16(scales_cm), _p8(zp_cm), _p16(out))
    return out


def kat_activations(M, K, seed=1):
    """Quarter-integers in [-4, 4]: the value family of the reference GEMM test's
    activations (uniform in [-4, 4] with 2 fractional bits), for which every
    product and partial sum is exact in fp32."""
    rng = np.random.default_rng(seed)
    return (rng.integers(-16, 17, size=(M, K)) / 4.0).astype(np.float16)


# --------------------------------------------------------------------------
# The reference's own code, when it has been built here (oracle/_ref/).


def have_ref_host() -> bool:
    return os.path.exists(_REF_HOST_PATH)


def have_ref_gpu() -> bool:
    return os.path.exists(_REF_GPU_PATH)


def ref_gpu_path() -> str:
    return _REF_GPU_PATH


def ref_host_prepack(block, colwise, K, N, q_plain, scales_cm, zp_cm):
    """Run the reference's host prepack helpers on plain-form inputs.

    The helpers take meta in the reference's LayoutQmeta (row-major when
    column-wise); the column-major -> LayoutQmeta transpose done here is the
    non-permuting part of the reference's meta prepack.
    """
    lib = ctypes.CDLL(_REF_HOST_PATH)
    packed = np.empty_like(q_plain)
    assert lib.ref_prepack_weights(K, N, _p8(q_plain), _p8(packed)) == 0
    bk, bn = blocking(block, colwise)
    mr, mc = K // bk, N // bn

    def to_qmeta(a):
        if a is None:
            return None
        return np.ascontiguousarray(a.reshape(mc, mr).T).reshape(-1) if colwise else a.copy()

    s_in, z_in = to_qmeta(scales_cm), to_qmeta(zp_cm)
    s_out = np.empty_like(s_in)
    z_out = np.empty_like(z_in) if z_in is not None else None
    assert lib.ref_prepack_meta(block, int(colwise), K, N, _p16(s_in), _p16(s_out), _p8(z_in), _p8(z_out)) == 0
    return packed, s_out, z_out
