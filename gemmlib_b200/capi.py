"""ctypes binding of the C ABI in ``include/ms_blkq4gemm.h``.

Arguments are raw device pointers (ints) and byte sizes, exactly as a C caller
would pass them; torch tensors are accepted for convenience and contribute their
``data_ptr()`` / byte size only.  Errors raise :class:`BlkQ4Error` carrying the
library's message.  Nothing here computes anything: if the shared library is
missing this module raises at import time.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libms_blkq4gemm.so")

SYMBOLS = (
    "blkq4_fp16_gemm_sm80",
    "blkq4_fp16_gemm_sm100",
    "blkq4_fp16_gemm_ws_sm100",
    "blkq4_gemm_workspace_size",
    "blkq4_fp16_gemm_static_ws_sm100",
    "blkq4_static_scratch_size",
    "blkq4_fp16_quant_sm80",
    "blkq4_fp16_quant_size_sm80",
    "blkq4_errmsg_create",
    "blkq4_errmsg_cstr",
    "blkq4_errmsg_destroy",
    "blkq4_last_kernel_status",
    "blkq4_gather_create",
    "blkq4_gather_connect",
    "blkq4_gather_local_block",
    "blkq4_gather_connect_pointers",
    "blkq4_fp16_gemm_gather_sm100",
    "blkq4_gather_status",
    "blkq4_gather_destroy",
    "blkq4_gather_reset",
    "blkq4_gather_supported_sm100",
    "blkq4_gemm_plan",
    "blkq4_gemm_plan_range_bound",
    "blkq4_reset",
    "blkq4_version",
)


class BlkQ4Error(RuntimeError):
    pass


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m gemmlib_b200.build` "
            "(there is no fallback implementation)"
        )
    lib = ctypes.CDLL(LIB_PATH)
    vp, sz, i, b = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_bool
    lib.blkq4_fp16_gemm_sm80.argtypes = [i, b, i, i, i, vp, vp, sz, vp, sz, vp, sz, vp, sz, vp, sz, vp]
    lib.blkq4_fp16_gemm_sm80.restype = i
    lib.blkq4_fp16_gemm_sm100.argtypes = [i, b, i, i, i, vp, vp, sz, vp, sz, vp, sz, vp, sz, vp, sz, vp, sz, ctypes.c_uint, vp]
    lib.blkq4_fp16_gemm_sm100.restype = i
    lib.blkq4_fp16_gemm_ws_sm100.argtypes = [i, b, i, i, i, vp, vp, sz, vp, sz, vp, sz, vp, sz, vp, sz, vp, sz,
                                             ctypes.c_uint, vp, sz, vp]
    lib.blkq4_fp16_gemm_ws_sm100.restype = i
    lib.blkq4_gemm_workspace_size.argtypes = [i, i, i]
    lib.blkq4_gemm_workspace_size.restype = sz
    lib.blkq4_fp16_gemm_static_ws_sm100.argtypes = [i, b, i, i, i, vp, vp, sz, vp, sz, vp, sz, vp, sz, vp, sz, vp, sz,
                                                    ctypes.c_uint, vp]
    lib.blkq4_fp16_gemm_static_ws_sm100.restype = i
    lib.blkq4_static_scratch_size.restype = sz
    lib.blkq4_fp16_quant_sm80.argtypes = [i, b, i, i, i, vp, vp, sz, vp, sz, vp, sz, vp, sz, vp]
    lib.blkq4_fp16_quant_sm80.restype = i
    i64p = ctypes.POINTER(ctypes.c_int64)  # int64_t& is passed as a pointer
    lib.blkq4_fp16_quant_size_sm80.argtypes = [i, b, i, i, i64p, i64p, vp]
    lib.blkq4_fp16_quant_size_sm80.restype = i
    lib.blkq4_errmsg_create.restype = vp
    lib.blkq4_errmsg_cstr.argtypes = [vp]
    lib.blkq4_errmsg_cstr.restype = ctypes.c_char_p
    lib.blkq4_errmsg_destroy.argtypes = [vp]
    lib.blkq4_version.restype = ctypes.c_char_p
    lib.blkq4_last_kernel_status.argtypes = [vp]
    lib.blkq4_last_kernel_status.restype = i
    lib.blkq4_gather_reset.argtypes = [vp]
    lib.blkq4_gather_reset.restype = i
    lib.blkq4_gather_supported_sm100.argtypes = [i, ctypes.c_bool, i, i, i]
    lib.blkq4_gather_supported_sm100.restype = i
    lib.blkq4_gemm_plan.argtypes = [i, i, i, sz, ctypes.POINTER(ctypes.c_int)]
    lib.blkq4_gemm_plan.restype = i
    lib.blkq4_gemm_plan_range_bound.argtypes = [i, i, i, i]
    lib.blkq4_gemm_plan_range_bound.restype = i
    lib.blkq4_reset.argtypes = [vp]
    lib.blkq4_reset.restype = i
    lib.blkq4_gather_create.argtypes = [i, i, sz, ctypes.POINTER(vp), vp, vp]
    lib.blkq4_gather_create.restype = i
    lib.blkq4_gather_connect.argtypes = [vp, vp, vp]
    lib.blkq4_gather_connect.restype = i
    lib.blkq4_gather_local_block.argtypes = [vp]
    lib.blkq4_gather_local_block.restype = vp
    lib.blkq4_gather_connect_pointers.argtypes = [vp, ctypes.POINTER(vp), vp]
    lib.blkq4_gather_connect_pointers.restype = i
    lib.blkq4_fp16_gemm_gather_sm100.argtypes = [vp, i, b, i, i, i, vp, vp, sz, vp, sz, vp, sz, vp, sz, vp, sz,
                                                 ctypes.c_uint, vp]
    lib.blkq4_fp16_gemm_gather_sm100.restype = i
    lib.blkq4_gather_status.argtypes = [vp, vp]
    lib.blkq4_gather_status.restype = i
    lib.blkq4_gather_destroy.argtypes = [vp]
    lib.blkq4_gather_destroy.restype = i
    return lib


lib = _load()


class _ErrMsg:
    def __enter__(self):
        self.p = lib.blkq4_errmsg_create()
        return self

    def __exit__(self, *exc):
        lib.blkq4_errmsg_destroy(self.p)

    def text(self) -> str:
        return lib.blkq4_errmsg_cstr(self.p).decode()


def _ptr_size(t):
    """(device pointer, byte size) of a torch tensor, or (0, 0) for None."""
    if t is None:
        return 0, 0
    if isinstance(t, tuple):
        return int(t[0]), int(t[1])
    n = t.numel() * t.element_size()
    return (t.data_ptr() if n else 0), n


def version() -> str:
    return lib.blkq4_version().decode()


def last_kernel_status(stream=0) -> int:
    """Synchronise ``stream`` and return the kernels' device status word (0 = no wait expired)."""
    return int(lib.blkq4_last_kernel_status(stream))


def quant_size(block_size: int, column_wise: bool, rows: int, columns: int):
    """-> (quant weight bytes, meta element count)."""
    w, m = ctypes.c_int64(0), ctypes.c_int64(0)
    with _ErrMsg() as e:
        rc = lib.blkq4_fp16_quant_size_sm80(
            block_size, column_wise, rows, columns, ctypes.byref(w), ctypes.byref(m), e.p
        )
        if rc != 0:
            raise BlkQ4Error(e.text())
    return w.value, m.value


def quant(block_size, column_wise, rows, columns, ld, weights, q_weights, q_scales, q_zp, stream=0):
    wp, ws = _ptr_size(weights)
    qp, qs = _ptr_size(q_weights)
    sp, ss = _ptr_size(q_scales)
    zp, zs = _ptr_size(q_zp)
    with _ErrMsg() as e:
        rc = lib.blkq4_fp16_quant_sm80(
            block_size, column_wise, rows, columns, ld, stream, wp, ws, qp, qs, sp, ss, zp, zs, e.p
        )
        if rc != 0:
            raise BlkQ4Error(e.text())


EARLY_WEIGHT_FETCH = 1  # BLKQ4_GEMM_EARLY_WEIGHT_FETCH


def gemm_workspace_size(m: int, n: int, k: int) -> int:
    """Bytes of zeroed workspace with which the tensor-core kernel would split K (0: it would not)."""
    return int(lib.blkq4_gemm_workspace_size(m, n, k))


def gather_supported(block_size: int, col_wise: bool, m: int, n_shard: int, k: int) -> bool:
    """Whether GatherContext.gemm takes the shape (fused GEMM + all-gather), else the caller computes
    locally and all-gathers with its own collective."""
    return bool(lib.blkq4_gather_supported_sm100(block_size, col_wise, m, n_shard, k))


def gemm_plan(m: int, n: int, k: int, workspace_size: int = 0) -> dict:
    """The work plan the tensor-core path would choose (host only; see blkq4_gemm_plan)."""
    out = (ctypes.c_int * 6)()
    if lib.blkq4_gemm_plan(m, n, k, workspace_size, out) != 0:
        raise BlkQ4Error(f"no plan for {m}x{n}x{k}")
    kernel = ("skinny", "one-cta", "pair")[out[0]]
    return {"kernel": kernel, "rows_per_tile": out[1], "tiles": out[2], "split": out[3], "balanced": bool(out[4]),
            "units": out[5]}


def gemm_plan_range_bound(total_steps: int, k_steps: int, units: int, b: int) -> int:
    return int(lib.blkq4_gemm_plan_range_bound(total_steps, k_steps, units, b))


def static_scratch_size() -> int:
    return int(lib.blkq4_static_scratch_size())


def gemm_static_ws(block_size, column_wise, m, n, k, act, q_weights, q_scales, q_zp, out, stream=0, flags=0,
                   bias=None):
    """``blkq4_fp16_gemm_static_ws_sm100``: split-K with the library's own device scratch array."""
    ap, as_ = _ptr_size(act)
    qp, qs = _ptr_size(q_weights)
    sp, ss = _ptr_size(q_scales)
    zp, zs = _ptr_size(q_zp)
    op, os_ = _ptr_size(out)
    bp, bs = _ptr_size(bias)
    with _ErrMsg() as e:
        rc = lib.blkq4_fp16_gemm_static_ws_sm100(
            block_size, column_wise, m, n, k, stream, ap, as_, qp, qs, sp, ss, zp, zs, op, os_, bp, bs, flags, e.p
        )
        if rc != 0:
            raise BlkQ4Error(e.text())


def gemm(block_size, column_wise, m, n, k, act, q_weights, q_scales, q_zp, out, stream=0, flags=0, bias=None,
         workspace=None):
    """Without ``flags`` and ``bias`` calls the reference-named entry point, otherwise
    ``blkq4_fp16_gemm_sm100``."""
    ap, as_ = _ptr_size(act)
    qp, qs = _ptr_size(q_weights)
    sp, ss = _ptr_size(q_scales)
    zp, zs = _ptr_size(q_zp)
    op, os_ = _ptr_size(out)
    bp, bs = _ptr_size(bias)
    wp, ws = _ptr_size(workspace)
    with _ErrMsg() as e:
        if ws:
            rc = lib.blkq4_fp16_gemm_ws_sm100(
                block_size, column_wise, m, n, k, stream, ap, as_, qp, qs, sp, ss, zp, zs, op, os_, bp, bs, flags,
                wp, ws, e.p
            )
        elif flags or bs:
            rc = lib.blkq4_fp16_gemm_sm100(
                block_size, column_wise, m, n, k, stream, ap, as_, qp, qs, sp, ss, zp, zs, op, os_, bp, bs, flags, e.p
            )
        else:
            rc = lib.blkq4_fp16_gemm_sm80(
                block_size, column_wise, m, n, k, stream, ap, as_, qp, qs, sp, ss, zp, zs, op, os_, e.p
            )
        if rc != 0:
            raise BlkQ4Error(e.text())


def reset(stream=0) -> None:
    """Clear the kernels' status words and the static scratch's flag words (``blkq4_reset``)."""
    if lib.blkq4_reset(stream) != 0:
        raise BlkQ4Error("blkq4_reset failed")


class GatherContext:
    """One rank's side of the fused GEMM + all-gather (``blkq4_gather_*``).

    ``handle`` (64 bytes) is this rank's IPC handle; collect the handles of all ranks, ordered
    by rank, and pass them to :meth:`connect` before the first :meth:`gemm`.
    """

    def __init__(self, world: int, rank: int, max_out_bytes: int):
        self.world, self.rank = int(world), int(rank)
        self._ctx = ctypes.c_void_p()
        buf = ctypes.create_string_buffer(64)
        with _ErrMsg() as e:
            if lib.blkq4_gather_create(world, rank, max_out_bytes, ctypes.byref(self._ctx), buf, e.p) != 0:
                raise BlkQ4Error(e.text())
        self.handle = bytes(buf.raw)

    def connect(self, handles):
        blob = b"".join(handles)
        if len(blob) != 64 * self.world:
            raise ValueError("need one 64-byte handle per rank")
        with _ErrMsg() as e:
            if lib.blkq4_gather_connect(self._ctx, blob, e.p) != 0:
                raise BlkQ4Error(e.text())

    def local_block(self) -> int:
        return int(lib.blkq4_gather_local_block(self._ctx) or 0)

    def connect_pointers(self, blocks):
        """Single process, several contexts: ``blocks[r]`` = ``local_block()`` of rank r's context."""
        arr = (ctypes.c_void_p * self.world)(*[ctypes.c_void_p(b) for b in blocks])
        with _ErrMsg() as e:
            if lib.blkq4_gather_connect_pointers(self._ctx, arr, e.p) != 0:
                raise BlkQ4Error(e.text())

    def gemm(self, block_size, column_wise, m, n_shard, k, act, q_weights, q_scales, q_zp, out_full, stream=0,
             flags=0):
        ap, as_ = _ptr_size(act)
        qp, qs = _ptr_size(q_weights)
        sp, ss = _ptr_size(q_scales)
        zp, zs = _ptr_size(q_zp)
        op, os_ = _ptr_size(out_full)
        with _ErrMsg() as e:
            rc = lib.blkq4_fp16_gemm_gather_sm100(
                self._ctx, block_size, column_wise, m, n_shard, k, stream, ap, as_, qp, qs, sp, ss, zp, zs,
                op, os_, flags, e.p)
            if rc != 0:
                raise BlkQ4Error(e.text())

    def status(self, stream=0) -> int:
        return int(lib.blkq4_gather_status(self._ctx, stream))

    def close(self):
        """Unmap the peers' blocks and free this rank's.  With more than one rank the caller must
        first have drained every rank's stream and passed a cross-rank barrier (PeerGather.close
        does both): peers store into this block from their own kernels."""
        if self._ctx:
            lib.blkq4_gather_destroy(self._ctx)
            self._ctx = ctypes.c_void_p()

    def reset(self):
        """After a wait that expired (status() != 0): clear the error word and the control words of
        this rank's block.  Collective in effect: every rank resets between the same two calls, with
        all streams drained."""
        if self._ctx and lib.blkq4_gather_reset(self._ctx) != 0:
            raise BlkQ4Error("blkq4_gather_reset failed")

    def __del__(self):
        # A garbage-collected context must not free memory that peers may still be storing into:
        # with several ranks only an explicit, ordered close() does that.
        try:
            if self.world <= 1:
                self.close()
            elif self._ctx:
                import warnings

                warnings.warn("GatherContext of a multi-rank exchange was dropped without close(); "
                              "its device block is left allocated", ResourceWarning)
        except Exception:
            pass
