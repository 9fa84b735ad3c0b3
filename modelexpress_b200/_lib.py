"""ctypes binding of ``libmxb200.so`` (the C ABI declared in ``include/mxb200.h``).

There is no CPU fallback: if the library is missing the import fails with
instructions to build it, and every compute call raises when CUDA reports an
error.
"""

from __future__ import annotations

import ctypes
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libmxb200.so")

OK = 0
ERR_NAMES = {-1: "MXB_ERR_ARG", -2: "MXB_ERR_BOUNDS", -3: "MXB_ERR_ALIGN", -4: "MXB_ERR_CUDA",
             -5: "MXB_ERR_TIMEOUT", -6: "MXB_ERR_PEER", -7: "MXB_ERR_NOMEM", -8: "MXB_ERR_STATE",
             -9: "MXB_ERR_UNSUPPORTED"}
MAX_DIMS = 8

DIGEST_SAFE32, DIGEST_ROWS, DIGEST_BLOCK64 = 1, 2, 4
SCATTER_DEFAULT, SCATTER_VECTOR, SCATTER_NO_SYNC, SCATTER_OVERLAP = 0, 1, 2, 4
PLACE_COPY_ENGINE, PLACE_ZERO_COPY = 0, 1
FANOUT_MAX_CHILDREN = 7

u64, u32, i32, i64 = ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int32, ctypes.c_int64


class Run(ctypes.Structure):
    _fields_ = [("src", u64), ("dst", u64), ("nbytes", u64)]


class Desc2D(ctypes.Structure):
    _fields_ = [("src", u64), ("dst", u64), ("rows", u64), ("row_bytes", u64),
                ("src_pitch", u64), ("dst_pitch", u64)]


class Span(ctypes.Structure):
    _fields_ = [("ptr", u64), ("nbytes", u64)]


class DigestOut(ctypes.Structure):
    _fields_ = [("nbytes", u64), ("row_sum", u64), ("row_sum_w", u64), ("tail_sum", u64),
                ("tail_sum_w", u64), ("ragged_sum", u64), ("block_hash", u64),
                ("safe_checksum", u32), ("reserved", u32)]


class Window(ctypes.Structure):
    _fields_ = [("ndim_src", i32), ("ndim_win", i32), ("keep_rank", i32), ("elsize", u32),
                ("global_shape", i64 * MAX_DIMS), ("win_offset", i64), ("win_shape", i64 * MAX_DIMS),
                ("win_stride", i64 * MAX_DIMS), ("dst_offset", i64), ("dst_stride", i64 * MAX_DIMS)]


class Shard(ctypes.Structure):
    _fields_ = [("ndim", i32), ("reserved", i32), ("offset", i64 * MAX_DIMS), ("shape", i64 * MAX_DIMS),
                ("addr", u64)]


class FanoutPiece(ctypes.Structure):
    _fields_ = [("range", u64), ("offset", u64), ("nbytes", u32), ("chunk", u32)]


class ConvertBox(ctypes.Structure):
    _fields_ = [("src", u64), ("dst", u64), ("ndim", u32), ("src_kind", u32), ("dst_kind", u32),
                ("elem_bytes", u32), ("extent", u64 * MAX_DIMS), ("dst_stride", i64 * MAX_DIMS),
                ("src_stride", i64 * MAX_DIMS)]


class ArenaBlock(ctypes.Structure):
    _fields_ = [("offset", u64), ("size", u64)]


class PlaceStats(ctypes.Structure):
    _fields_ = [("bytes_placed", u64), ("chunks", u64), ("launches", u64),
                ("seconds_total", ctypes.c_double), ("seconds_gather", ctypes.c_double),
                ("seconds_device", ctypes.c_double), ("bytes_direct", u64),
                ("seconds_plan", ctypes.c_double)]


# name -> (restype, argtypes); every symbol include/mxb200.h declares
_P = ctypes.POINTER
_vp = ctypes.c_void_p
SIGNATURES = {
    "mxb_ctx_create": (i32, [_P(i32), i32, _P(_vp)]),
    "mxb_ctx_destroy": (i32, [_vp]),
    "mxb_last_error": (ctypes.c_char_p, []),
    "mxb_version": (i32, []),
    "mxb_sync": (i32, [_vp, i32]),
    "mxb_launch_count": (u64, [_vp]),
    "mxb_alloc": (i32, [_vp, i32, u64, _P(u64)]),
    "mxb_free": (i32, [_vp, i32, u64]),
    "mxb_host_alloc": (i32, [u64, _P(u64)]),
    "mxb_host_free": (i32, [u64]),
    "mxb_host_register": (i32, [u64, u64, _P(u64), _P(u64)]),
    "mxb_host_unregister": (i32, [u64]),
    "mxb_host_is_pinned": (i32, [u64, u64]),
    "mxb_register_extent": (i32, [_vp, u64, u64]),
    "mxb_clear_extents": (i32, [_vp]),
    "mxb_ipc_export": (i32, [u64, _P(ctypes.c_uint8), _P(u64)]),
    "mxb_ipc_open": (i32, [_P(ctypes.c_uint8), u64, _P(u64)]),
    "mxb_ipc_close": (i32, [u64, u64]),
    "mxb_coalesce_runs": (i64, [_P(Run), u64, _P(Desc2D), u64]),
    "mxb_plan_pull": (i32, [_P(Window), _P(Shard), u64, u64, _P(Desc2D), _P(u32), u64, _P(u64)]),
    "mxb_plan_reshard": (i32, [_P(Desc2D), u64, u64, u64, u64, u64, _P(Desc2D), u64, _P(u64)]),
    "mxb_scatter": (i32, [_vp, i32, _P(Desc2D), u64, u32]),
    "mxb_read_runs": (i32, [_vp, i32, _P(Run), u64]),
    "mxb_table_create": (i32, [_vp, i32, _P(Desc2D), u64, _P(_vp)]),
    "mxb_table_launch": (i32, [_vp, u32]),
    "mxb_table_bytes": (u64, [_vp]),
    "mxb_table_engine": (i32, [_vp, u32]),
    "mxb_table_destroy": (i32, [_vp]),
    "mxb_copy_probe": (i32, [_vp, i32, u64, u64, u64, i32, _P(ctypes.c_float)]),
    "mxb_event_record": (i32, [_vp, i32, i32]),
    "mxb_event_elapsed": (i32, [_vp, i32, i32, i32, _P(ctypes.c_float)]),
    "mxb_ring_create": (i32, [_vp, i32, u64, u32, _P(_vp)]),
    "mxb_ring_destroy": (i32, [_vp]),
    "mxb_place": (i32, [_vp, _P(Desc2D), u64, i32, u32, _P(PlaceStats)]),
    "mxb_image_create": (i32, [_vp, _P(Desc2D), u64, i32, _P(_vp), _P(PlaceStats)]),
    "mxb_image_place": (i32, [_vp, _P(Desc2D), u64, _P(PlaceStats)]),
    "mxb_image_bytes": (u64, [_vp]),
    "mxb_image_destroy": (i32, [_vp]),
    "mxb_digest": (i32, [_vp, i32, _P(Span), u64, u32, _P(DigestOut)]),
    "mxb_block_hashes": (i32, [_vp, i32, u64, u64, u64]),
    "mxb_digest_noalloc": (i32, [i32, _P(Span), u64, u32, _P(DigestOut), _vp]),
    "mxb_arena_create": (i32, [i32, u64, _P(_vp)]),
    "mxb_arena_malloc": (i32, [_vp, u64, _P(u64)]),
    "mxb_arena_free": (i32, [_vp, u64]),
    "mxb_arena_range": (i32, [_vp, _P(u64), _P(u64), _P(u64)]),
    "mxb_arena_blocks": (i32, [_vp, _P(ArenaBlock), u64, _P(u64)]),
    "mxb_arena_export_fd": (i32, [_vp, u64, _P(i32)]),
    "mxb_arena_import": (i32, [i32, u64, _P(ArenaBlock), _P(i32), u64, _P(_vp)]),
    "mxb_arena_destroy": (i32, [_vp]),
    "mxb_arena_set_default": (i32, [i32, _vp]),
    "mxb_arena_torch_malloc": (_vp, [ctypes.c_ssize_t, ctypes.c_int, _vp]),
    "mxb_arena_torch_free": (None, [_vp, ctypes.c_ssize_t, ctypes.c_int, _vp]),
    "mxb_convert_boxes": (i32, [_vp, i32, _P(ConvertBox), u64, u32, _P(u64)]),
    "mxb_fanout_plan": (i32, [_P(Span), u64, u64, _P(FanoutPiece), u64, _P(u64), _P(u32), u64, _P(u64)]),
    "mxb_fanout_create": (i32, [_vp, i32, _P(Span), u64, u64, _P(_vp)]),
    "mxb_fanout_create_pieces": (i32, [_vp, i32, _P(Span), u64, u64, u64, _P(_vp)]),
    "mxb_fanout_plan_pieces": (i32, [_P(Span), u64, u64, u64, _P(FanoutPiece), u64, _P(u64), _P(u32), u64, _P(u64)]),
    "mxb_fanout_counters": (u64, [_vp]),
    "mxb_fanout_set_child": (i32, [_vp, i32, _P(Span), u64, u64]),
    "mxb_fanout_set_engine": (i32, [_vp, i32]),
    "mxb_fanout_run": (i32, [_vp, i32, u32]),
    "mxb_fanout_wait": (i32, [_vp, _P(ctypes.c_float)]),
    "mxb_fanout_destroy": (i32, [_vp]),
}


class MxbError(RuntimeError):
    def __init__(self, code: int, where: str, text: str):
        self.code = code
        super().__init__(f"{where}: {ERR_NAMES.get(code, code)}: {text}")


class MxbTimeout(MxbError, TimeoutError):
    pass


_lib = None


def load():
    """Load the shared library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing. Build it with `python -m modelexpress_b200.build` "
            "(needs nvcc); this package has no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(code: int, where: str) -> None:
    if code == OK:
        return
    text = load().mxb_last_error().decode("utf-8", "replace")
    if code == -5:
        raise MxbTimeout(code, where, text)
    raise MxbError(code, where, text)


def desc_array(descs) -> ctypes.Array:
    """Sequence of 6-tuples (or an (n,6) uint64 numpy array) -> Desc2D array."""
    import numpy as np

    a = np.ascontiguousarray(np.asarray(descs, dtype=np.uint64).reshape(-1, 6))
    arr = (Desc2D * max(1, a.shape[0]))()
    if a.shape[0]:
        ctypes.memmove(arr, a.ctypes.data, a.nbytes)
    return arr, a.shape[0]


def run_array(runs) -> ctypes.Array:
    import numpy as np

    a = np.ascontiguousarray(np.asarray(runs, dtype=np.uint64).reshape(-1, 3))
    arr = (Run * max(1, a.shape[0]))()
    if a.shape[0]:
        ctypes.memmove(arr, a.ctypes.data, a.nbytes)
    return arr, a.shape[0]


def span_array(spans) -> ctypes.Array:
    import numpy as np

    a = np.ascontiguousarray(np.asarray(spans, dtype=np.uint64).reshape(-1, 2))
    arr = (Span * max(1, a.shape[0]))()
    if a.shape[0]:
        ctypes.memmove(arr, a.ctypes.data, a.nbytes)
    return arr, a.shape[0]
