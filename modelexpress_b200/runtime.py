"""Object wrappers over the C ABI: context, staging ring, fan-out node.

Plain integers are used for device addresses so that callers may pass
``tensor.data_ptr()``, a peer pointer or a pinned host address alike.
"""

from __future__ import annotations

import ctypes
import threading
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import (DIGEST_BLOCK64, DIGEST_ROWS, DIGEST_SAFE32, PLACE_COPY_ENGINE,
                   PLACE_ZERO_COPY, SCATTER_VECTOR, SCATTER_DEFAULT, SCATTER_NO_SYNC, SCATTER_OVERLAP,
                   check)

__all__ = ["Context", "Ring", "PackedImage", "Fanout", "Table", "PlaceResult", "default_context",
           "host_register", "host_unregister", "host_is_pinned", "plan_pull", "plan_reshard",
           "DIGEST_SAFE32", "DIGEST_ROWS", "DIGEST_BLOCK64", "SCATTER_DEFAULT", "SCATTER_VECTOR",
           "SCATTER_NO_SYNC", "SCATTER_OVERLAP", "PLACE_COPY_ENGINE", "PLACE_ZERO_COPY"]


_close_lock = threading.Lock()


@dataclass
class PlaceResult:
    bytes_placed: int
    chunks: int
    launches: int
    seconds_total: float
    seconds_gather: float
    seconds_device: float
    bytes_direct: int = 0        # of bytes_placed: read from pinned sources, no host copy
    seconds_plan: float = 0.0


class Context:
    """A set of CUDA devices of this process with peer access enabled."""

    def __init__(self, devices=(0,)):
        self._lib = _lib.load()
        self.devices = [int(d) for d in devices]
        ids = (ctypes.c_int32 * len(self.devices))(*self.devices)
        h = ctypes.c_void_p()
        check(self._lib.mxb_ctx_create(ids, len(self.devices), ctypes.byref(h)), "mxb_ctx_create")
        self._h = h
        self._background: list = []   # threads still releasing objects of this context
        self._rings: dict = {}        # (dev, bytes, slots) -> Ring kept between loads
        self._rings_lock = threading.Lock()

    def cached_ring(self, ring_bytes: int, slots: int, dev: int | None = None) -> "Ring":
        """The staging ring loads of this context share.  Pinning host memory and allocating
        the device staging cost more than a tenth of a 2 GB load, so the ring a load makes is
        kept for the next one (``drop_cached_rings`` gives the memory back)."""
        key = (self._dev(dev), int(ring_bytes), int(slots))
        with self._rings_lock:
            ring = self._rings.get(key)
            if ring is None or ring._h is None:
                ring = self._rings[key] = Ring(self, key[0], key[1], key[2])
            return ring

    def drop_cached_rings(self) -> None:
        with self._rings_lock:
            rings, self._rings = list(self._rings.values()), {}
        for r in rings:
            r.close()

    def close(self):
        if getattr(self, "_h", None):
            for t in self._background:
                t.join()
            self._background = []
            self.drop_cached_rings()
            self._lib.mxb_ctx_destroy(self._h)
            self._h = None

    def release_later(self, obj) -> None:
        """Close ``obj`` (a ring) on a background thread; ``close()`` waits for it."""
        import threading

        self._background = [t for t in self._background if t.is_alive()]
        t = threading.Thread(target=obj.close, name="mxb-release", daemon=True)
        self._background.append(t)
        t.start()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- memory ------------------------------------------------------------
    def alloc(self, nbytes: int, dev: int | None = None) -> int:
        out = ctypes.c_uint64()
        check(self._lib.mxb_alloc(self._h, self._dev(dev), int(nbytes), ctypes.byref(out)), "mxb_alloc")
        return out.value

    def free(self, ptr: int, dev: int | None = None) -> None:
        check(self._lib.mxb_free(self._h, self._dev(dev), int(ptr)), "mxb_free")

    def register_extent(self, base: int, nbytes: int) -> None:
        check(self._lib.mxb_register_extent(self._h, int(base), int(nbytes)), "mxb_register_extent")

    def clear_extents(self) -> None:
        check(self._lib.mxb_clear_extents(self._h), "mxb_clear_extents")

    def sync(self, dev: int | None = None) -> None:
        check(self._lib.mxb_sync(self._h, self._dev(dev)), "mxb_sync")

    @property
    def launch_count(self) -> int:
        return int(self._lib.mxb_launch_count(self._h))

    def _dev(self, dev):
        return self.devices[0] if dev is None else int(dev)

    # -- kernels -----------------------------------------------------------
    def scatter(self, descs, dev: int | None = None, flags: int = SCATTER_DEFAULT) -> None:
        """descs: iterable of (src, dst, rows, row_bytes, src_pitch, dst_pitch)."""
        arr, n = _lib.desc_array(descs)
        check(self._lib.mxb_scatter(self._h, self._dev(dev), arr, n, flags), "mxb_scatter")

    ELEM_KINDS = {"raw": 0, "f32": 1, "f16": 2, "bf16": 3}

    @classmethod
    def convert_array(cls, boxes):
        """Marshal ``(src, dst, extents, dst_strides, src_kind, dst_kind, elem_bytes[, src_strides])``
        tuples once (a list that is replayed every step need not be marshalled every step).
        Without ``src_strides`` the source box is contiguous."""
        boxes = list(boxes)
        arr = (_lib.ConvertBox * max(1, len(boxes)))()
        for i, box in enumerate(boxes):
            src, dst, extents, strides, sk, dk, eb = box[:7]
            src_strides = box[7] if len(box) > 7 and box[7] is not None else None
            if len(extents) != len(strides) or len(extents) > _lib.MAX_DIMS or (
                    src_strides is not None and len(src_strides) != len(extents)):
                raise ValueError("convert box: extents and strides must have the same rank, at most 8")
            b = arr[i]
            b.src, b.dst, b.ndim = int(src), int(dst), len(extents)
            b.src_kind, b.dst_kind, b.elem_bytes = cls.ELEM_KINDS[sk], cls.ELEM_KINDS[dk], int(eb)
            for d, (e, st) in enumerate(zip(extents, strides)):
                b.extent[d], b.dst_stride[d] = int(e), int(st)
                b.src_stride[d] = int(src_strides[d]) if src_strides is not None else 0
        return arr, len(boxes)

    def convert_boxes(self, boxes, dev: int | None = None, flags: int = SCATTER_DEFAULT) -> int:
        """boxes: iterable of (src, dst, extents, dst_strides, src_kind, dst_kind, elem_bytes), or
        what ``convert_array`` returned: each contiguous staged box lands with the destination's
        strides (in elements), cast when the kinds ("raw", "f32", "f16", "bf16") differ.
        One launch per pair of kinds present; returns bytes read + written."""
        prepared = isinstance(boxes, tuple) and len(boxes) == 2 and isinstance(boxes[0], ctypes.Array)
        arr, n = boxes if prepared else self.convert_array(boxes)
        moved = ctypes.c_uint64(0)
        check(self._lib.mxb_convert_boxes(self._h, self._dev(dev), arr, n, flags, ctypes.byref(moved)),
              "mxb_convert_boxes")
        return int(moved.value)

    def read_runs(self, runs, dev: int | None = None) -> None:
        """runs: iterable of (src, dst, nbytes); returns when the bytes are visible."""
        arr, n = _lib.run_array(runs)
        check(self._lib.mxb_read_runs(self._h, self._dev(dev), arr, n), "mxb_read_runs")

    def digest(self, spans, modes: int, dev: int | None = None) -> list:
        """spans: iterable of (ptr, nbytes) -> list of DigestOut records."""
        arr, n = _lib.span_array(spans)
        out = (_lib.DigestOut * max(1, n))()
        check(self._lib.mxb_digest(self._h, self._dev(dev), arr, n, modes, out), "mxb_digest")
        return [out[i] for i in range(n)]

    def block_hashes(self, ptr: int, nbytes: int, out_ptr: int, dev: int | None = None) -> None:
        check(self._lib.mxb_block_hashes(self._h, self._dev(dev), int(ptr), int(nbytes), int(out_ptr)),
              "mxb_block_hashes")

    def table(self, descs, dev: int | None = None) -> "Table":
        return Table(self, self._dev(dev), descs)

    def copy_probe(self, src: int, dst: int, nbytes: int, reps: int = 3, dev: int | None = None) -> float:
        """Milliseconds per launch of the plain copy kernel (``mxb_copy_probe``)."""
        ms = ctypes.c_float(0.0)
        check(self._lib.mxb_copy_probe(self._h, self._dev(dev), int(src), int(dst), int(nbytes), int(reps),
                                       ctypes.byref(ms)), "mxb_copy_probe")
        return float(ms.value)

    def event_record(self, slot: int, dev: int | None = None) -> None:
        check(self._lib.mxb_event_record(self._h, self._dev(dev), int(slot)), "mxb_event_record")

    def event_elapsed_ms(self, a: int, b: int, dev: int | None = None) -> float:
        ms = ctypes.c_float(0.0)
        check(self._lib.mxb_event_elapsed(self._h, self._dev(dev), int(a), int(b), ctypes.byref(ms)),
              "mxb_event_elapsed")
        return float(ms.value)

    def ring(self, ring_bytes: int = 2 << 30, slots: int = 32, dev: int | None = None) -> "Ring":
        return Ring(self, self._dev(dev), ring_bytes, slots)

    def fanout(self, local_spans, chunk_bytes: int, dev: int | None = None, piece_bytes: int = 65536) -> "Fanout":
        return Fanout(self, self._dev(dev), local_spans, chunk_bytes, piece_bytes)


def coalesce_runs(runs) -> np.ndarray:
    """Host-only: fold a run list into 2-D records; returns an (m, 6) uint64 array."""
    lib = _lib.load()
    arr, n = _lib.run_array(runs)
    cap = max(1, n)
    out = (_lib.Desc2D * cap)()
    m = lib.mxb_coalesce_runs(arr, n, out, cap)
    if m < 0:
        raise _lib.MxbError(int(m), "mxb_coalesce_runs", "capacity")
    res = np.zeros((m, 6), dtype=np.uint64)
    if m:
        ctypes.memmove(res.ctypes.data, out, m * ctypes.sizeof(_lib.Desc2D))
    return res


def plan_pull(global_shape, elsize: int, win_offset: int, win_shape, win_stride, dst_offset: int,
              dst_stride, shards, dst_base: int, keep_rank: bool = True) -> tuple:
    """Host-only: the descriptor compiler behind the C ABI (``mxb_plan_pull``).
    ``shards`` is a list of ``(offset tuple, shape tuple, addr)``.  Returns
    ``(records (m, 6) uint64, shard index of each record (m,) uint32)``; raises
    ``MxbError`` with code -9 for a window that is not a permuted box of its source."""
    lib = _lib.load()
    w = _lib.Window()
    w.ndim_src, w.ndim_win, w.keep_rank, w.elsize = len(global_shape), len(win_shape), int(keep_rank), int(elsize)
    if max(w.ndim_src, w.ndim_win) > _lib.MAX_DIMS:
        raise ValueError(f"at most {_lib.MAX_DIMS} dims")
    for d, v in enumerate(global_shape):
        w.global_shape[d] = int(v)
    for d in range(len(win_shape)):
        w.win_shape[d], w.win_stride[d], w.dst_stride[d] = int(win_shape[d]), int(win_stride[d]), int(dst_stride[d])
    w.win_offset, w.dst_offset = int(win_offset), int(dst_offset)
    arr = (_lib.Shard * max(1, len(shards)))()
    for k, (off, shp, addr) in enumerate(shards):
        arr[k].ndim = len(off)
        if len(off) != len(shp) or len(off) > _lib.MAX_DIMS:
            raise ValueError("shard rank does not match the source rank")
        for d in range(len(off)):
            arr[k].offset[d], arr[k].shape[d] = int(off[d]), int(shp[d])
        arr[k].addr = int(addr)
    cap = 64
    while True:
        out = (_lib.Desc2D * cap)()
        which = (ctypes.c_uint32 * cap)()
        n = ctypes.c_uint64()
        rc = lib.mxb_plan_pull(ctypes.byref(w), arr, len(shards), int(dst_base), out, which, cap,
                               ctypes.byref(n))
        if rc == -7 and n.value > cap:
            cap = int(n.value)
            continue
        check(rc, "mxb_plan_pull")
        break
    res = np.zeros((n.value, 6), dtype=np.uint64)
    if n.value:
        ctypes.memmove(res.ctypes.data, out, n.value * ctypes.sizeof(_lib.Desc2D))
    return res, np.array(which[: n.value], dtype=np.uint32)


def plan_reshard(regions, shard_lo: int, shard_hi: int, src_base: int, max_record_bytes: int = 0) -> np.ndarray:
    """Host-only: ``mxb_plan_reshard``; ``regions`` are ``(byte offset in the flat
    tensor, dst address, rows, row_bytes, src_pitch, dst_pitch)``."""
    lib = _lib.load()
    arr, n_in = _lib.desc_array(regions)
    cap = max(16, 4 * n_in)
    while True:
        out = (_lib.Desc2D * cap)()
        n = ctypes.c_uint64()
        rc = lib.mxb_plan_reshard(arr, n_in, int(shard_lo), int(shard_hi), int(src_base),
                                  int(max_record_bytes), out, cap, ctypes.byref(n))
        if rc == -7 and n.value > cap:
            cap = int(n.value)
            continue
        check(rc, "mxb_plan_reshard")
        break
    res = np.zeros((n.value, 6), dtype=np.uint64)
    if n.value:
        ctypes.memmove(res.ctypes.data, out, n.value * ctypes.sizeof(_lib.Desc2D))
    return res


class Table:
    """A descriptor table resident on the device; ``launch`` replays it."""

    def __init__(self, ctx: Context, dev: int, descs):
        self.ctx, self.dev = ctx, dev
        arr, n = _lib.desc_array(descs)
        h = ctypes.c_void_p()
        check(ctx._lib.mxb_table_create(ctx._h, dev, arr, n, ctypes.byref(h)), "mxb_table_create")
        self._h = h

    @property
    def nbytes(self) -> int:
        return int(self.ctx._lib.mxb_table_bytes(self._h))

    def engine(self, flags: int = SCATTER_DEFAULT) -> str:
        """Which tile engines a launch with ``flags`` runs: "vector", "bulk" or "bulk+vector"."""
        return ("vector", "bulk", "bulk+vector")[self.ctx._lib.mxb_table_engine(self._h, int(flags))]

    def launch(self, flags: int = SCATTER_DEFAULT) -> None:
        check(self.ctx._lib.mxb_table_launch(self._h, int(flags)), "mxb_table_launch")

    def close(self):
        if getattr(self, "_h", None):
            # the object lives inside its context: if that was closed first there is
            # nothing left to release
            if getattr(self.ctx, "_h", None):
                self.ctx._lib.mxb_table_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Ring:
    """Pinned staging ring bound to one device."""

    def __init__(self, ctx: Context, dev: int, ring_bytes: int, slots: int):
        self.ctx, self.dev = ctx, dev
        h = ctypes.c_void_p()
        check(ctx._lib.mxb_ring_create(ctx._h, dev, int(ring_bytes), int(slots), ctypes.byref(h)),
              "mxb_ring_create")
        self._h = h
        self._images: list = []      # kept images use this ring's staging buffers

    def place(self, items, host_threads: int = 8, mode: int = PLACE_COPY_ENGINE) -> PlaceResult:
        """items: (host_src, device_dst, rows, row_bytes, src_pitch, dst_pitch) records."""
        arr, n = _lib.desc_array(items)
        st = _lib.PlaceStats()
        check(self.ctx._lib.mxb_place(self._h, arr, n, int(host_threads), int(mode), ctypes.byref(st)),
              "mxb_place")
        return PlaceResult(st.bytes_placed, st.chunks, st.launches, st.seconds_total,
                           st.seconds_gather, st.seconds_device, st.bytes_direct, st.seconds_plan)

    def keep(self, items, host_threads: int = 8) -> tuple:
        """Place ``items`` and keep their packed bytes page-locked for later loads:
        ``(PackedImage, PlaceResult)`` (``mxb_image_create``)."""
        arr, n = _lib.desc_array(items)
        st = _lib.PlaceStats()
        h = ctypes.c_void_p()
        check(self.ctx._lib.mxb_image_create(self._h, arr, n, int(host_threads), ctypes.byref(h),
                                             ctypes.byref(st)), "mxb_image_create")
        img = PackedImage(self, h)
        self._images.append(img)
        return img, PlaceResult(st.bytes_placed, st.chunks, st.launches, st.seconds_total,
                                st.seconds_gather, st.seconds_device, st.bytes_direct, st.seconds_plan)

    def close(self):
        for img in list(getattr(self, "_images", [])):
            img.close()
        with _close_lock:            # a background release and __del__ may both get here
            h, self._h = getattr(self, "_h", None), None
        if h:
            # the object lives inside its context: if that was closed first there is
            # nothing left to release
            if getattr(self.ctx, "_h", None):
                self.ctx._lib.mxb_ring_destroy(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class PackedImage:
    """A rank's slices kept page-locked in host memory as they cross PCIe; ``place``
    loads them again with no host copy (``mxb_image_place``)."""

    def __init__(self, ring: Ring, handle):
        self.ring, self._h = ring, handle

    @property
    def nbytes(self) -> int:
        return int(self.ring.ctx._lib.mxb_image_bytes(self._h)) if self._h else 0

    def place(self, items=None) -> PlaceResult:
        """``items``: the same slices with (possibly) new destination addresses."""
        if not self._h:
            raise RuntimeError("the image has been released")
        st = _lib.PlaceStats()
        if items is None:
            rc = self.ring.ctx._lib.mxb_image_place(self._h, None, 0, ctypes.byref(st))
        else:
            arr, n = _lib.desc_array(items)
            rc = self.ring.ctx._lib.mxb_image_place(self._h, arr, n, ctypes.byref(st))
        check(rc, "mxb_image_place")
        return PlaceResult(st.bytes_placed, st.chunks, st.launches, st.seconds_total,
                           st.seconds_gather, st.seconds_device, st.bytes_direct, st.seconds_plan)

    def close(self):
        h, self._h = self._h, None
        if h:
            if self in self.ring._images:
                self.ring._images.remove(self)
            if getattr(self.ring, "_h", None) and getattr(self.ring.ctx, "_h", None):
                self.ring.ctx._lib.mxb_image_destroy(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Fanout:
    """One node of a chunked, pipelined broadcast (see ``fanout.py`` for topologies)."""

    def __init__(self, ctx: Context, dev: int, local_spans, chunk_bytes: int, piece_bytes: int = 65536):
        self.ctx, self.dev = ctx, dev
        arr, n = _lib.span_array(local_spans)
        self.n = n
        h = ctypes.c_void_p()
        check(ctx._lib.mxb_fanout_create_pieces(ctx._h, dev, arr, n, int(chunk_bytes), int(piece_bytes),
                                                ctypes.byref(h)), "mxb_fanout_create")
        self._h = h
        self.children = 0

    ENGINES = {"vector": 0, "bulk": 1, "dma": 2}

    def set_engine(self, engine: str) -> None:
        """"vector" (16-byte peer stores straight from HBM), "bulk" (staged through shared memory
        with bulk copies) or, for a root whose children only receive, "dma" (copy engines, then one
        launch that announces every chunk); the nodes of one broadcast may differ."""
        if engine not in self.ENGINES:
            raise ValueError(f"unknown fan-out engine {engine!r}")
        check(self.ctx._lib.mxb_fanout_set_engine(self._h, self.ENGINES[engine]), "mxb_fanout_set_engine")

    @property
    def counters(self) -> int:
        return int(self.ctx._lib.mxb_fanout_counters(self._h))

    def add_child(self, child_spans, child_counters: int) -> None:
        arr, n = _lib.span_array(child_spans)
        check(self.ctx._lib.mxb_fanout_set_child(self._h, self.children, arr, n, int(child_counters)),
              "mxb_fanout_set_child")
        self.children += 1

    def run(self, is_root: bool, timeout_ms: int = 2000) -> None:
        check(self.ctx._lib.mxb_fanout_run(self._h, 1 if is_root else 0, int(timeout_ms)),
              "mxb_fanout_run")

    def wait(self) -> float:
        ms = ctypes.c_float(0.0)
        check(self.ctx._lib.mxb_fanout_wait(self._h, ctypes.byref(ms)), "mxb_fanout_wait")
        return float(ms.value)

    def close(self):
        if getattr(self, "_h", None):
            # the object lives inside its context: if that was closed first there is
            # nothing left to release
            if getattr(self.ctx, "_h", None):
                self.ctx._lib.mxb_fanout_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def ipc_export(ptr: int) -> tuple:
    lib = _lib.load()
    h = (ctypes.c_uint8 * 64)()
    off = ctypes.c_uint64()
    check(lib.mxb_ipc_export(int(ptr), h, ctypes.byref(off)), "mxb_ipc_export")
    return bytes(h), off.value


def ipc_open(handle: bytes, offset: int) -> int:
    lib = _lib.load()
    h = (ctypes.c_uint8 * 64)(*handle)
    out = ctypes.c_uint64()
    check(lib.mxb_ipc_open(h, int(offset), ctypes.byref(out)), "mxb_ipc_open")
    return out.value


def host_register(addr: int, nbytes: int) -> tuple:
    """Pin host memory in place (``mxb_host_register``); returns the page-aligned
    ``(base, nbytes)`` actually pinned, to be handed to ``host_unregister``."""
    lib = _lib.load()
    base, size = ctypes.c_uint64(), ctypes.c_uint64()
    check(lib.mxb_host_register(int(addr), int(nbytes), ctypes.byref(base), ctypes.byref(size)),
          "mxb_host_register")
    return base.value, size.value


def host_unregister(base: int) -> None:
    check(_lib.load().mxb_host_unregister(int(base)), "mxb_host_unregister")


def host_is_pinned(addr: int, nbytes: int) -> bool:
    return bool(_lib.load().mxb_host_is_pinned(int(addr), int(nbytes)))


_default: dict = {}


def default_context(device: int = 0) -> Context:
    """Process-wide single-device context, created on first use."""
    ctx = _default.get(device)
    if ctx is None:
        ctx = _default[device] = Context([device])
    return ctx
