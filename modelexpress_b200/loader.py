"""Checkpoint placement: safetensors files -> this rank's GPU parameters.

``place_checkpoint`` is the B200 replacement for the host-staged load the
reference reaches through engines/vllm/adapter.py:316-329: instead of one CPU
``narrow`` and one pageable H2D ``copy_`` per tensor, the rank's slices are
described once (``layout.plan_checkpoint``), gathered into a pinned ring by host
threads, sent over PCIe on the copy-engine stream and written into the shards
by one persistent scatter launch per ring chunk.

``B200ScatterStrategy`` packages that as a load strategy with the reference's
plugin contract (load_strategy/base.py:37-76): ``name``, ``requires``,
``is_available(ctx)``, ``load(result, ctx) -> LoadResult``, ``rollback(ctx)``;
an expected miss raises ``StrategyFailed(mutated=False)``, a failure after
parameter bytes were touched raises ``StrategyFailed(mutated=True)``.
"""

from __future__ import annotations

import mmap
import os
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Any

import numpy as np

from .layout import CheckpointPlan, plan_checkpoint
from ._lib import MxbError
from .runtime import (PLACE_COPY_ENGINE, Context, PlaceResult, Ring, default_context, host_register,
                      host_unregister)
from .safetensors_index import SAFETENSORS_DTYPES, checkpoint_index


# The ring a load creates for itself: pinning host memory sits inside the time to loaded
# weights, and the pipeline is as fast with four 32 MiB chunks as with a ring of gigabytes.
RING_BYTES = 128 << 20
RING_SLOTS = 4
PIN_MODES = ("off", "keep", "pages", "pages_after")


class StrategyFailed(Exception):
    """adapter.py:24-34 of the reference: ``mutated`` tells the chain whether the
    model must be re-initialised before the next strategy runs."""

    def __init__(self, message: str, mutated: bool = False):
        super().__init__(message)
        self.mutated = mutated


@dataclass
class LoadResult:
    """load_strategy/context.py:40-51."""

    value: Any
    model: Any = None
    publishable: bool = True
    metadata: dict = field(default_factory=dict)


class FileImage:
    """A checkpoint file mapped into host memory; ``address`` is the host address of byte 0.

    ``pinnable`` maps the file readable and writable, the form ``mxb_host_register``
    can pin; nothing ever stores through the mapping.  Where the file may be opened
    for writing the mapping is shared: its page-cache pages are pinned where they
    are.  A file that is read-only to this process is mapped privately instead, which
    still pins but makes the kernel give the mapping its own copy of every pinned
    page first (several times slower, and the pinned ranges then exist twice in host
    memory).  ``pin_spans`` page-locks the byte ranges a rank keeps, after which
    ``mxb_place`` reads them with the copy engine directly and no host thread copies
    a byte."""

    def __init__(self, path: str, pinnable: bool = False):
        self.path = path
        self.shared = False
        if pinnable:
            try:
                self._f = open(path, "r+b")
                self.shared = True
            except OSError:
                self._f = open(path, "rb")
        else:
            self._f = open(path, "rb")
        self.size = os.fstat(self._f.fileno()).st_size
        if pinnable:
            self._map(self.shared)
            if self.shared and self.size >= mmap.PAGESIZE:
                # A shared writable mapping can be page-locked only where the file system allows
                # long-term pins of its pages (memory file systems do, disk-backed ones refuse):
                # try one page now, before anyone has been given an address.
                try:
                    base, _n = host_register(self.address, mmap.PAGESIZE)
                    host_unregister(base)
                except MxbError:
                    self._np = None
                    self._mm.close()
                    self.shared = False
                    self._map(False)
        else:
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
            self._np = np.frombuffer(self._mm, dtype=np.uint8)
            self.address = self._np.ctypes.data
        self.pinnable = pinnable
        self._pinned: list = []           # (base, nbytes) ranges registered by this image
        self._pin_lock = threading.Lock()
        self.pinned_bytes = 0
        self.pin_seconds = 0.0

    def _map(self, shared: bool) -> None:
        self._mm = mmap.mmap(self._f.fileno(), 0, flags=mmap.MAP_SHARED if shared else mmap.MAP_PRIVATE,
                             prot=mmap.PROT_READ | mmap.PROT_WRITE)
        self._np = np.frombuffer(self._mm, dtype=np.uint8)
        self.address = self._np.ctypes.data

    def pin_spans(self, spans, merge_gap: int = 1 << 20) -> int:
        """Pin the union of ``(offset, nbytes)`` ranges of the file (page-aligned,
        neighbours closer than ``merge_gap`` joined) that is not pinned yet; returns
        the bytes newly pinned."""
        if not self.pinnable:
            raise RuntimeError(f"{self.path} was not mapped pinnable")
        with self._pin_lock:
            return self._pin_spans(spans, merge_gap)

    def _pin_spans(self, spans, merge_gap: int) -> int:
        page = mmap.PAGESIZE
        want = sorted((int(o) // page * page, min(self.size, -(-(int(o) + int(n)) // page) * page))
                      for o, n in spans if n)
        merged: list = []
        for lo, hi in want:
            if merged and lo <= merged[-1][1] + merge_gap:
                merged[-1][1] = max(merged[-1][1], hi)
            else:
                merged.append([lo, hi])
        have = sorted((b - self.address, b - self.address + n) for b, n in self._pinned)
        t0 = time.perf_counter()
        added = 0
        def pin(lo: int, hi: int) -> int:
            base, n = host_register(self.address + lo, hi - lo)
            self._pinned.append((base, n))
            return n

        for lo, hi in merged:
            cur = lo                      # carve out what earlier calls pinned already
            for plo, phi in have:
                if phi <= cur:
                    continue
                if plo >= hi:
                    break
                if plo > cur:
                    added += pin(cur, plo)
                cur = max(cur, phi)
            if cur < hi:
                added += pin(cur, hi)
        self.pinned_bytes += added
        self.pin_seconds += time.perf_counter() - t0
        return added

    def unpin(self) -> None:
        for base, _n in self._pinned:
            host_unregister(base)
        self._pinned = []
        self.pinned_bytes = 0

    def close(self):
        self.unpin()
        self._np = None
        try:
            self._mm.close()
        finally:
            self._f.close()


class HostImages:
    """Checkpoint files kept mapped (and, where asked, pinned) between loads of the same
    process: the second load of a checkpoint — another replica, a reload after a weight
    swap, the next refit from a host copy — finds its bytes page-locked and goes over
    PCIe with no host copy.  Keyed by path, size and modification time."""

    def __init__(self):
        self._images: dict = {}
        self._plans: dict = {}
        self._captured: dict = {}     # (checkpoint path, device) -> _KeptCapture
        self._lock = threading.Lock()

    def prepared(self, model_path: str, tp_rank: int, tp_size: int, family: str) -> "Prepared":
        """The parsed headers and the rank's placement plan of a checkpoint, kept for
        as long as its files keep their size and modification time (the reference
        keeps its transfer plan between refits the same way, receiver.py:553)."""
        key = (os.path.realpath(model_path), int(tp_rank), int(tp_size), family)
        with self._lock:
            hit = self._plans.get(key)
        if hit is not None and hit.fresh():
            return hit
        prep = Prepared.build(model_path, tp_rank, tp_size, family)
        with self._lock:
            self._plans[key] = prep
        return prep

    def open(self, path: str) -> FileImage:
        st = os.stat(path)
        key = (os.path.realpath(path), st.st_size, st.st_mtime_ns)
        with self._lock:
            im = self._images.get(key)
            if im is None:
                for k in [k for k in self._images if k[0] == key[0]]:   # the file changed
                    self._images.pop(k).close()
                im = self._images[key] = FileImage(path, pinnable=True)
            return im

    @property
    def pinned_bytes(self) -> int:
        return sum(im.pinned_bytes for im in self._images.values())

    @property
    def packed_bytes(self) -> int:
        return (sum(img.nbytes for prep in self._plans.values() for img in prep.packed.values())
                + sum(img.nbytes for kept in self._captured.values() for img, _r, _w in kept.batches))

    def close(self) -> None:
        with self._lock:
            for prep in self._plans.values():
                for img in prep.packed.values():
                    img.close()
                prep.packed = {}
            for kept in self._captured.values():
                kept.close()
            self._captured = {}
            for im in self._images.values():
                im.close()
            self._images = {}
            self._plans = {}


@dataclass
class _KeptCapture:
    """What a captured load leaves behind for the next load of the same checkpoint into a
    model of the same shapes: the packed images of its batches, where every record lands
    (destination tensor name + byte offset), the staged casts and the engine-loaded rest."""

    stamps: tuple
    batches: list                # [(PackedImage, records (n, 6), [(dest name, byte offset)])]
    stagings: list               # [(converts, staging tensor)]
    leftover: list               # source names the engine's loader handles
    summary: dict                # copies, records, reasons, written_params

    def close(self) -> None:
        for img, _r, _w in self.batches:
            img.close()
        self.batches = []


@dataclass
class Prepared:
    """Headers and placement plan of one checkpoint for one rank, with the record
    geometry as arrays so that a load only has to add base addresses."""

    index: dict
    plan: CheckpointPlan
    files: list                 # absolute paths, sorted
    geometry: np.ndarray        # (n, 6) uint64: file offset, parameter offset, rows, row_bytes, pitches
    file_of: np.ndarray         # (n,) index into files
    stamps: tuple               # (dir mtime, ((path, size, mtime_ns), ...)) the plan was built from
    model_path: str = ""
    pinned_in: tuple = ()       # ids of the FileImages this rank's ranges are already pinned in
    packed: dict = field(default_factory=dict)   # device index -> runtime.PackedImage of this rank's bytes

    @staticmethod
    def _stamps(model_path: str, files) -> tuple:
        per_file = []
        for p in files:
            st = os.stat(p)
            per_file.append((p, st.st_size, st.st_mtime_ns))
        return (os.stat(model_path).st_mtime_ns if os.path.isdir(model_path) else 0, tuple(per_file))

    @classmethod
    def build(cls, model_path: str, tp_rank: int, tp_size: int, family: str) -> "Prepared":
        index = checkpoint_index(model_path)
        plan = plan_checkpoint({n: {"shape": i["shape"], "dtype": i["dtype"]} for n, i in index.items()},
                               tp_rank, tp_size, family)
        files = sorted({i["file"] for i in index.values()})
        check_index(index, {p: os.path.getsize(p) for p in files})
        geometry = np.empty((len(plan.placements), 6), dtype=np.uint64)
        file_of = np.empty(len(plan.placements), dtype=np.int64)
        where = {p: k for k, p in enumerate(files)}
        for k, pl in enumerate(plan.placements):
            info = index[pl.src_name]
            geometry[k] = pl.record(int(info["file_offset"]), 0)
            file_of[k] = where[info["file"]]
        return cls(index, plan, files, geometry, file_of, cls._stamps(model_path, files), model_path)

    def fresh(self) -> bool:
        try:
            return self._stamps(self.model_path, self.files) == self.stamps
        except OSError:
            return False

    def items(self, file_address: dict, params: dict) -> np.ndarray:
        """(n, 6) uint64 records: host source address -> device destination address."""
        dst = np.empty(len(self.plan.placements), dtype=np.uint64)
        for k, pl in enumerate(self.plan.placements):
            t = params[pl.dst_name]
            spec = self.plan.params[pl.dst_name]
            if tuple(t.shape) != tuple(spec.shape) or not t.is_contiguous():
                raise ValueError(f"{pl.dst_name}: destination tensor must be contiguous with shape "
                                 f"{tuple(spec.shape)}, got {tuple(t.shape)}")
            if t.element_size() != SAFETENSORS_DTYPES[pl.dtype][0]:
                raise ValueError(f"{pl.dst_name}: element size differs from the checkpoint's {pl.dtype}")
            dst[k] = t.data_ptr()
        out = self.geometry.copy()
        out[:, 0] += np.array([file_address[p] for p in self.files], dtype=np.uint64)[self.file_of]
        out[:, 1] += dst
        return out


host_images = HostImages()


def check_index(index: dict, sizes: dict) -> None:
    """Every tensor's byte range must lie inside its file and match its shape; a
    truncated or half-written shard fails here (``ValueError``) instead of letting a
    copy run past the end of the mapping."""
    for name, info in index.items():
        elsize = SAFETENSORS_DTYPES[info["dtype"]][0]
        numel = 1
        for extent in info["shape"]:
            numel *= int(extent)
        if int(info["size"]) != numel * elsize:
            raise ValueError(f"{name}: header gives {info['size']} bytes for shape {list(info['shape'])} "
                             f"of {info['dtype']}")
        if int(info["file_offset"]) + int(info["size"]) > sizes[info["file"]]:
            raise ValueError(f"{name}: bytes [{info['file_offset']}, "
                             f"{int(info['file_offset']) + int(info['size'])}) lie beyond the end of "
                             f"{info['file']} ({sizes[info['file']]} bytes): truncated file?")


def item_spans(items: np.ndarray, file_address: dict, sizes: dict | None = None) -> dict:
    """{file: [(offset, nbytes)]}: the source byte span of every record."""
    out: dict = {p: [] for p in file_address}
    bases = sorted((a, p) for p, a in file_address.items())
    for src, _dst, rows, rb, sp, _dp in items.tolist():
        if not rows or not rb:
            continue
        for a, p in reversed(bases):
            if src >= a:
                out[p].append((src - a, (rows - 1) * sp + rb))
                break
    return out


def torch_dtype(tag: str):
    import torch

    return getattr(torch, SAFETENSORS_DTYPES[tag][1])


def allocate_params(plan: CheckpointPlan, device) -> dict:
    """Fresh device tensors for every parameter of the plan (zero-filled where
    the checkpoint does not cover every byte, e.g. vocabulary padding)."""
    import torch

    out = {}
    for name, spec in plan.params.items():
        maker = torch.zeros if spec.zero_fill else torch.empty
        out[name] = maker(tuple(spec.shape), dtype=torch_dtype(spec.dtype), device=device)
    return out


def placement_items(plan: CheckpointPlan, index: dict, file_address: dict, params: dict) -> np.ndarray:
    """(n, 6) uint64 records: host source address -> device destination address."""
    items = np.empty((len(plan.placements), 6), dtype=np.uint64)
    for i, pl in enumerate(plan.placements):
        info = index[pl.src_name]
        dst = params[pl.dst_name]
        spec = plan.params[pl.dst_name]
        if tuple(dst.shape) != tuple(spec.shape) or not dst.is_contiguous():
            raise ValueError(f"{pl.dst_name}: destination tensor must be contiguous with shape "
                             f"{tuple(spec.shape)}, got {tuple(dst.shape)}")
        if dst.element_size() != SAFETENSORS_DTYPES[pl.dtype][0]:
            raise ValueError(f"{pl.dst_name}: element size differs from the checkpoint's {pl.dtype}")
        items[i] = pl.record(file_address[info["file"]] + info["file_offset"], dst.data_ptr())
    return items


@dataclass
class PlacedCheckpoint:
    params: dict
    plan: CheckpointPlan
    stats: PlaceResult
    timings: dict = field(default_factory=dict)   # seconds per phase of the call


def place_checkpoint(model_path: str, tp_rank: int, tp_size: int, device=None, *,
                     params: dict | None = None, ring: Ring | None = None,
                     ctx: Context | None = None, host_threads: int | None = None,
                     mode: int = PLACE_COPY_ENGINE, family: str = "auto",
                     ring_bytes: int = RING_BYTES, ring_slots: int = RING_SLOTS,
                     pin: str = "off", images: HostImages | None = None) -> PlacedCheckpoint:
    """Load this rank's tensor-parallel shards of a safetensors checkpoint.

    ``params`` may hold pre-allocated destination tensors (an engine's own
    parameters, keyed by the engine's names); otherwise they are allocated.

    ``pin`` decides what is kept in host memory for later loads of the same files:
    ``"off"``          nothing: map the files, gather through the pinned ring, unmap;
    ``"keep"``         this rank's bytes, packed as they cross PCIe, in page-locked memory
                       (as large as the rank's shard).  The first load gathers into that
                       image instead of the ring; every later load is one contiguous
                       copy-engine transfer and one scatter launch per chunk, with no host
                       thread and no file access;
    ``"pages"``        the files stay mapped in ``images`` (default: the process-wide
                       ``host_images``) and the page ranges this rank reads are page-locked
                       before placing, so that the copy engine gathers from the files' own
                       pages; costs no extra memory but far more time to pin;
    ``"pages_after"``  place through the ring now and page-lock the ranges on a background
                       thread for the loads to come.
    """
    import torch

    if pin not in PIN_MODES:
        raise ValueError(f"pin must be one of {PIN_MODES}, not {pin!r}")
    timings: dict = {}
    t_start = time.perf_counter()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError("place_checkpoint needs a CUDA device (no CPU fallback)")
    dev_index = dev.index if dev.index is not None else torch.cuda.current_device()
    cache = (images if images is not None else host_images) if pin != "off" else None
    prep = (cache.prepared(model_path, tp_rank, tp_size, family) if cache is not None
            else Prepared.build(model_path, tp_rank, tp_size, family))
    index, plan = prep.index, prep.plan
    timings["index_and_plan"] = time.perf_counter() - t_start
    if ctx is None:
        ctx = ring.ctx if ring is not None else default_context(dev_index)
    t = time.perf_counter()
    if ring is None:
        ring = ctx.cached_ring(ring_bytes, ring_slots, dev_index)   # made once, kept for later loads
    timings["ring_create"] = time.perf_counter() - t
    if params is None:
        params = allocate_params(plan, dev)
    else:
        # bytes the checkpoint does not cover (vocabulary padding rows) must read as zero,
        # as they do after the engine's own loader
        for name, spec in plan.params.items():
            if spec.zero_fill and name in params:
                params[name].zero_()
    # the library works on its own streams: whatever the caller queued on torch's
    # stream for these tensors (allocation fills, earlier writes) must be done first
    torch.cuda.current_stream(dev).synchronize()
    opened = {}
    try:
        t = time.perf_counter()
        for path in prep.files:
            opened[path] = cache.open(path) if cache is not None else FileImage(path)
        timings["map"] = time.perf_counter() - t
        addresses = {p: im.address for p, im in opened.items()}
        items = prep.items(addresses, params)
        timings["pin"] = 0.0
        ids = tuple(id(opened[p]) for p in prep.files)
        if pin == "pages" and prep.pinned_in != ids:
            t = time.perf_counter()
            for p, spans in item_spans(items, addresses, None).items():
                opened[p].pin_spans(spans)
            prep.pinned_in = ids
            timings["pin"] = time.perf_counter() - t
        # three quarters of the cores: the gather threads share DRAM bandwidth with the PCIe DMA
        threads = host_threads or max(2, min(32, (os.cpu_count() or 8) * 3 // 4))
        t = time.perf_counter()
        stats = None
        if pin == "keep":
            packed = prep.packed.get(dev_index)
            if packed is not None and packed._h:
                try:
                    stats = packed.place(items)
                except MxbError as e:
                    if e.code != -8:      # anything but "the destinations no longer fit this image"
                        raise
                    packed.close()
            if stats is None:
                prep.packed[dev_index], stats = ring.keep(items, threads)
        else:
            stats = ring.place(items, threads, mode)
        timings["place"] = time.perf_counter() - t
        if pin == "pages_after" and prep.pinned_in != ids:
            spans = item_spans(items, addresses, None)

            def pin_later():
                for p, sp in spans.items():
                    opened[p].pin_spans(sp)
                prep.pinned_in = ids

            bg = threading.Thread(target=pin_later, name="mxb-pin", daemon=True)
            bg.start()
            ctx._background.append(bg)
    finally:
        _release(ctx, opened.values() if cache is None else (), None)
    timings["total"] = time.perf_counter() - t_start
    return PlacedCheckpoint(params, plan, stats, {k: round(v, 6) for k, v in timings.items()})


@dataclass
class CapturedPlacement:
    """Outcome of ``place_captured``."""

    stats: PlaceResult
    copies: int                 # recorded copies that became scatter records
    records: int
    converted: list             # parameters filled through a dtype cast
    engine_loaded: list         # sources left to the engine's own loader
    reasons: dict               # source -> why capture or planning gave it up
    written_params: set         # parameters and buffers that received records
    timings: dict = field(default_factory=dict)   # seconds: capture, ring_create, place_wait, engine


class _Leftovers:
    def __init__(self, images, ring):
        self.images, self.ring = list(images), ring

    def close(self) -> None:
        for im in self.images:
            try:
                im.close()
            except BufferError:   # a tensor over the mapping is still alive: the GC unmaps it
                pass
        if self.ring is not None:
            self.ring.close()


def _release(ctx: Context, images, ring: Ring | None) -> None:
    """What a load leaves behind is torn down off the caller's path: unmapping the
    checkpoint files is tens of milliseconds of page-table work for a fresh mapping of
    a tmpfs file; the loaded weights do not wait for it."""
    ctx.release_later(_Leftovers(images, ring))


def _engine_tensor(image: FileImage, info: dict):
    """A real (host) tensor over the checkpoint bytes, for the engine's loader."""
    import torch

    import warnings

    with warnings.catch_warnings():
        # the mapping is read-only and so is every use the engine's loader makes of a source
        warnings.filterwarnings("ignore", message="The given buffer is not writable")
        raw = torch.frombuffer(image._mm, dtype=torch.uint8, count=int(info["size"]),
                               offset=int(info["file_offset"]))
    return raw.view(torch_dtype(info["dtype"])).reshape(tuple(info["shape"]))


@dataclass
class CapturedTable:
    """What one capture of an engine's loader compiles to."""

    records: np.ndarray         # (n, 6) uint64 scatter records
    converts: list              # planner.ConvertSpec for copies that change dtype
    staging_bytes: int          # device staging those converts need
    reasons: dict               # source -> why it is left to the engine's loader
    copies: int                 # recorded copies that became records
    written_params: set         # parameters and buffers at least one record writes into


def model_destinations(model) -> dict:
    """{name: tensor} over parameters and buffers, shared ones under every name."""
    import torch

    return {n: (t.data if isinstance(t, torch.nn.Parameter) else t)
            for n, t in list(model.named_parameters(remove_duplicate=False))
            + list(model.named_buffers(remove_duplicate=False))}


def captured_table(model, index: dict, file_address: dict, *, load_weights=None, device=None,
                   alloc_staging=None, dests: dict | None = None, state=None,
                   min_row_bytes: int = 16) -> CapturedTable:
    """Dry-run ``load_weights`` over the checkpoint's header and compile what it
    copies into scatter records from ``file_address[file] + file_offset`` to the
    model's own tensors.  ``alloc_staging(nbytes) -> address`` provides the
    buffer dtype-changing copies are staged in; without it such copies are left
    to the engine's loader.  ``state`` (``geometry.CaptureState``) is shared by the
    calls that compile one checkpoint part by part.  A copy that transposes its
    source element by element (GPT-2's Conv1D weights) is a correct but wasteful
    record list of rows narrower than ``min_row_bytes``; such sources are left to
    the engine's loader (0 keeps them)."""
    from .geometry import capture_geometry
    from .planner import ShardSpec, SourceSpec, convert_staging_bytes, plan_transfer_2d

    loader = load_weights if load_weights is not None else model.load_weights
    manifest = [(n, torch_dtype(i["dtype"]), tuple(i["shape"])) for n, i in index.items()]
    cap = capture_geometry(model, manifest, loader, device=device, state=state)
    if dests is None:
        dests = model_destinations(model)
    sources = {}
    for name, info in index.items():
        elsize = SAFETENSORS_DTYPES[info["dtype"]][0]
        shape = tuple(int(x) for x in info["shape"])
        sources[name] = SourceSpec(shape, torch_dtype(info["dtype"]), elsize, [
            ShardSpec(tuple(0 for _ in shape), shape, info["file"],
                      int(file_address[info["file"]]) + int(info["file_offset"]), elsize)])
    staging_bytes = convert_staging_bytes(cap.copies, sources) if alloc_staging is not None else 0
    convert_base = int(alloc_staging(staging_bytes)) if staging_bytes else None
    table, not_planned, converts = plan_transfer_2d(
        cap.copies, sources, lambda n: dests[n].data_ptr(), convert_base)
    reasons = dict(cap.unsupported_reasons)
    for n in not_planned:
        reasons.setdefault(n, "the copied window is not a box of the source tensor, or changes dtype")
    dropped = set(not_planned)
    if min_row_bytes and len(table):
        # rows narrower than this, many of them: an element-wise transpose
        narrow = (table[:, 3] < np.uint64(min_row_bytes)) & (table[:, 2] > np.uint64(64))
        if narrow.any():
            transposed = set()
            for c in cap.copies:
                if c.src_name in dropped or len(c.src_stride) < 2 or c.src_stride[-1] == 1:
                    continue
                transposed.add(c.src_name)
            if transposed:
                keep = [c for c in cap.copies if c.src_name not in transposed and c.src_name not in dropped]
                table, _np2, converts = plan_transfer_2d(keep, sources, lambda n: dests[n].data_ptr(),
                                                         convert_base)
                for n in transposed:
                    reasons.setdefault(n, "the copy transposes the source element by element")
                dropped |= transposed
    planned = [c for c in cap.copies if c.src_name not in dropped]
    return CapturedTable(table, converts, staging_bytes, reasons, len(planned),
                         {c.param_name for c in planned})


def place_captured(model, model_path: str, device=None, *, load_weights=None,
                   ring: Ring | None = None, ctx: Context | None = None,
                   host_threads: int | None = None, mode: int = PLACE_COPY_ENGINE,
                   ring_bytes: int = RING_BYTES, ring_slots: int = RING_SLOTS,
                   on_unsupported: str = "engine", pipeline: bool = True,
                   first_batch: int = 32, min_row_bytes: int = 16, pin: str = "off",
                   images: HostImages | None = None) -> CapturedPlacement:
    """Load a safetensors checkpoint into ``model`` for ANY architecture whose
    engine-side ``load_weights`` only slices and copies.

    The engine's own loader is dry-run once over byte-less placeholders
    (``geometry.capture_geometry``), which yields, for this rank, the exact window
    of every checkpoint tensor and where it lands — fused projections, expert
    stacks, tensor-parallel shards, vocabulary padding, renamed or skipped
    tensors, all as the engine itself decides them.  Those copies become 2-D
    records (``planner.plan_transfer_2d``; the file is the single published shard
    of each tensor) and go through the pinned ring and the scatter kernel.  A
    copy whose checkpoint dtype differs from the parameter's is staged on the
    device and cast there.  Sources the loader has to compute on (a scalar read
    with ``.item()``, a transposing ``contiguous()``) are few and small: with
    ``on_unsupported="engine"`` they are handed to the same ``load_weights`` as
    real host tensors afterwards (so where two sources write the same bytes,
    the engine-loaded one wins), with ``"raise"`` the call fails before any
    byte is written.  ``stats.seconds_total`` spans the dry run and the
    placement, which overlap (``pipeline``).  ``pin`` as in ``place_checkpoint``; with
    ``"keep"`` a later load of the same files into a model of the same shapes skips the
    dry run and the gather and replays the kept images (engines that reload weights
    into a live model, e.g. after a sleep, take this path).
    An exception of the engine's loader that arrives after the first batch has been
    handed to the ring is re-raised as ``StrategyFailed(mutated=True)``: parameter
    bytes have been overwritten by then."""
    import torch

    from .planner import apply_converts

    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError("place_captured needs a CUDA device (no CPU fallback)")
    dev_index = dev.index if dev.index is not None else torch.cuda.current_device()
    loader = load_weights if load_weights is not None else model.load_weights
    index = checkpoint_index(model_path)
    dests = model_destinations(model)
    if ctx is None:
        ctx = ring.ctx if ring is not None else default_context(dev_index)
    if pin not in PIN_MODES:
        raise ValueError(f"pin must be one of {PIN_MODES}, not {pin!r}")
    cache = (images if images is not None else host_images) if pin != "off" else None
    files = sorted({i["file"] for i in index.values()})
    stamps = Prepared._stamps(model_path, files)
    kept_key = (os.path.realpath(model_path), dev_index)
    if pin == "keep":
        kept = cache._captured.get(kept_key)
        if kept is not None and kept.stamps == stamps:
            replay = _replay_captured(kept, model, dests, loader, index, cache, dev)
            if replay is not None:
                return replay
        if kept is not None:
            cache._captured.pop(kept_key).close()
    images = {}
    pool = ThreadPoolExecutor(1)          # the ring is one pipeline: its calls run in order
    made: list = []
    try:
        for path in files:
            images[path] = cache.open(path) if cache is not None else FileImage(path)
        check_index(index, {p: im.size for p, im in images.items()})
        addresses = {p: im.address for p, im in images.items()}
        threads = host_threads or max(2, min(32, (os.cpu_count() or 8) * 3 // 4))
        names = list(index)
        # the dry run costs tens of microseconds of Python per tensor: it is done in batches
        # (small first, then doubling) so that the ring is already moving batch k while
        # batch k+1 is being captured
        cuts, step = [0], max(1, int(first_batch))
        while cuts[-1] < len(names):
            cuts.append(min(len(names), cuts[-1] + step))
            step *= 2
        if not pipeline or on_unsupported != "engine":
            cuts = [0, len(names)]       # one batch: nothing is written before all is planned
        from .geometry import CaptureState

        state = CaptureState(model)
        parts, pending, stagings = [], [], []
        timings = {"capture": 0.0, "ring_create": 0.0, "place_wait": 0.0, "engine": 0.0}
        t0 = time.perf_counter()

        def make_ring():
            # first job of the placing thread: pinning the ring overlaps the first dry-run batch
            tc = time.perf_counter()
            made.append(ctx.cached_ring(ring_bytes, ring_slots, dev_index))
            timings["ring_create"] = time.perf_counter() - tc

        kept_batches: list = []

        def place_batch(records):
            r = ring if ring is not None else made[0]
            if pin != "keep":
                return r.place(records, threads, mode)
            img, stats = r.keep(records, threads)
            kept_batches.append((img, records, _record_homes(records, dests, stagings)))
            return stats

        ring_job = pool.submit(make_ring) if ring is None else None
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            held = []

            def alloc_staging(nbytes: int, held=held) -> int:
                held.append(torch.empty(nbytes, dtype=torch.uint8, device=dev))
                return held[0].data_ptr()

            tc = time.perf_counter()
            try:
                cap = captured_table(model, {n: index[n] for n in names[lo:hi]}, addresses,
                                     load_weights=loader, device=dev, alloc_staging=alloc_staging,
                                     dests=dests, state=state, min_row_bytes=min_row_bytes)
            except Exception as e:
                if pending:     # earlier batches are already being written
                    raise StrategyFailed(f"{type(e).__name__}: {e}", mutated=True) from e
                raise
            timings["capture"] += time.perf_counter() - tc
            parts.append(cap)
            if cap.reasons and on_unsupported != "engine":
                first = next(iter(cap.reasons))
                raise StrategyFailed(
                    f"{len(cap.reasons)} source tensor(s) need the engine's loader, e.g. "
                    f"{first}: {cap.reasons[first]}", mutated=False)
            if cap.converts:
                stagings.append((cap.converts, held[0]))
            if len(cap.records):
                # the library works on its own streams: what the caller (or the dry run's
                # real side effects, e.g. zeroed vocabulary padding) queued on torch's
                # stream must be done before these destinations are written
                torch.cuda.current_stream(dev).synchronize()
                if pin == "pages":
                    tp = time.perf_counter()
                    for p, spans in item_spans(cap.records, addresses).items():
                        images[p].pin_spans(spans)
                    timings["pin"] = timings.get("pin", 0.0) + time.perf_counter() - tp
                pending.append(pool.submit(place_batch, cap.records))
        tc = time.perf_counter()
        if ring_job is not None:
            ring_job.result()
        results = [f.result() for f in pending]
        timings["place_wait"] = time.perf_counter() - tc
        seconds = time.perf_counter() - t0
        for converts, buf in stagings:
            apply_converts(converts, buf, dests, ctx)
        reasons = {}
        for cap in parts:
            reasons.update(cap.reasons)
        leftover = [n for n in names if n in reasons]
        if leftover:
            tc = time.perf_counter()
            loader((n, _engine_tensor(images[index[n]["file"]], index[n])) for n in leftover)
            timings["engine"] = time.perf_counter() - tc
        torch.cuda.current_stream(dev).synchronize()
        if pin == "keep":
            written_now = set()
            for cap in parts:
                written_now |= cap.written_params
            cache._captured[kept_key] = _KeptCapture(
                stamps, kept_batches, list(stagings), list(leftover),
                {"copies": sum(c.copies for c in parts), "records": sum(len(c.records) for c in parts),
                 "reasons": dict(reasons), "written_params": written_now})
        if pin == "pages_after":
            spans_all: dict = {}
            for part in parts:
                for p, spans in item_spans(part.records, addresses).items():
                    spans_all.setdefault(p, []).extend(spans)
            bg = threading.Thread(target=lambda: [images[p].pin_spans(sp) for p, sp in spans_all.items()],
                                  name="mxb-pin", daemon=True)
            bg.start()
            ctx._background.append(bg)
    finally:
        pool.shutdown(wait=True)
        _release(ctx, images.values() if cache is None else (), None)
    stats = PlaceResult(sum(r.bytes_placed for r in results), sum(r.chunks for r in results),
                        sum(r.launches for r in results), seconds,
                        sum(r.seconds_gather for r in results), sum(r.seconds_device for r in results))
    written = set()
    for cap in parts:
        written |= cap.written_params
    return CapturedPlacement(stats, sum(c.copies for c in parts), sum(len(c.records) for c in parts),
                             [c.param_name for cv, _b in stagings for c in cv], leftover, reasons,
                             written, {k: round(v, 4) for k, v in timings.items()})


def _record_homes(records: np.ndarray, dests: dict, stagings: list) -> list:
    """(destination name, byte offset) of every record: which parameter, buffer or cast
    staging buffer its destination address lies in."""
    spans = []
    for name, t in dests.items():
        n = t.numel() * t.element_size()
        if n:
            spans.append((t.data_ptr(), t.data_ptr() + n, name))
    for k, (_conv, buf) in enumerate(stagings):
        spans.append((buf.data_ptr(), buf.data_ptr() + buf.numel(), f"\0staging{k}"))
    spans.sort()
    starts = np.array([s[0] for s in spans], dtype=np.uint64)
    homes = []
    for dst in records[:, 1].tolist():
        k = int(np.searchsorted(starts, np.uint64(dst), side="right")) - 1
        if k < 0 or dst >= spans[k][1]:
            raise RuntimeError("a record's destination lies in no known tensor")
        homes.append((spans[k][2], int(dst - spans[k][0])))
    return homes


def _replay_captured(kept: _KeptCapture, model, dests: dict, loader, index: dict, cache, dev):
    """A load from kept images: no dry run, no gather.  Returns ``None`` when the model no
    longer fits what was kept (another shape, or a destination at another 16-byte phase)."""
    import torch

    from .planner import apply_converts

    t0 = time.perf_counter()
    bases = {name: t.data_ptr() for name, t in dests.items()}
    for k, (_conv, buf) in enumerate(kept.stagings):
        bases[f"\0staging{k}"] = buf.data_ptr()
    torch.cuda.current_stream(dev).synchronize()
    results = []
    try:
        for img, records, homes in kept.batches:
            items = records.copy()
            items[:, 1] = np.array([bases[name] + off for name, off in homes], dtype=np.uint64)
            results.append(img.place(items))
    except (KeyError, MxbError) as e:
        if isinstance(e, MxbError) and e.code != -8:
            raise
        if results:      # some batches were written before the mismatch showed
            raise StrategyFailed(f"kept image no longer fits the model: {e}", mutated=True) from e
        return None
    for converts, buf in kept.stagings:
        apply_converts(converts, buf, dests)
    timings = {"capture": 0.0, "ring_create": 0.0, "place_wait": round(time.perf_counter() - t0, 4),
               "engine": 0.0}
    if kept.leftover:
        tc = time.perf_counter()
        opened = {p: cache.open(p) for p in sorted({index[n]["file"] for n in kept.leftover})}
        loader((n, _engine_tensor(opened[index[n]["file"]], index[n])) for n in kept.leftover)
        timings["engine"] = round(time.perf_counter() - tc, 4)
    torch.cuda.current_stream(dev).synchronize()
    seconds = time.perf_counter() - t0
    stats = PlaceResult(sum(r.bytes_placed for r in results), sum(r.chunks for r in results),
                        sum(r.launches for r in results), seconds, 0.0,
                        sum(r.seconds_device for r in results), sum(r.bytes_direct for r in results), 0.0)
    return CapturedPlacement(stats, kept.summary["copies"], kept.summary["records"],
                             [c.param_name for cv, _b in kept.stagings for c in cv], list(kept.leftover),
                             dict(kept.summary["reasons"]), set(kept.summary["written_params"]), timings)


class B200ScatterStrategy:
    """Load strategy placing weights with the scatter kernel.

    Plug it ahead of the engine-native fallback in the chain
    (load_strategy/__init__.py:71-78).  ``ctx`` needs ``model_config.model``
    (checkpoint directory), ``device_id`` and ``adapter``; the adapter must offer
    ``tp_layout(result) -> (tp_rank, tp_size)`` and
    ``named_destinations(result) -> {param_name: tensor}`` so that bytes land
    in the engine's own parameters.
    """

    name = "b200_scatter"
    requires: tuple = ()

    def __init__(self, ring_bytes: int = RING_BYTES, ring_slots: int = RING_SLOTS, host_threads: int | None = None,
                 pin: str | None = None):
        self.ring_bytes, self.ring_slots, self.host_threads = ring_bytes, ring_slots, host_threads
        # what to keep in host memory for later loads (place_checkpoint's ``pin``); MXB_PIN=keep
        # suits engines that reload weights into a live model
        self.pin = pin if pin is not None else os.environ.get("MXB_PIN", "off")
        self._touched = False

    def is_available(self, ctx) -> bool:
        try:
            import torch

            from . import _lib

            _lib.load()
            return bool(torch.cuda.is_available()) and getattr(ctx, "adapter", None) is not None
        except Exception:
            return False

    def load(self, result: LoadResult, ctx) -> LoadResult:
        model_dir = getattr(ctx.model_config, "model", None)
        if not model_dir or not os.path.isdir(model_dir):
            raise StrategyFailed(f"no local checkpoint directory at {model_dir!r}", mutated=False)
        try:
            tp_rank, tp_size = ctx.adapter.tp_layout(result)
            params = ctx.adapter.named_destinations(result)
        except AttributeError as e:
            raise StrategyFailed(f"adapter lacks a hook this strategy needs: {e}", mutated=False) from e
        self._touched = False
        try:
            self._touched = True
            placed = place_checkpoint(model_dir, tp_rank, tp_size, f"cuda:{ctx.device_id}",
                                      params=params, ring_bytes=self.ring_bytes,
                                      ring_slots=self.ring_slots, host_threads=self.host_threads,
                                      pin=self.pin)
        except (KeyError, ValueError) as e:
            # layout could not be expressed: nothing was written yet
            raise StrategyFailed(str(e), mutated=False) from e
        except Exception as e:
            raise StrategyFailed(str(e), mutated=True) from e
        result.metadata["b200_scatter"] = {
            "bytes_placed": placed.stats.bytes_placed, "seconds": placed.stats.seconds_total,
            "chunks": placed.stats.chunks}
        return result

    def rollback(self, ctx) -> None:
        self._touched = False


class B200CapturedStrategy(B200ScatterStrategy):
    """The same placement, planned from the engine's own ``load_weights`` instead of
    layout rules (``place_captured``): it covers whatever architecture the engine
    can load.  The adapter needs one hook, ``model_of(result) -> torch.nn.Module``
    (default: ``result.model``); ranks and shard shapes are whatever the engine's
    loader makes of its parallel state."""

    name = "b200_captured"

    def load(self, result: LoadResult, ctx) -> LoadResult:
        model_dir = getattr(ctx.model_config, "model", None)
        if not model_dir or not os.path.isdir(model_dir):
            raise StrategyFailed(f"no local checkpoint directory at {model_dir!r}", mutated=False)
        hook = getattr(ctx.adapter, "model_of", None)
        model = hook(result) if hook is not None else result.model
        if model is None or not hasattr(model, "load_weights"):
            raise StrategyFailed("the engine model has no load_weights to capture", mutated=False)
        self._touched = True
        try:
            placed = place_captured(model, model_dir, f"cuda:{ctx.device_id}",
                                    ring_bytes=self.ring_bytes, ring_slots=self.ring_slots,
                                    host_threads=self.host_threads, pin=self.pin)
        except StrategyFailed:
            raise
        except (KeyError, ValueError, FileNotFoundError) as e:
            raise StrategyFailed(str(e), mutated=False) from e
        except Exception as e:
            raise StrategyFailed(str(e), mutated=True) from e
        result.metadata[self.name] = {
            "bytes_placed": placed.stats.bytes_placed, "seconds": placed.stats.seconds_total,
            "chunks": placed.stats.chunks, "records": placed.records,
            "engine_loaded": len(placed.engine_loaded), "converted": len(placed.converted),
            "timings": placed.timings}
        return result
