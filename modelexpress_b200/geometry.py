"""Geometry capture: which window of each checkpoint tensor an engine's own weight
loader copies into which window of which parameter.

The reference dry-runs ``model.load_weights`` with zero-storage placeholders that
append every view op to a chain, stamps each parameter's ``weight_loader`` to know
where a ``copy_`` lands, and later replays the chain on a ``meta`` tensor
(refit/reshard/geometry.py:100-301, refit/reshard/slice_plan.py:136-167).  This
module reaches the same facts by a different route:

* a ``TracedSource`` carries a ``meta`` *window* of its full tensor.  Every op a
  loader applies runs on that window at once, and is accepted if and only if the
  result is still a view of the same storage — there is no allowlist to maintain
  and no replay: ``chunk``, ``unbind``, ``select``, ``split``, ``squeeze`` and the
  rest work because torch itself says they are views.  Anything that would need
  the bytes (arithmetic, a dtype cast, ``.item()``, a materialising
  ``contiguous()``) raises ``UnsupportedReshard`` for that source only;
* the sink (``copy_`` or ``dest[key] = src``) finds the destination parameter by
  the *storage* the written tensor lives in, so loaders need no stamping, buffers
  and default loaders are covered, and the recorded offset is relative to the
  parameter even when it is itself a view into a larger arena.  A write into a
  tensor that is no parameter (a temporary the loader transforms afterwards)
  makes the source unsupported instead of silently incomplete;
* all sources go through ONE ``load_weights`` call; a source that fails is
  dropped and the call resumes behind it;
* the dry run is watched: a real op that reads or writes a region some source
  was already recorded into (a loader that rescales a parameter in place after
  copying into it, or derives a second tensor from it) ran on bytes that had not
  landed, so that source is given up too instead of ending up subtly wrong.

The recorded ``ViewCopy`` holds the window as ``(offset, shape, stride)`` in
elements of the full source tensor.  ``planner.plan_pull_2d`` turns it into
scatter records; no tensor data is touched anywhere here.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import Any, Callable, Iterable

import torch
import torch.utils._python_dispatch

from .planner import UnsupportedReshard

logger = logging.getLogger("modelexpress_b200.geometry")

__all__ = ["ViewCopy", "CaptureResult", "CaptureState", "TracedSource", "capture_geometry",
           "summarize_unsupported"]


@dataclass
class ViewCopy:
    """One recorded ``dest.copy_(window of source)``.

    ``src_*`` describe the window in elements of the full, row-major source
    tensor; ``dest_*`` describe where it lands in elements relative to element 0
    of parameter ``param_name`` (the reference's RecordedCopy, types.py:57-70,
    carries an op-chain in place of the resolved window)."""

    src_name: str
    src_offset: int
    src_shape: tuple
    src_stride: tuple
    src_dtype: Any
    param_name: str
    dest_offset: int
    dest_shape: tuple
    dest_stride: tuple
    dest_dtype: Any


@dataclass
class CaptureResult:
    """types.py:73-86 with the same field meanings; ``unattributed`` counts writes
    into tensors that are not parameters (their sources are also listed in
    ``unsupported``)."""

    copies: list = field(default_factory=list)
    unsupported: list = field(default_factory=list)
    unattributed: int = 0
    unsupported_reasons: dict = field(default_factory=dict)


def summarize_unsupported(reasons: dict | None) -> list:
    """Distinct causes with their counts, most frequent first (types.py:27-54)."""
    counts: dict = {}
    for why in (reasons or {}).values():
        counts[why] = counts.get(why, 0) + 1
    return sorted(counts.items(), key=lambda kv: (-kv[1], kv[0]))


class _Recorder:
    def __init__(self, model: torch.nn.Module):
        # storage identity -> [(name, first element, elements)]
        self.by_storage: dict = {}
        tensors = list(model.named_parameters(remove_duplicate=False))
        tensors += list(model.named_buffers(remove_duplicate=False))
        for name, t in tensors:
            data = t.data if isinstance(t, torch.nn.Parameter) else t
            key = data.untyped_storage()._cdata
            span = _extent(data)
            self.by_storage.setdefault(key, []).append((name, int(data.storage_offset()), span))
        self.copies: list = []
        self.unattributed = 0
        self.written: dict = {}   # storage identity -> [(first element, one past last, source)]
        self.tainted: dict = {}   # source -> why its recorded copies cannot be trusted
        self.current = None       # the source most recently handed to the loader

    def touch(self, t: torch.Tensor, what: str) -> None:
        """A real op reads or writes ``t``: every source already recorded into an
        overlapping region is tainted, because the op ran on bytes that will only
        land later (a loader that rescales a parameter after copying into it)."""
        try:
            regions = self.written.get(t.untyped_storage()._cdata)
        except (RuntimeError, NotImplementedError):   # a tensor type without storage
            return
        if not regions:
            return
        lo = int(t.storage_offset())
        hi = lo + _extent(t)
        for first, last, src in regions:
            if lo < last and first < hi:
                self.tainted.setdefault(src, f"the loader runs {what} on the destination after the copy")
                # the source being loaded right now used those bytes: it has to run again
                # once they are really there
                if self.current is not None and self.current != src:
                    self.tainted.setdefault(
                        self.current, f"its loader runs {what} on bytes that {src!r} provides")

    def owner(self, dest: torch.Tensor):
        """(parameter name, offset of ``dest`` relative to it) or None."""
        cands = self.by_storage.get(dest.untyped_storage()._cdata)
        if not cands:
            return None
        lo = int(dest.storage_offset())
        hi = lo + _extent(dest)
        for name, first, span in cands:
            if first <= lo and hi <= first + span:
                return name, lo - first
        return None


def _extent(t: torch.Tensor) -> int:
    """Elements from the first to one past the last element ``t`` addresses."""
    if t.numel() == 0:
        return 0
    return 1 + sum((int(n) - 1) * int(s) for n, s in zip(t.shape, t.stride()))


def _leaves(tree):
    """Tensors among call arguments: the arguments themselves and what lists,
    tuples and dicts of them hold (``torch.cat([a, b])``)."""
    out, stack = [], [tree]
    while stack:
        x = stack.pop()
        if isinstance(x, torch.Tensor):
            out.append(x)
        elif isinstance(x, (list, tuple)):
            stack.extend(x)
        elif isinstance(x, dict):
            stack.extend(x.values())
    return out


def _is_identity_move(func, args, kwargs) -> bool:
    """``.to(device)`` / ``.cuda()`` / ``.to(same dtype)``: no change of bytes."""
    if func is torch.Tensor.cuda or func is torch.Tensor.cpu:
        return True
    if func is not torch.Tensor.to:
        return False
    me = args[0]
    if kwargs.get("copy"):
        return False
    for a in list(args[1:]) + [kwargs.get("dtype"), kwargs.get("other")]:
        if isinstance(a, torch.dtype) and a != me.dtype:
            return False
        if isinstance(a, torch.Tensor) and a.dtype != me.dtype:
            return False
    return True


class TracedSource(torch.Tensor):
    """A checkpoint tensor without bytes: shape, dtype and device answer as usual,
    view ops return further ``TracedSource`` windows, writes are recorded."""

    _name: str
    _window: torch.Tensor      # meta view into _base_meta
    _base_meta: torch.Tensor   # meta, the full tensor
    _rec: Any

    @staticmethod
    def __new__(cls, name, base, window, device, rec):
        t = torch.Tensor._make_wrapper_subclass(
            cls, window.shape, strides=window.stride(), storage_offset=window.storage_offset(),
            dtype=window.dtype, device=device, requires_grad=False)
        t._name, t._base_meta, t._window, t._rec = name, base, window, rec
        return t

    @classmethod
    def source(cls, name: str, shape, dtype, device="cpu", rec=None) -> "TracedSource":
        base = torch.empty(tuple(int(s) for s in shape), dtype=dtype, device="meta")
        return cls(name, base, base, device, rec)

    def _wrap(self, window: torch.Tensor) -> "TracedSource":
        return TracedSource(self._name, self._base_meta, window, self.device, self._rec)

    def _is_view(self, t: torch.Tensor) -> bool:
        # same storage and same element type: a window of the source's bytes
        base = self._base_meta
        return (t.dtype == base.dtype and t.device.type == "meta"
                and t.untyped_storage()._cdata == base.untyped_storage()._cdata)

    def _fail(self, what: str):
        raise _Unsupported(self._name, what)

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func is torch.Tensor.copy_ and len(args) >= 2 and isinstance(args[1], cls) \
                and not isinstance(args[0], cls):
            return args[1]._sink(args[0])
        if func is torch.Tensor.__setitem__ and len(args) == 3 and isinstance(args[2], cls) \
                and not isinstance(args[0], cls):
            with torch._C.DisableTorchFunctionSubclass():
                dest = args[0][args[1]]
            src = args[2]
            if tuple(dest.shape) != tuple(src.shape):
                src._fail(f"assignment broadcasts {tuple(src.shape)} into {tuple(dest.shape)}")
            src._sink(dest)
            return None
        traced = [a for a in _leaves((args, kwargs)) if isinstance(a, cls)]
        me = args[0] if args and isinstance(args[0], cls) else None
        if me is None or len(traced) != 1:
            who = traced[0] if traced else None
            name = getattr(func, "__name__", str(func))
            if who is None:
                with torch._C.DisableTorchFunctionSubclass():
                    return func(*args, **kwargs)
            who._fail(f"{name} takes the source as an operand")
        if _is_identity_move(func, args, kwargs):
            return me
        try:
            with torch._C.DisableTorchFunctionSubclass():
                out = func(me._window, *args[1:], **kwargs)
        except _Unsupported:
            raise
        except Exception as e:
            me._fail(f"{getattr(func, '__name__', func)} needs the tensor's bytes ({type(e).__name__})")
        if isinstance(out, torch.Tensor):
            if not me._is_view(out):
                me._fail(f"{getattr(func, '__name__', func)} is not a view of the source")
            return me._wrap(out)
        if isinstance(out, (tuple, list)) and out and all(isinstance(o, torch.Tensor) for o in out):
            if not all(me._is_view(o) for o in out):
                me._fail(f"{getattr(func, '__name__', func)} is not a view of the source")
            return type(out)(me._wrap(o) for o in out)
        # metadata (shape, dtype, device, dim(), numel(), ...): answer from the wrapper,
        # whose device is the one the source claims to live on
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        if func is torch.ops.aten.copy_.default and len(args) >= 2 and isinstance(args[1], cls) \
                and not isinstance(args[0], cls):
            # a destination class that runs copy_ with subclass overrides switched off
            return args[1]._sink(args[0])
        for a in _leaves((args, kwargs or {})):
            if isinstance(a, cls):
                a._fail(f"{func} needs the tensor's bytes")
        return func(*args, **(kwargs or {}))

    def _sink(self, dest: torch.Tensor):
        rec = self._rec
        if rec is None:
            return dest
        if tuple(dest.shape) != tuple(self.shape):
            self._fail(f"copy_ broadcasts {tuple(self.shape)} into {tuple(dest.shape)}")
        found = rec.owner(dest)
        if found is None:
            rec.unattributed += 1
            self._fail("written into a tensor that is not a parameter or buffer of the model")
        name, offset = found
        w = self._window
        lo = int(dest.storage_offset())
        rec.written.setdefault(dest.untyped_storage()._cdata, []).append(
            (lo, lo + _extent(dest), self._name))
        rec.copies.append(ViewCopy(
            src_name=self._name, src_offset=int(w.storage_offset()),
            src_shape=tuple(int(s) for s in w.shape), src_stride=tuple(int(s) for s in w.stride()),
            src_dtype=w.dtype, param_name=name, dest_offset=int(offset),
            dest_shape=tuple(int(s) for s in dest.shape),
            dest_stride=tuple(int(s) for s in dest.stride()), dest_dtype=dest.dtype))
        return dest


class _Watch(torch.utils._python_dispatch.TorchDispatchMode):
    """Sees every real op the loader runs during the dry run.  Ops that only make
    views are ignored; anything else that touches a region a source was already
    recorded into taints that source (see ``_Recorder.touch``)."""

    def __init__(self, rec: _Recorder):
        super().__init__()
        self.rec = rec

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if self.rec.written and not getattr(func, "is_view", False):
            for a in _leaves((args, kwargs)):
                if not isinstance(a, TracedSource):
                    self.rec.touch(a, str(func))
        return func(*args, **kwargs)


class _Unsupported(UnsupportedReshard):
    def __init__(self, src_name: str, what: str):
        super().__init__(f"{what}")
        self.src_name = src_name


class CaptureState:
    """What several ``capture_geometry`` calls over parts of one checkpoint share:
    the regions already recorded into, so that a loader in a later part that works
    on bytes an earlier part provides is still noticed."""

    def __init__(self, model: torch.nn.Module):
        self.recorder = _Recorder(model)
        self.reported: set = set()


def capture_geometry(model: torch.nn.Module, manifest: Iterable,
                     load_weights: Callable | None = None, device=None,
                     isolate: bool = False, state: CaptureState | None = None) -> CaptureResult:
    """Dry-run the model's weight loading and return every recorded copy.

    ``manifest`` lists ``(name, dtype, shape)`` for every full source tensor
    (the safetensors header has exactly this).  ``load_weights`` defaults to
    ``model.load_weights`` and must accept an iterable of ``(name, tensor)``.
    The model may be the live one: a recorded ``copy_`` moves nothing, while
    whatever else the loader does to a destination (zeroing vocabulary padding)
    happens for real, as it must.  ``device`` is the device the placeholders
    claim to live on (default: where the model's first parameter is), so a
    loader's ``.to(param.device)`` is the identity.  ``isolate`` feeds one
    source per ``load_weights`` call, as the reference does
    (geometry.py:282-293); by default one call takes them all and is resumed
    behind a source that fails.  ``state`` carries what earlier calls over other
    parts of the same checkpoint recorded; a source of an earlier call can then
    turn up in ``unsupported`` here, when a loader of this part touched its bytes."""
    loader = load_weights if load_weights is not None else model.load_weights
    if state is None:
        state = CaptureState(model)
    rec = state.recorder
    first_copy = len(rec.copies)
    if device is None:
        first = next(iter(model.parameters()), None)
        device = first.device if first is not None else torch.device("cpu")
    items = [(str(n), dt, tuple(int(s) for s in sh)) for n, dt, sh in manifest]
    result = CaptureResult()

    def feed(seq):
        for name, dtype, shape in seq:
            rec.current = name
            yield name, TracedSource.source(name, shape, dtype, device, rec)
        rec.current = None

    def failed(name: str, why: str):
        if name not in result.unsupported_reasons:
            result.unsupported.append(name)
        result.unsupported_reasons[name] = why
        rec.copies = [c for c in rec.copies if c.src_name != name]

    watch = _Watch(rec)
    if isolate:
        for item in items:
            try:
                with watch:
                    loader(feed([item]))
            except _Unsupported as e:
                failed(e.src_name, str(e))
    else:
        start = 0
        order = {name: i for i, (name, _d, _s) in enumerate(items)}
        while start < len(items):
            try:
                with watch:
                    loader(feed(items[start:]))
                break
            except _Unsupported as e:
                at = order.get(e.src_name, start)
                failed(e.src_name, str(e))
                # sources behind the failing one may have been fetched but not loaded
                later = {n for n, _d, _s in items[at + 1:]}
                rec.copies = [c for c in rec.copies if c.src_name not in later]
                start = max(at, start) + 1
    for name, why in rec.tainted.items():
        if name not in state.reported:
            state.reported.add(name)
            failed(name, why)
    mine = {n for n, _d, _s in items}
    result.copies = [c for c in rec.copies[first_copy:] if c.src_name in mine]
    rec.copies = rec.copies[:first_copy] + result.copies
    result.unattributed = rec.unattributed
    for why, count in summarize_unsupported(result.unsupported_reasons):
        logger.warning("capture: %d source(s) unsupported: %s", count, why)
    logger.info("capture: %d copies from %d sources, %d unsupported", len(result.copies),
                len(items), len(result.unsupported))
    return result
