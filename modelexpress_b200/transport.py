"""The mover plugin: ``Transport.read(descriptors)`` executed by the scatter kernel.

Mirrors refit/reshard/transport/base.py of the reference: ``ReadDescriptor``
has the same fields, ``MxbTransport`` has the same ``read`` contract as
``InMemoryReferenceTransport`` (synchronous: on return the bytes are visible;
``session`` is informative because addresses are absolute) and keeps the same
``bytes_moved`` / ``reads_issued`` counters.  Source and destination addresses
must be reachable from the transport's device: local HBM, a peer GPU's HBM
mapped into this process, or pinned host memory.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Protocol, runtime_checkable

import numpy as np

from .runtime import Context, default_context


@dataclass
class ReadDescriptor:
    """One remote->local READ: copy ``nbytes`` from ``session``'s ``src_addr`` to
    the local ``dst_addr`` (both absolute)."""

    session: str
    src_addr: int
    dst_addr: int
    nbytes: int


@runtime_checkable
class Transport(Protocol):
    def read(self, descriptors: list) -> None: ...


class MxbTransport:
    """``Transport`` whose moves run as one persistent scatter launch on a B200.

    The run list is folded into 2-D records on the host (a row-parallel slice of
    4096 one-KiB runs becomes one record) and moved by the sm_100a kernel.
    The launch runs on the library's own stream and ``read`` returns after it has
    finished; work the caller queued earlier on another stream for the same
    buffers must have completed (synchronise that stream first).
    Raises ``MxbError`` (``RuntimeError``) on a CUDA failure and ``MxbTimeout``
    (``TimeoutError``) when a device-side wait ran out; unknown sessions raise
    ``KeyError`` when a session table was given, as the NIXL transport does.
    """

    def __init__(self, ctx: Context | None = None, device: int | None = None,
                 sessions: dict | None = None) -> None:
        self._ctx = ctx
        self._device = device
        self._sessions = sessions
        self.bytes_moved = 0
        self.reads_issued = 0

    @property
    def ctx(self) -> Context:
        if self._ctx is None:
            self._ctx = default_context(self._device or 0)
        return self._ctx

    def read(self, descriptors: list) -> None:
        live = [d for d in descriptors if d.nbytes]
        if self._sessions is not None:
            for d in live:
                if d.session not in self._sessions:
                    raise KeyError(d.session)
        if not live:
            return
        runs = np.empty((len(live), 3), dtype=np.uint64)
        for i, d in enumerate(live):
            runs[i, 0], runs[i, 1], runs[i, 2] = d.src_addr, d.dst_addr, d.nbytes
        self.ctx.read_runs(runs, self._device)
        self.bytes_moved += int(runs[:, 2].sum())
        self.reads_issued += len(live)
