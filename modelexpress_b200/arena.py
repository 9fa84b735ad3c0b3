"""Device arena on CUDA virtual memory management, and its crossing of process boundaries.

Mirrors the reference's ``VmmArena`` and its allocator hook (vmm/arena.py:155-350,
vmm/hook.py:111-200): one reserved address range, one physical block per ``malloc``, torch
routed into it through ``CUDAPluggableAllocator`` + ``MemPool`` inside ``use_arena``.  Where the
reference registers the range with its NIC once per load (``registered_range``,
arena.py:322-330), this arena is exported to NVLink peers on the same box: the blocks travel as
POSIX file descriptors over a unix socket and the importing process maps them at the same
offsets of a range of its own, so every tensor of the model is reachable there as
``imported.base + (address - arena.base)`` through one mapping.
"""

from __future__ import annotations

import array
import contextlib
import ctypes
import json
import os
import socket
import threading

from . import _lib
from ._lib import check

DEFAULT_RESERVE = 256 << 30   # address space only; memory is committed per malloc


class Arena:
    """``Arena(device)`` reserves; ``malloc`` / ``free`` / ``close`` as the reference's arena."""

    def __init__(self, device: int = 0, reserve_bytes: int = DEFAULT_RESERVE, _handle=None):
        self._lib = _lib.load()
        self.device = int(device)
        if _handle is None:
            h = ctypes.c_void_p()
            check(self._lib.mxb_arena_create(self.device, int(reserve_bytes), ctypes.byref(h)), "mxb_arena_create")
            self._h, self.imported = h, False
        else:
            self._h, self.imported = _handle, True

    # -- the reference's surface ------------------------------------------------
    def malloc(self, size: int) -> int:
        if size <= 0:
            raise ValueError("size must be positive")
        p = ctypes.c_uint64(0)
        check(self._lib.mxb_arena_malloc(self._h, int(size), ctypes.byref(p)), "mxb_arena_malloc")
        return int(p.value)

    def free(self, ptr: int) -> None:
        check(self._lib.mxb_arena_free(self._h, int(ptr)), "mxb_arena_free")

    def _range(self):
        b, u, s = ctypes.c_uint64(0), ctypes.c_uint64(0), ctypes.c_uint64(0)
        check(self._lib.mxb_arena_range(self._h, ctypes.byref(b), ctypes.byref(u), ctypes.byref(s)),
              "mxb_arena_range")
        return int(b.value), int(u.value), int(s.value)

    @property
    def base(self) -> int:
        return self._range()[0]

    @property
    def used_bytes(self) -> int:
        return self._range()[1]

    @property
    def total_bytes(self) -> int:
        return self._range()[2]

    def registered_range(self) -> tuple:
        """``(base, used)``: the range a peer has to map to see every allocation so far."""
        b, u, _s = self._range()
        return b, u

    def blocks(self) -> list:
        """Live blocks as ``(offset, size)``, in address order."""
        n = ctypes.c_uint64(0)
        self._lib.mxb_arena_blocks(self._h, None, 0, ctypes.byref(n))
        arr = (_lib.ArenaBlock * max(1, n.value))()
        check(self._lib.mxb_arena_blocks(self._h, arr, n.value, ctypes.byref(n)), "mxb_arena_blocks")
        return [(int(arr[i].offset), int(arr[i].size)) for i in range(n.value)]

    @property
    def live_allocation_count(self) -> int:
        return len(self.blocks())

    @property
    def mapped_bytes(self) -> int:
        return sum(s for _o, s in self.blocks())

    def contains(self, ptr: int, nbytes: int = 1) -> bool:
        b, u, _s = self._range()
        return b <= ptr and ptr + nbytes <= b + u

    def close(self) -> None:
        if getattr(self, "_h", None):
            if getattr(self, "_pool", None) is not None:
                # torch hands back what its pool still caches (through the free entry point)
                import torch

                self._pool = None
                torch.cuda.empty_cache()
            self._lib.mxb_arena_destroy(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- crossing a process boundary ---------------------------------------------
    def export_fds(self) -> tuple:
        """``(layout, fds)``: the layout as a JSON-able dict and one descriptor per live block
        (the caller closes them once sent)."""
        blocks = self.blocks()
        fds = []
        try:
            for off, _size in blocks:
                fd = ctypes.c_int32(-1)
                check(self._lib.mxb_arena_export_fd(self._h, off, ctypes.byref(fd)), "mxb_arena_export_fd")
                fds.append(int(fd.value))
        except Exception:
            for fd in fds:
                os.close(fd)
            raise
        _b, used, _s = self._range()
        return {"device": self.device, "span": used, "blocks": [list(b) for b in blocks]}, fds

    @classmethod
    def import_fds(cls, layout: dict, fds: list, device: int) -> "Arena":
        """Map another process's blocks for ``device``; the descriptors stay the caller's."""
        blocks = layout["blocks"]
        if len(blocks) != len(fds):
            raise ValueError("one descriptor per block is required")
        arr = (_lib.ArenaBlock * max(1, len(blocks)))()
        for i, (off, size) in enumerate(blocks):
            arr[i].offset, arr[i].size = int(off), int(size)
        cfds = (ctypes.c_int32 * max(1, len(fds)))(*[int(f) for f in fds])
        h = ctypes.c_void_p()
        check(_lib.load().mxb_arena_import(int(device), int(layout["span"]), arr, cfds, len(blocks),
                                           ctypes.byref(h)), "mxb_arena_import")
        return cls(device, _handle=h)


# ---------------------------------------------------------------------------
# descriptors over a unix socket (SCM_RIGHTS)
# ---------------------------------------------------------------------------

_FDS_PER_MESSAGE = 200   # below the kernel's limit of 253 descriptors per message


def send_arena(sock: socket.socket, arena: Arena) -> None:
    """The arena's layout and block descriptors to the peer at the other end of ``sock``."""
    layout, fds = arena.export_fds()
    try:
        head = json.dumps(layout).encode()
        sock.sendall(len(head).to_bytes(8, "little") + head)
        for i in range(0, len(fds), _FDS_PER_MESSAGE):
            part = fds[i: i + _FDS_PER_MESSAGE]
            sock.sendmsg([b"F"], [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", part))])
    finally:
        for fd in fds:
            os.close(fd)


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = b""
    while len(buf) < n:
        part = sock.recv(n - len(buf))
        if not part:
            raise ConnectionError("the peer closed the socket while sending its arena")
        buf += part
    return buf


def recv_arena(sock: socket.socket, device: int) -> Arena:
    """The peer's arena, mapped for ``device`` of this process."""
    n = int.from_bytes(_recv_exact(sock, 8), "little")
    layout = json.loads(_recv_exact(sock, n))
    want, fds = len(layout["blocks"]), []
    try:
        while len(fds) < want:
            size = array.array("i").itemsize * _FDS_PER_MESSAGE
            msg, anc, _flags, _addr = sock.recvmsg(1, socket.CMSG_SPACE(size))
            if not msg:
                raise ConnectionError("the peer closed the socket while sending descriptors")
            for level, kind, data in anc:
                if level == socket.SOL_SOCKET and kind == socket.SCM_RIGHTS:
                    got = array.array("i")
                    got.frombytes(data[: len(data) - len(data) % got.itemsize])
                    fds += list(got)
        return Arena.import_fds(layout, fds[:want], device)
    finally:
        for fd in fds:
            os.close(fd)


class ArenaServer:
    """Serves one arena on a unix socket path: every connection receives the current layout
    and descriptors (what a serving replica runs beside its manifest)."""

    def __init__(self, arena: Arena, path: str):
        self.arena, self.path = arena, path
        with contextlib.suppress(FileNotFoundError):
            os.unlink(path)
        self._sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        self._sock.bind(path)
        self._sock.listen(16)
        self._sock.settimeout(0.2)
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                conn, _ = self._sock.accept()
            except socket.timeout:
                continue
            except OSError:
                return
            with conn:
                try:
                    send_arena(conn, self.arena)
                except (OSError, _lib.MxbError):
                    pass      # a peer that hung up, or an arena closed under us: serve the next one

    def close(self) -> None:
        self._stop.set()
        self._thread.join(timeout=2)
        self._sock.close()
        with contextlib.suppress(FileNotFoundError):
            os.unlink(self.path)


def fetch_arena(path: str, device: int, timeout_s: float = 5.0) -> Arena:
    """Connect to an ``ArenaServer`` and map what it serves."""
    with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as s:
        s.settimeout(timeout_s)
        s.connect(path)
        return recv_arena(s, device)


# ---------------------------------------------------------------------------
# torch through the arena (vmm/hook.py:111-200)
# ---------------------------------------------------------------------------

_pool_lock = threading.Lock()
_allocator = None


def _mem_pool(arena: Arena, device: int):
    """One pluggable allocator per process (torch keeps a raw pointer to it) and one torch
    memory pool per arena: torch caches what it frees inside a pool, so a pool shared between
    arenas would hand a later arena's tensors the cached blocks of an earlier one."""
    global _allocator
    import torch
    from torch.cuda.memory import CUDAPluggableAllocator, MemPool

    with _pool_lock:
        if _allocator is None:
            _allocator = CUDAPluggableAllocator(_lib.LIB_PATH, "mxb_arena_torch_malloc", "mxb_arena_torch_free")
        if getattr(arena, "_pool", None) is None:
            with torch.cuda.device(device):
                arena._pool = MemPool(_allocator.allocator())
        return arena._pool


@contextlib.contextmanager
def use_arena(arena: Arena, device: int | None = None):
    """Tensors torch allocates on ``device`` inside the block come out of ``arena``
    (the reference's ``use_arena``, vmm/hook.py:164-200).  They must be gone, and torch's
    cache of the pool emptied, before the arena is closed."""
    import torch

    dev = arena.device if device is None else int(device)
    pool = _mem_pool(arena, dev)
    check(_lib.load().mxb_arena_set_default(dev, arena._h), "mxb_arena_set_default")
    try:
        with torch.cuda.use_mem_pool(pool, device=torch.device("cuda", dev)):
            yield arena
    finally:
        _lib.load().mxb_arena_set_default(dev, None)


# ---------------------------------------------------------------------------
# the arenas of this process that peers may map
# ---------------------------------------------------------------------------

_published: dict = {}   # socket path -> (Arena, ArenaServer)
_by_device: dict = {}   # device -> socket path of the arena the last load on it filled


def publish_arena(arena: Arena, socket_path: str) -> str:
    """Serve ``arena`` on ``socket_path``; manifests and requests written by this process from
    now on name tensors inside it by that path and their offset (``lookup``)."""
    with _pool_lock:
        if socket_path in _published:
            return socket_path
        _published[socket_path] = (arena, ArenaServer(arena, socket_path))
    return socket_path


def withdraw_arena(socket_path: str) -> None:
    with _pool_lock:
        entry = _published.pop(socket_path, None)
    if entry is not None:
        entry[1].close()


def lookup(ptr: int, nbytes: int):
    """``(socket path, offset)`` when ``[ptr, ptr + nbytes)`` lies in a published arena."""
    with _pool_lock:
        items = list(_published.items())
    for path, (arena, _server) in items:
        if arena._h and arena.contains(ptr, max(1, nbytes)):
            return path, ptr - arena.base
    return None


def _env_on() -> bool:
    return (os.environ.get("MXB_VMM_ARENA") or os.environ.get("MX_VMM_ARENA") or "0") == "1"


@contextlib.contextmanager
def maybe_enter_arena(device: int, socket_dir: str | None = None):
    """With ``MXB_VMM_ARENA=1`` (or the reference's ``MX_VMM_ARENA=1``): what the engine
    allocates inside the block comes out of a fresh arena, which is published for peers once the
    block has completed (the load envelope of vmm/runtime.py:40-135: a failed body closes the
    arena; a second load on the device replaces the first arena, whose tensors must be gone).
    Otherwise a no-op.  Yields the arena or ``None``."""
    if not _env_on():
        yield None
        return
    import logging
    import tempfile

    log = logging.getLogger(__name__)
    arena = Arena(int(device))
    try:
        with use_arena(arena, int(device)):
            yield arena
    except BaseException:
        arena.close()
        raise
    prior = _by_device.pop(int(device), None)
    if prior is not None:
        log.warning("device %d: a second load replaces the arena of the first; its tensors must be gone", device)
        old = _published.get(prior)
        withdraw_arena(prior)
        if old is not None:
            old[0].close()
    path = os.path.join(socket_dir or tempfile.gettempdir(), f"mxb-arena-{os.getpid()}-{int(device)}.sock")
    _by_device[int(device)] = publish_arena(arena, path)
    log.info("device %d: arena published at %s (%d blocks, %d bytes mapped)", device, path,
             arena.live_allocation_count, arena.mapped_bytes)
