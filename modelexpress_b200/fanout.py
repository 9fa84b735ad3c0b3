"""Serving-peer fan-out: weights resident on one GPU pushed to the box's others.

The reference's warm start pulls every tensor from a serving peer through NIXL
(load_strategy/rdma_strategy.py:467-610 -> nixl_transfer.py:769-952): manifests
are matched by name, size and dtype, then one RDMA READ per tensor is posted.
On one NVSwitch box the same transfer is a chunked, pipelined broadcast whose
hops are P2P stores: ``topology`` gives each GPU a parent and children, every
GPU runs one fan-out kernel, and chunks flow down the chain or tree as soon as
they arrive.

``match_manifests`` applies the reference's matching rule
(nixl_transfer.py:835-850); ``Broadcast`` wires up the nodes when one process
drives several GPUs; with one process per GPU the ranks exchange IPC handles
and call the same node API themselves.
"""

from __future__ import annotations

from dataclasses import dataclass

from .runtime import Context, Fanout


class ManifestMismatchError(RuntimeError):
    """types.py:40-47 of the reference: source and target disagree on a tensor."""


@dataclass
class TensorDescriptor:
    """p2p.proto:127-142: one manifest row."""

    name: str
    addr: int
    size: int
    device_id: int
    dtype: str


def match_manifests(source: list, target: list) -> list:
    """[(name, src_addr, dst_addr, size)] for every target tensor, matched by
    name; a size or dtype difference raises ``ManifestMismatchError``; target
    tensors the source lacks are reported the same way (a partial copy would
    leave random weights behind)."""
    by_name = {d.name: d for d in source}
    out, missing = [], []
    for t in target:
        s = by_name.get(t.name)
        if s is None:
            missing.append(t.name)
            continue
        if s.size != t.size or s.dtype != t.dtype:
            raise ManifestMismatchError(
                f"{t.name}: source {s.size} B {s.dtype} != target {t.size} B {t.dtype}")
        out.append((t.name, s.addr, t.addr, t.size))
    if missing:
        raise ManifestMismatchError(f"source lacks {len(missing)} tensor(s): {missing[:5]}")
    return out


def topology(kind: str, n: int, root: int = 0) -> list:
    """children[i] for every GPU i of an n-GPU broadcast rooted at ``root``:
    ``chain`` (root -> next -> ...), ``tree`` (binary), ``flat`` (root stores
    to everyone)."""
    order = [root] + [g for g in range(n) if g != root]
    children = [[] for _ in range(n)]
    if kind == "chain":
        for a, b in zip(order, order[1:]):
            children[a].append(b)
    elif kind == "tree":
        for i, g in enumerate(order):
            for j in (2 * i + 1, 2 * i + 2):
                if j < n:
                    children[g].append(order[j])
    elif kind == "flat":
        children[root] = order[1:]
    else:
        raise ValueError(f"unknown topology {kind!r}")
    return children


def plan_pieces(sizes, chunk_bytes: int, piece_bytes: int = 65536) -> tuple:
    """Host only (``mxb_fanout_plan_pieces``): how ranges of the given sizes are cut into pieces
    (of at most ``piece_bytes``) and chunks.  Returns ``(pieces, chunk_pieces)``: ``pieces`` is a list of
    ``(range, offset, nbytes, chunk)``, ``chunk_pieces[c]`` what a child's arrival
    counter ``c`` reaches per broadcast."""
    import ctypes

    from . import _lib

    lib = _lib.load()
    spans, n = _lib.span_array([(4096, int(s)) for s in sizes])
    np_, nc = ctypes.c_uint64(), ctypes.c_uint64()
    rc = lib.mxb_fanout_plan_pieces(spans, n, int(chunk_bytes), int(piece_bytes), None, 0, ctypes.byref(np_),
                                    None, 0, ctypes.byref(nc))
    if rc not in (0, -7):
        _lib.check(rc, "mxb_fanout_plan")
    pieces = (_lib.FanoutPiece * max(1, np_.value))()
    per_chunk = (ctypes.c_uint32 * max(1, nc.value))()
    _lib.check(lib.mxb_fanout_plan_pieces(spans, n, int(chunk_bytes), int(piece_bytes), pieces, np_.value,
                                          ctypes.byref(np_), per_chunk, nc.value, ctypes.byref(nc)),
               "mxb_fanout_plan")
    return ([(int(p.range), int(p.offset), int(p.nbytes), int(p.chunk)) for p in pieces[: np_.value]],
            [int(x) for x in per_chunk[: nc.value]])


class Broadcast:
    """One process driving every GPU of the broadcast (tests, single-process
    servers).  ``spans[g]`` lists GPU g's (ptr, nbytes) ranges, same sizes on
    every GPU."""

    def __init__(self, ctx: Context, devices: list, spans: list, chunk_bytes: int,
                 kind: str = "chain", root_index: int = 0, engine: str | None = None,
                 piece_bytes: int = 65536):
        self.devices = devices
        self.root = root_index
        self.children = topology(kind, len(devices), root_index)
        self.nodes = [Fanout(ctx, dev, spans[i], chunk_bytes, piece_bytes) for i, dev in enumerate(devices)]
        if engine is not None:
            for node in self.nodes:
                node.set_engine(engine)
        for i, kids in enumerate(self.children):
            for k in kids:
                self.nodes[i].add_child(spans[k], self.nodes[k].counters)

    def run(self, timeout_ms: int = 5000) -> list:
        """Launch every node (leaves first, so no node waits for a launch that
        has not been queued), wait, return per-GPU device milliseconds."""
        order = [i for i in range(len(self.nodes)) if i != self.root] + [self.root]
        for i in order:
            self.nodes[i].run(i == self.root, timeout_ms)
        return [node.wait() for node in self.nodes]

    def close(self):
        for n in self.nodes:
            n.close()


def manifest_from_module(model, device_id: int | None = None) -> list:
    """Manifest rows for every CUDA tensor of a module tree, with the reference's
    rules (tensor_utils.py:299-360): parameters then buffers; contiguous tensors
    as they are, non-contiguous ones as the flat bytes of their whole storage
    under ``name.__storage``; tensors sharing a ``data_ptr`` listed once (tied
    weights); zero-element tensors keep their name and skip the de-duplication."""
    import torch

    rows, seen = [], set()
    named = list(model.named_parameters()) + list(model.named_buffers())
    for name, tensor in named:
        t = tensor.data if hasattr(tensor, "data") else tensor
        if not t.is_cuda:
            continue
        dev = t.device.index if device_id is None else device_id
        if t.numel() == 0:
            rows.append(TensorDescriptor(name, 0, 0, dev, str(t.dtype)))
            continue
        if t.is_contiguous():
            ptr, size, nm, dt = t.data_ptr(), t.numel() * t.element_size(), name, str(t.dtype)
        else:
            sv = torch.empty(0, dtype=torch.uint8, device=t.device).set_(t.untyped_storage())
            ptr, size, nm, dt = sv.data_ptr(), sv.numel(), f"{name}.__storage", "torch.uint8"
        if ptr in seen:
            continue
        seen.add(ptr)
        rows.append(TensorDescriptor(nm, ptr, size, dev, dt))
    return rows


# ---------------------------------------------------------------------------
# The strategy seam: a serving peer publishes, a starting replica receives
# ---------------------------------------------------------------------------
#
# The reference's warm start (load_strategy/rdma_strategy.py:142-257, 467-610): find
# READY sources, fetch the source worker's tensor manifest (p2p.proto:127-142, served by
# metadata/worker_server.py:101-121), match it against the target's own tensors by name,
# size and dtype (nixl_transfer.py:835-850), move the bytes, try the next of at most three
# candidates when a transfer fails, re-initialise the model first if the failed transfer
# may have written into it.  Here the manifest travels as a JSON file in a rendezvous
# directory (the gRPC service stays with the control plane), memory is reached through
# CUDA IPC handles, the source pushes with the fan-out kernel and the target's own kernel
# waits, with a bound, for the chunks to arrive.

import json
import os
import time
import uuid

MAX_SOURCE_RETRIES = 3   # rdma_strategy.py:39


def _tensor_rows(tensors: dict, device_id: int) -> list:
    """Manifest rows of named contiguous CUDA tensors (tied tensors once)."""
    rows, seen = [], set()
    for name, t in tensors.items():
        t = t.data if hasattr(t, "data") else t
        if not t.is_cuda or not t.is_contiguous():
            continue
        size = t.numel() * t.element_size()
        if size and t.data_ptr() in seen:
            continue
        seen.add(t.data_ptr())
        rows.append(TensorDescriptor(name, t.data_ptr() if size else 0, size, device_id, str(t.dtype)))
    return rows


def _export_rows(rows: list) -> list:
    """JSON-able manifest: every row with the way a peer reaches it: the socket of the
    published arena it lies in and its offset there (one mapping for all such rows), else the
    CUDA IPC handle of its allocation and its offset inside that allocation."""
    from . import arena as arena_mod
    from .runtime import ipc_export

    out = []
    for d in rows:
        row = {"name": d.name, "size": d.size, "device_id": d.device_id, "dtype": d.dtype,
               "handle": "", "offset": 0}
        hit = arena_mod.lookup(d.addr, d.size) if d.size else None
        if hit is not None:
            row["arena"], row["offset"] = hit
        elif d.size:
            handle, row["offset"] = ipc_export(d.addr)
            row["handle"] = handle.hex()
        out.append(row)
    return out


class _PeerMemory:
    """A peer's memory as mapped by this process: one IPC mapping per allocation, however many
    tensors lie in it, or one imported arena per socket, however many allocations it holds."""

    def __init__(self, device: int = 0):
        self.device = int(device)
        self._base: dict = {}
        self._arenas: dict = {}

    def address(self, handle_hex: str, offset: int, arena: str | None = None, nbytes: int = 1) -> int:
        if arena:
            return self._arena_address(arena, int(offset), int(nbytes))
        from .runtime import ipc_open

        base = self._base.get(handle_hex)
        if base is None:
            base = self._base[handle_hex] = ipc_open(bytes.fromhex(handle_hex), 0)
        return base + int(offset)

    def row_address(self, row: dict) -> int:
        return self.address(row.get("handle", ""), row["offset"], row.get("arena"), int(row.get("size", 1)) or 1)

    def _arena_address(self, path: str, offset: int, nbytes: int) -> int:
        from .arena import fetch_arena

        mapped = self._arenas.get(path)
        if mapped is not None and offset + nbytes > mapped.used_bytes:
            mapped.close()        # the peer's arena has grown since it was mapped
            mapped = None
        if mapped is None:
            mapped = self._arenas[path] = fetch_arena(path, self.device)
        if offset + nbytes > mapped.used_bytes:
            raise ManifestMismatchError(f"offset {offset} + {nbytes} lies outside the arena served at {path}")
        return mapped.base + offset

    def close(self) -> None:
        from . import _lib

        lib = _lib.load()
        for base in self._base.values():
            lib.mxb_ipc_close(int(base), 0)
        self._base = {}
        for mapped in self._arenas.values():
            mapped.close()
        self._arenas = {}


def _write_json(path: str, obj) -> None:
    tmp = f"{path}.{uuid.uuid4().hex}.tmp"
    with open(tmp, "w") as f:
        json.dump(obj, f)
    os.replace(tmp, path)       # readers never see a half-written file


class FanoutSource:
    """The serving side: publishes its tensors as a manifest and pushes them to the
    replicas that ask (``serve``).  ``tensors`` is ``{name: CUDA tensor}``."""

    def __init__(self, tensors: dict, rendezvous_dir: str, source_id: str, ctx: Context | None = None,
                 device: int | None = None, chunk_bytes: int = 256 << 10, digests: bool = True,
                 piece_bytes: int = 256 << 10, engine: str | None = "dma"):
        import torch

        from .runtime import default_context

        self.dev = torch.cuda.current_device() if device is None else int(device)
        self.ctx = ctx if ctx is not None else default_context(self.dev)
        self.dir, self.id, self.chunk_bytes = rendezvous_dir, source_id, int(chunk_bytes)
        # a push is one hop: larger pieces (fewer system-scope fences per byte) are faster there,
        # and the copy engines faster still ("dma"; None: the library's default, the store kernel,
        # or what MXB_FANOUT_ENGINE names)
        self.piece_bytes = min(int(piece_bytes), int(chunk_bytes))
        self.engine = None if os.environ.get("MXB_FANOUT_ENGINE") else engine
        self.rows = _tensor_rows(tensors, self.dev)
        self._keep = tensors
        self._digests = None
        if digests:
            from .runtime import DIGEST_ROWS, DIGEST_SAFE32

            recs = self.ctx.digest([(d.addr, d.size) for d in self.rows], DIGEST_SAFE32 | DIGEST_ROWS, self.dev)
            self._digests = [[int(r.safe_checksum), int(r.row_sum), int(r.row_sum_w), int(r.tail_sum),
                              int(r.tail_sum_w), int(r.ragged_sum)] for r in recs]
        self._peers = _PeerMemory(self.dev)

    @property
    def manifest_path(self) -> str:
        return os.path.join(self.dir, f"{self.id}.manifest.json")

    def publish(self) -> str:
        """Write the manifest; from now on targets can find this source."""
        import torch

        torch.cuda.synchronize(self.dev)
        rows = _export_rows(self.rows)
        if self._digests is not None:
            for r, d in zip(rows, self._digests):
                r["digest"] = d
        _write_json(self.manifest_path, {"source_id": self.id, "status": "READY", "device_id": self.dev,
                                         "chunk_bytes": self.chunk_bytes, "piece_bytes": self.piece_bytes,
                                         "tensors": rows})
        return self.manifest_path

    def withdraw(self) -> None:
        try:
            os.remove(self.manifest_path)
        except FileNotFoundError:
            pass

    def pending_requests(self) -> list:
        pre, suf = f"{self.id}.request.", ".json"
        return sorted(os.path.join(self.dir, f) for f in os.listdir(self.dir)
                      if f.startswith(pre) and f.endswith(suf))

    def serve(self, timeout_s: float = 10.0, max_requests: int = 1, poll_s: float = 0.002) -> int:
        """Answer up to ``max_requests`` requests (one push each); returns how many were served."""
        served, t0 = 0, time.perf_counter()
        while served < max_requests and time.perf_counter() - t0 < timeout_s:
            reqs = self.pending_requests()
            if not reqs:
                time.sleep(poll_s)
                continue
            for path in reqs[: max_requests - served]:
                with open(path) as f:
                    req = json.load(f)
                os.remove(path)
                self.push(req)
                served += 1
        return served

    def push(self, req: dict) -> None:
        """One push: the requested tensors into the target's memory, chunk counters raised
        as each chunk completes; then the ``done`` marker the request names."""
        by_name = {d.name: d for d in self.rows}
        local, child = [], []
        for row in req["tensors"]:
            d = by_name[row["name"]]
            if not d.size:
                continue
            local.append((d.addr, d.size))
            child.append((self._peers.row_address(row), d.size))
        counters = self._peers.address(req["counters"]["handle"], req["counters"]["offset"])
        node = self.ctx.fanout(local, int(req["chunk_bytes"]), self.dev, int(req.get("piece_bytes", 65536)))
        try:
            if self.engine:
                node.set_engine(self.engine)
            node.add_child(child, counters)
            node.run(True, int(req.get("timeout_ms", 5000)))
            ms = node.wait()
        finally:
            node.close()
        _write_json(req["done"], {"device_ms": ms, "bytes": sum(n for _p, n in local)})

    def close(self) -> None:
        self.withdraw()
        self._peers.close()


class B200FanoutStrategy:
    """Load strategy: receive the weights from a serving peer on the same box.

    First in the chain, ahead of the strategies that read the checkpoint
    (load_strategy/__init__.py:71-78 puts the RDMA strategy there).  No manifest in
    the rendezvous directory, a manifest that does not match, a source that is not
    READY: ``StrategyFailed(mutated=False)``.  A push that does not arrive within
    the timeout, or arrives with other bytes than the source published:
    ``StrategyFailed(mutated=True)`` after the next of at most three candidates has
    been tried (the adapter's ``reinit_for_retry`` is called in between when it has
    one, as rdma_strategy.py:209-247 does)."""

    name = "b200_fanout"
    requires: tuple = ()

    def __init__(self, rendezvous_dir: str | None = None, timeout_ms: int = 5000,
                 wait_for_push: bool | None = None):
        self.dir = rendezvous_dir
        self.timeout_ms = int(timeout_ms)
        # True: launch the receiving kernel only after the source reported its push done
        # (needed when source and target share one GPU: kernels that wait on each other
        # must not depend on being scheduled together); None: MXB_FANOUT_WAIT_FOR_PUSH
        self.wait_for_push = wait_for_push
        self.last: dict = {}

    def _dir(self, ctx) -> str | None:
        return self.dir or getattr(ctx, "fanout_dir", None) or os.environ.get("MXB_FANOUT_DIR")

    def is_available(self, ctx) -> bool:
        d = self._dir(ctx)
        try:
            import torch

            from . import _lib

            _lib.load()
            return bool(d) and os.path.isdir(d) and bool(torch.cuda.is_available())
        except Exception:
            return False

    def candidates(self, ctx) -> list:
        d = self._dir(ctx)
        if not d or not os.path.isdir(d):
            return []
        found = []
        for f in sorted(os.listdir(d)):
            if not f.endswith(".manifest.json"):
                continue
            try:
                with open(os.path.join(d, f)) as fh:
                    m = json.load(fh)
            except (OSError, ValueError):
                continue
            if m.get("status") == "READY":
                found.append(m)
        return found

    def rollback(self, ctx) -> None:
        pass

    def load(self, result, ctx):
        from .loader import StrategyFailed

        sources = self.candidates(ctx)
        if not sources:
            raise StrategyFailed("no serving peer has published a manifest", mutated=False)
        dests = (ctx.adapter.named_destinations(result)
                 if getattr(ctx, "adapter", None) is not None and hasattr(ctx.adapter, "named_destinations")
                 else {n: p.data for n, p in result.model.named_parameters()})
        mutated = False
        errors = []
        for attempt, manifest in enumerate(sources[:MAX_SOURCE_RETRIES]):
            try:
                self.last = self._receive(manifest, dests, ctx)
                result.metadata[self.name] = self.last
                return result
            except StrategyFailed as e:
                errors.append(f"{manifest.get('source_id')}: {e}")
                if e.mutated:
                    mutated = True
                    reinit = getattr(getattr(ctx, "adapter", None), "reinit_for_retry", None)
                    if reinit is not None and attempt + 1 < min(len(sources), MAX_SOURCE_RETRIES):
                        try:
                            result = reinit(result)
                            dests = ctx.adapter.named_destinations(result)
                        except Exception as reinit_error:
                            raise StrategyFailed(f"failed to reinitialize the target after source "
                                                 f"{manifest.get('source_id')} failed: {reinit_error}",
                                                 mutated=True) from reinit_error
        raise StrategyFailed("; ".join(errors), mutated=mutated)

    def _receive(self, manifest: dict, dests: dict, ctx) -> dict:
        import torch

        from ._lib import MxbTimeout
        from .loader import StrategyFailed
        from .runtime import DIGEST_ROWS, DIGEST_SAFE32, default_context

        dev = int(getattr(ctx, "device_id", torch.cuda.current_device()))
        mx = default_context(dev)
        source = [TensorDescriptor(r["name"], 0, int(r["size"]), int(r["device_id"]), r["dtype"])
                  for r in manifest["tensors"]]
        target = _tensor_rows(dests, dev)
        try:
            matched = match_manifests(source, target)
        except ManifestMismatchError as e:
            raise StrategyFailed(str(e), mutated=False) from e
        want = {r["name"]: r.get("digest") for r in manifest["tensors"]}
        rows = [d for d in target if d.size]
        spans = [(d.addr, d.size) for d in rows]
        chunk = int(manifest.get("chunk_bytes", 1 << 20))
        piece = int(manifest.get("piece_bytes", 65536))
        torch.cuda.synchronize(dev)
        node = mx.fanout(spans, chunk, dev, piece)
        d = self._dir(ctx)
        req_id = uuid.uuid4().hex
        done = os.path.join(d, f"{manifest['source_id']}.done.{req_id}.json")
        try:
            from .runtime import ipc_export

            ch, coff = ipc_export(node.counters)
            request = {"chunk_bytes": chunk, "piece_bytes": piece, "timeout_ms": self.timeout_ms, "done": done,
                       "counters": {"handle": ch.hex(), "offset": coff},
                       "tensors": [r for r in _export_rows(rows)]}
            request_path = os.path.join(d, f"{manifest['source_id']}.request.{req_id}.json")
            _write_json(request_path, request)
            t0 = time.perf_counter()
            wait_first = self.wait_for_push
            if wait_first is None:
                wait_first = os.environ.get("MXB_FANOUT_WAIT_FOR_PUSH") == "1"
            if wait_first:
                while not os.path.exists(done):
                    if (time.perf_counter() - t0) * 1e3 > self.timeout_ms:
                        # nothing of ours is in flight and nothing was written: an expected miss
                        raise StrategyFailed(f"source {manifest['source_id']} did not push within "
                                             f"{self.timeout_ms} ms", mutated=False)
                    time.sleep(0.001)
            try:
                node.run(False, self.timeout_ms)    # waits (bounded, on the device) for every chunk
                ms = node.wait()
            except MxbTimeout as e:
                # some chunks may have landed: the parameters are no longer what they were
                raise StrategyFailed(f"push from {manifest['source_id']} did not complete: {e}",
                                     mutated=True) from e
            seconds = time.perf_counter() - t0
        finally:
            node.close()
            # a request nobody picked up must not be answered after this call has given up
            for leftover in (done, locals().get("request_path")):
                try:
                    if leftover:
                        os.remove(leftover)
                except FileNotFoundError:
                    pass
        if any(v is not None for v in want.values()):
            recs = mx.digest(spans, DIGEST_SAFE32 | DIGEST_ROWS, dev)
            for drow, r in zip(rows, recs):
                have = [int(r.safe_checksum), int(r.row_sum), int(r.row_sum_w), int(r.tail_sum),
                        int(r.tail_sum_w), int(r.ragged_sum)]
                if want.get(drow.name) is not None and have != want[drow.name]:
                    raise StrategyFailed(f"{drow.name}: received bytes differ from what "
                                         f"{manifest['source_id']} published", mutated=True)
        nbytes = sum(n for _p, n in spans)
        return {"source_id": manifest["source_id"], "tensors": len(matched), "bytes": nbytes,
                "seconds": seconds, "device_ms": ms, "gbps": nbytes / seconds / 1e9 if seconds else 0.0}
