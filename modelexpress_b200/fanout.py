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


class Broadcast:
    """One process driving every GPU of the broadcast (tests, single-process
    servers).  ``spans[g]`` lists GPU g's (ptr, nbytes) ranges, same sizes on
    every GPU."""

    def __init__(self, ctx: Context, devices: list, spans: list, chunk_bytes: int,
                 kind: str = "chain", root_index: int = 0):
        self.devices = devices
        self.root = root_index
        self.children = topology(kind, len(devices), root_index)
        self.nodes = [Fanout(ctx, dev, spans[i], chunk_bytes) for i, dev in enumerate(devices)]
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
