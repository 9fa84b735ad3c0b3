"""Strict verification of received weights against published shard digests.

Mirrors the receiving half of the reference's digest scheme: a publisher
attaches ``tensor_digest`` of each shard it owns to the shard table
(refit/reshard/verify.py:186-196, rendezvous.py:99-115), and the strict staged
transfer recomputes the digest of the same box out of the assembled tensor and
refuses the update on a mismatch
(modelexpress_rl/inference/nixl_staged_transfer.py:529-549).  Here every box of
every source is digested in ONE kernel launch instead of one reduction chain
plus several ``.item()`` syncs per shard.
"""

from __future__ import annotations

from .digest import digest_many
from .runtime import DIGEST_ROWS


def shard_region(full_tensor, global_shape, shard_offset, shape):
    """The sub-box of an assembled source that one publisher owns, as a
    contiguous copy (refit/reshard/verify.py:158-183, same rank check)."""
    if not len(global_shape) == len(shard_offset) == len(shape):
        raise ValueError(
            f"rank mismatch: global_shape {tuple(global_shape)}, shard_offset "
            f"{tuple(shard_offset)} and shape {tuple(shape)} must have equal rank")
    view = full_tensor.reshape(tuple(global_shape))
    for axis, (start, extent) in enumerate(zip(shard_offset, shape)):
        view = view.narrow(axis, int(start), int(extent))
    return view.contiguous()


def published_digests(shards: dict, ctx=None) -> dict:
    """{key: tensor} -> {key: tensor_digest hex}: what a publisher attaches."""
    keys = list(shards)
    res = digest_many([shards[k] for k in keys], DIGEST_ROWS, ctx)
    return {k: r["tensor_digest"] for k, r in zip(keys, res)}


def verify_sources(assembled: dict, sources: dict, ctx=None) -> int:
    """Check every published shard digest against the assembled tensors.

    ``assembled[name]`` is the full source tensor as received; ``sources[name]``
    has ``global_shape`` and ``shards`` (each with ``shard_offset``, ``shape``,
    ``digest``).  Raises ``RuntimeError`` with the reference's messages when a
    digest is missing or differs; returns the number of shards verified."""
    regions, labels = [], []
    for name, source in sources.items():
        tensor = assembled[name]
        for shard in source.shards:
            if not shard.digest:
                raise RuntimeError(f"source {name!r} did not publish a verification digest")
            regions.append(shard_region(tensor, source.global_shape, shard.shard_offset, shard.shape))
            labels.append((name, tuple(shard.shard_offset), shard.digest))
    if not regions:
        return 0
    res = digest_many(regions, DIGEST_ROWS, ctx)
    for (name, offset, want), r in zip(labels, res):
        if r["tensor_digest"] != want:
            raise RuntimeError(f"staged weight digest mismatch for source {name!r} at offset {offset}")
    return len(regions)
