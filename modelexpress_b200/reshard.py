"""RL-refit reshard: flat FSDP shards on every GPU -> inference TP layout.

The reference does this as a pull (refit/reshard/receiver.py:759-1043): each
inference rank plans byte runs against every trainer's shard table
(slice_plan.py:297-339), reads them through NIXL, re-slices full-pulled sources
with ``_foreach_copy_`` and lets the engine loader fuse q/k/v and gate/up.
Here every *source* rank pushes: one persistent scatter launch per GPU stores
its pieces of every destination parameter straight into the owning GPU's HBM
over NVLink (peer stores), already at their fused qkv_proj / gate_up_proj
offsets, so there is no staging buffer and no second pass.  The plan is a pure
function of (parameter shapes, world size, TP size).

Input layout: every parameter flattened and cut into ``world`` equal contiguous
pieces, piece ``s`` on rank ``s`` (what FSDP holds;
modelexpress_rl/train/engines/fsdp/publisher.py:71-147 publishes those boxes).
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .layout import CheckpointPlan, plan_checkpoint
from .safetensors_index import SAFETENSORS_DTYPES

ARENA_ALIGN = 256


def _align(v: int, a: int = ARENA_ALIGN) -> int:
    return (v + a - 1) // a * a


@dataclass
class ArenaLayout:
    """Offsets of named buffers inside one contiguous device arena."""

    offsets: dict
    sizes: dict
    total: int


def shard_arena(index: dict, world: int) -> ArenaLayout:
    """Arena holding one rank's flat FSDP piece of every parameter."""
    offsets, sizes, pos = {}, {}, 0
    for name, info in index.items():
        n = SAFETENSORS_DTYPES[info["dtype"]][0]
        for s in info["shape"]:
            n *= int(s)
        if n % world:
            raise ValueError(f"{name}: {n} bytes do not split {world} ways")
        offsets[name], sizes[name] = pos, n // world
        pos = _align(pos + n // world)
    return ArenaLayout(offsets, sizes, pos)


def param_arena(plan: CheckpointPlan) -> ArenaLayout:
    """Arena holding one inference rank's parameters (same on every rank)."""
    offsets, sizes, pos = {}, {}, 0
    for name, spec in plan.params.items():
        offsets[name], sizes[name] = pos, spec.nbytes
        pos = _align(pos + spec.nbytes)
    return ArenaLayout(offsets, sizes, pos)


def clip_records(so: int, do: int, rows: int, rb: int, sp: int, dp: int, lo: int, hi: int,
                 src_base: int, dst_base: int) -> list:
    """The part of a strided region (row r = source bytes [so + r*sp, +rb)) that
    lies in the source byte range [lo, hi), as records whose source address is
    ``src_base + (byte - lo)`` and whose destination keeps the region's layout."""
    if rows == 1:
        a, b = max(so, lo), min(so + rb, hi)
        if a >= b:
            return []
        n = b - a
        return [(src_base + a - lo, dst_base + do + (a - so), 1, n, n, n)]
    r_lo = max(0, (lo - so - rb) // sp + 1)
    r_hi = min(rows - 1, -((so - hi) // sp) - 1)  # ceil((hi - so) / sp) - 1
    out = []
    if r_lo > r_hi:
        return out
    first_full, last_full = r_lo, r_hi
    start = so + r_lo * sp
    if start < lo:  # first row clipped at its head
        a, b = lo, min(start + rb, hi)
        out.append((src_base, dst_base + do + r_lo * dp + (a - start), 1, b - a, b - a, b - a))
        first_full = r_lo + 1
    start = so + r_hi * sp
    tail = None
    if start + rb > hi and r_hi >= first_full:  # last row clipped at its end
        a, b = start, hi
        tail = (src_base + a - lo, dst_base + do + r_hi * dp, 1, b - a, b - a, b - a)
        last_full = r_hi - 1
    if last_full >= first_full:
        n = last_full - first_full + 1
        s0 = so + first_full * sp
        out.append((src_base + s0 - lo, dst_base + do + first_full * dp, n, rb,
                    sp if n > 1 else rb, dp if n > 1 else rb))
    if tail:
        out.append(tail)
    return out


def split_record(rec, max_bytes: int = 8 << 20) -> list:
    """Cut a record into pieces of at most ``max_bytes`` (whole rows, or 256-byte
    multiples of one long row) so that the merge below can interleave finely."""
    src, dst, rows, rb, sp, dp = (int(x) for x in rec)
    if rows * rb <= max_bytes:
        return [rec]
    out = []
    if rows == 1:
        step = max(256, max_bytes // 256 * 256)
        for off in range(0, rb, step):
            n = min(step, rb - off)
            out.append((src + off, dst + off, 1, n, n, n))
    else:
        per = max(1, max_bytes // rb)
        for r0 in range(0, rows, per):
            n = min(per, rows - r0)
            out.append((src + r0 * sp, dst + r0 * dp, n, rb, sp if n > 1 else rb, dp if n > 1 else rb))
    return out


def plan_reshard(index: dict, world: int, tp_size: int, src_rank: int, shard_base: int,
                 param_bases: list, family: str = "auto", shards: ArenaLayout | None = None,
                 params: ArenaLayout | None = None) -> np.ndarray:
    """Records rank ``src_rank`` must push: sources inside its shard arena at
    ``shard_base``, destinations inside rank t's parameter arena at
    ``param_bases[t]`` (addresses valid in this process).  (n, 6) uint64."""
    from .runtime import plan_reshard as clip_native   # mxb_plan_reshard: clip + split in the library

    shards = shards or shard_arena(index, world)
    per_dst = []
    for t in range(tp_size):
        plan = plan_checkpoint(index, t, tp_size, family)
        pa = params or param_arena(plan)
        recs = []
        for pl in plan.placements:
            so, do, rows, rb, sp, dp = pl.geometry()
            per = shards.sizes[pl.src_name]
            lo, hi = src_rank * per, (src_rank + 1) * per
            got = clip_native([(so, param_bases[t] + pa.offsets[pl.dst_name] + do, rows, rb, sp, dp)],
                              lo, hi, shard_base + shards.offsets[pl.src_name], 8 << 20)
            recs += [tuple(r) for r in got.tolist()]
        per_dst.append(recs)
    # All-to-all schedule.  The kernel walks the table in order, so table order is
    # link order: the destinations' record lists are merged by progress (the list
    # that is furthest behind, in bytes, goes next; ties start at destination s+1),
    # so every peer link and the local copies are busy from the first tile to the
    # last instead of all sources hitting destination 0's ingress first.
    order = [(src_rank + 1 + i) % tp_size for i in range(tp_size)]
    totals = [sum(r[2] * r[3] for r in per_dst[t]) or 1 for t in range(tp_size)]
    done = [0] * tp_size
    cursor = [0] * tp_size
    out = []
    remaining = sum(len(r) for r in per_dst)
    while remaining:
        best = None
        for t in order:
            if cursor[t] >= len(per_dst[t]):
                continue
            frac = done[t] / totals[t]
            if best is None or frac < best[0]:
                best = (frac, t)
        t = best[1]
        rec = per_dst[t][cursor[t]]
        out.append(rec)
        cursor[t] += 1
        done[t] += rec[2] * rec[3]
        remaining -= 1
    return np.array(out, dtype=np.uint64).reshape(-1, 6)


def reshard_bytes(records: np.ndarray) -> int:
    return int((records[:, 2] * records[:, 3]).sum()) if len(records) else 0
