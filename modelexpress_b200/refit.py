"""RL refit, receiving side: published trainer shards -> this rank's live parameters.

The reference's ``ReshardReceiver`` (refit/reshard/receiver.py:336-1043) does, per
inference rank: discover the trainers' shard tables, dry-run the engine's loader
to learn which slices it needs (``_capture``), plan byte segments
(``plan_transfer``), RDMA them into receive buffers through NIXL every step
(``update_weights``), cast the dtype-mismatched ones and install the buffers into
the live parameters.  This module is the data-plane core of that cycle on one
NVLink box, with the control plane left to the caller:

* ``PublishedShard`` / ``PublishedTensor`` / ``merge_shard_tables`` /
  ``build_sources`` are the shard-table types and helpers of
  refit/reshard/rendezvous.py:68-272 with the same fields and rules, so tables
  decoded by the reference's rendezvous can be passed in as they are;
* ``ReshardReceiver.prepare`` captures the model's ``load_weights`` once
  (``geometry.capture_geometry``), plans 2-D records against the shards
  (``planner.plan_transfer_2d``) and uploads them as ONE resident table;
* ``ReshardReceiver.update_weights(step)`` replays that table in one persistent
  launch: trainer shards are read in place over NVLink (peer memory mapped by the
  caller, e.g. with ``runtime.ipc_open``) and written straight into the live
  parameters — there is no receive buffer and no install step for parameters kept
  at the served dtype; dtype-changing copies go through a small staging buffer
  and one cast each, as in the reference (receiver.py:964-971);
* ``verify=True`` digests every published shard in place in one launch and compares
  with the digest its publisher attached, before a byte is written (the strict gate
  of modelexpress_rl/inference/nixl_staged_transfer.py:529-549).

Quantised engines whose live parameters are not the load-time parameters need
the engine's own post-load processing after the bytes land; that hook is the
caller's (``install`` argument), as ``_install`` is the subclass's in the reference.
"""

from __future__ import annotations

import json
import logging
import math
import os
import time
from dataclasses import dataclass, field
from typing import Callable

from .planner import (DirectCast, ShardSpec, SourceSpec, apply_converts, convert_staging_bytes,
                      plan_transfer_2d)
from .runtime import Context, Table, default_context

__all__ = ["IncompleteRefit", "check_coverage", "check_throughput_ceiling",
           "PublishedShard", "PublishedTensor", "merge_shard_tables", "build_sources",
           "encode_shard_table", "decode_shard_table", "decode_shard_entries", "publish_local_shards",
           "ReshardReceiver", "SHARD_TABLE_SCHEMA"]

SHARD_TABLE_SCHEMA = "mx.reshard.shard_table.v1"   # rendezvous.py:52


@dataclass
class PublishedShard:
    """rendezvous.py:68-84: the sub-box one trainer rank owns and where to read it."""

    agent_name: str
    device_id: int
    addr: int
    shard_offset: tuple
    shape: tuple
    digest: str | None = None


@dataclass
class PublishedTensor:
    """rendezvous.py:87-96: a full source tensor and the shards that cover it."""

    name: str
    dtype: str  # e.g. "torch.bfloat16"
    elsize: int
    full_shape: tuple
    shards: list = field(default_factory=list)


def encode_shard_table(tensors: list) -> bytes:
    """The JSON blob a publisher hands to the rendezvous, byte for byte what
    rendezvous.py:99-133 writes: ``digest`` is left out, not written as null,
    when a shard has none."""
    import json

    def shard(s) -> dict:
        out = {"agent_name": s.agent_name, "device_id": s.device_id, "addr": s.addr,
               "shard_offset": list(s.shard_offset), "shape": list(s.shape)}
        if s.digest is not None:
            out["digest"] = s.digest
        return out

    payload = {"schema": SHARD_TABLE_SCHEMA,
               "tensors": [{"name": t.name, "dtype": t.dtype, "elsize": t.elsize,
                            "full_shape": list(t.full_shape),
                            "shards": [shard(s) for s in t.shards]} for t in tensors]}
    return json.dumps(payload).encode("utf-8")


def decode_shard_entries(entries: list) -> list:
    """Parsed shard-table entries -> ``PublishedTensor`` list (rendezvous.py:145-175)."""
    return [PublishedTensor(t["name"], t["dtype"], int(t["elsize"]), tuple(t["full_shape"]),
                            [PublishedShard(s["agent_name"], int(s["device_id"]), int(s["addr"]),
                                            tuple(s["shard_offset"]), tuple(s["shape"]), s.get("digest"))
                             for s in t["shards"]]) for t in entries]


def decode_shard_table(blob: bytes) -> list:
    """Inverse of ``encode_shard_table``; a blob of another schema raises
    ``ValueError`` (rendezvous.py:136-142)."""
    import json

    payload = json.loads(blob.decode("utf-8"))
    schema = payload.get("schema")
    if schema != SHARD_TABLE_SCHEMA:
        raise ValueError(f"unexpected shard-table schema {schema!r} (want {SHARD_TABLE_SCHEMA!r})")
    return decode_shard_entries(payload["tensors"])


def publish_local_shards(shards: dict, agent_name: str, *, digests: bool = True, ctx=None) -> list:
    """A trainer rank's table: ``shards`` maps a source name to
    ``(local CUDA tensor, full_shape, shard_offset)``.  All digests of the table
    come from ONE launch of the digest kernel (the reference digests shard by
    shard on the publisher, verify.py:186-196, and only when asked to)."""
    from .digest import digest_many
    from .runtime import DIGEST_ROWS

    names = list(shards)
    tensors = [shards[n][0] for n in names]
    for n, t in zip(names, tensors):
        if not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{n}: a published shard must be a contiguous CUDA tensor")
    digs = [r["tensor_digest"] for r in digest_many(tensors, DIGEST_ROWS, ctx)] if digests and tensors \
        else [None] * len(names)
    out = []
    for n, t, dg in zip(names, tensors, digs):
        _t, full_shape, offset = shards[n]
        out.append(PublishedTensor(n, str(t.dtype), int(t.element_size()), tuple(int(x) for x in full_shape), [
            PublishedShard(agent_name, int(t.device.index or 0), int(t.data_ptr()),
                           tuple(int(x) for x in offset), tuple(int(x) for x in t.shape), dg)]))
    return out


def merge_shard_tables(tables: list) -> list:
    """Per-rank tables -> one table, shards of a name concatenated across ranks,
    ONE representative per exact (offset, shape) so that replicated publishers
    are read once; inconsistent shape/dtype across ranks raises ``ValueError``
    (rendezvous.py:220-272)."""
    merged: dict = {}
    seen: dict = {}
    for table in tables:
        for t in table:
            cur = merged.get(t.name)
            if cur is None:
                merged[t.name] = PublishedTensor(t.name, t.dtype, t.elsize, tuple(t.full_shape), [])
                seen[t.name] = {}
            elif tuple(cur.full_shape) != tuple(t.full_shape) or cur.dtype != t.dtype:
                raise ValueError(
                    f"tensor {t.name!r} published with inconsistent shape/dtype across ranks: "
                    f"{cur.full_shape}/{cur.dtype} vs {t.full_shape}/{t.dtype}")
            for shard in t.shards:
                seen[t.name].setdefault((tuple(shard.shard_offset), tuple(shard.shape)), shard)
    for name, tensor in merged.items():
        tensor.shards.extend(seen[name].values())
    return list(merged.values())


def _torch_dtype(label: str):
    import torch

    return getattr(torch, str(label).replace("torch.", ""))


def build_sources(tensors: list, map_address: Callable | None = None) -> dict:
    """Published tensors -> ``{name: SourceSpec}`` for the planner
    (rendezvous.py:184-217).  ``map_address(shard) -> int`` translates a
    publisher's address into one this process can read (a CUDA IPC mapping of
    the trainer's arena); without it addresses are taken as they are."""
    sources = {}
    for t in tensors:
        shards = [ShardSpec(tuple(s.shard_offset), tuple(s.shape), s.agent_name,
                            int(map_address(s)) if map_address is not None else int(s.addr),
                            int(t.elsize), s.digest) for s in t.shards]
        sources[t.name] = SourceSpec(tuple(t.full_shape), _torch_dtype(t.dtype), int(t.elsize), shards)
    return sources


logger = logging.getLogger("modelexpress_b200.refit")


class IncompleteRefit(RuntimeError):
    """The refit was planned without error and still writes too few of the engine's
    parameter bytes (refit/reshard/types.py:27-35): not a geometry problem, so it is
    a type of its own that handlers for unplannable sources do not swallow."""


_TRUTHY = ("1", "true", "yes", "on")


def _env(name: str, default: str = "") -> str:
    """``MXB_<name>``, else the reference's ``MX_<name>`` (envs.py:65-75), read at call time."""
    v = os.environ.get("MXB_" + name)
    return v if v is not None else os.environ.get("MX_" + name, default)


def _env_float(name: str, default: float) -> float:
    try:
        return float(_env(name, str(default)))
    except ValueError:
        return default


def check_coverage(coverage: float, written_bytes: int, engine_bytes: int, missed: list,
                   n_params: int) -> None:
    """The coverage gate of refit/reshard/receiver.py:746-755.  Opt-in
    (``RESHARD_REQUIRE_FULL_COVERAGE``): partial refits are a feature, but a refit
    that is meant to be complete and leaves parameters at their previous values
    passes every digest check, because bytes that are never requested are never
    checked.  ``RESHARD_COVERAGE_FLOOR`` (default 0.995) leaves room for derived
    buffers that are not refit material."""
    if _env("RESHARD_REQUIRE_FULL_COVERAGE").strip().lower() not in _TRUTHY:
        return
    floor = _env_float("RESHARD_COVERAGE_FLOOR", 0.995)
    if coverage < floor:
        raise IncompleteRefit(
            f"refit covers {100.0 * coverage:.2f}% of the engine's parameter bytes "
            f"({written_bytes} of {engine_bytes}); {len(missed)} of {n_params} params would keep their "
            f"previous values, e.g. {sorted(missed)[:5]}. Set MXB_RESHARD_REQUIRE_FULL_COVERAGE=0 for "
            f"an intentionally partial refit.")


def check_throughput_ceiling(step: int, wire_bytes: int, wire_s: float, rank: int = 0) -> None:
    """Refuse a rate the links cannot produce (refit/reshard/receiver.py:1045-1106):
    such a step did not move its payload, whatever the completions say, so it is
    reported as failed instead of being filed as the fastest one.  The ceiling
    (``RESHARD_MAX_GBPS``, gigabits per second per rank, 0 or a non-finite value =
    off) is the operator's: on one box it is NVLink ingress plus local HBM."""
    ceiling = _env_float("RESHARD_MAX_GBPS", 0.0)
    if not math.isfinite(ceiling) or ceiling <= 0 or wire_bytes <= 0 or wire_s <= 0:
        return
    implied = wire_bytes * 8 / wire_s / 1e9
    if implied <= ceiling:
        return
    detail = {"schema": "refit-impossible-throughput-v1", "rank": rank, "step": step,
              "wire_bytes": wire_bytes, "wire_s": round(wire_s, 6), "implied_gbps": round(implied, 1),
              "ceiling_gbps": ceiling}
    logger.warning("MX_REFIT_IMPOSSIBLE_THROUGHPUT %s", json.dumps(detail))
    raise RuntimeError(
        f"[reshard] step {step} moved {wire_bytes} bytes in {wire_s:.4f}s, an implied {implied:.1f} Gbps "
        f"against a per-rank ceiling of {ceiling:.1f} Gbps. The links cannot deliver that, so the step "
        f"did not move its payload. Treat this refit as failed, not fast.")


class ReshardReceiver:
    """One inference rank's refit cycle: ``prepare`` once, ``update_weights`` per step."""

    def __init__(self, model, *, device=None, ctx: Context | None = None,
                 load_weights: Callable | None = None, install: Callable | None = None):
        import torch

        self.model = model
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None \
            else torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("ReshardReceiver needs a CUDA device (no CPU fallback)")
        self._dev = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.ctx = ctx if ctx is not None else default_context(self._dev)
        self._load_weights = load_weights
        self._install = install
        self._table: Table | None = None
        self._sources: dict = {}
        self._converts: list = []
        self._staged: list = []
        self._direct = None
        self._staging = None
        self._dests: dict = {}
        self.plan: dict = {}

    # ------------------------------------------------------------------ prepare
    def prepare(self, sources, map_address: Callable | None = None) -> dict:
        """Capture, plan and upload.  ``sources`` is ``{name: SourceSpec}`` or a list
        of ``PublishedTensor``.  Fails closed (``RuntimeError``) when a source the
        loader uses cannot be planned, like the reference's receiver; returns the
        plan summary also kept in ``self.plan``."""
        import torch

        from .geometry import capture_geometry
        from .loader import model_destinations

        t0 = time.perf_counter()
        if not isinstance(sources, dict):
            sources = build_sources(list(sources), map_address)
        manifest = [(n, s.dtype, tuple(s.global_shape)) for n, s in sources.items()]
        cap = capture_geometry(self.model, manifest, self._load_weights, device=self.device)
        t_capture = time.perf_counter() - t0
        dests = model_destinations(self.model)
        # shards are device memory this GPU reads in place: a cast between float dtypes needs no
        # staging (MXB_RESHARD_FUSED_CASTS=0 stages the served dtype and casts afterwards)
        fuse = _env("RESHARD_FUSED_CASTS", "1") != "0"
        nbytes = convert_staging_bytes(cap.copies, sources, fuse_casts=fuse)
        staging = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=self.device)
        table, not_planned, converts = plan_transfer_2d(
            cap.copies, sources, lambda n: dests[n].data_ptr(), staging.data_ptr() if nbytes else None,
            fuse_casts=fuse, dst_elsize=lambda n: dests[n].element_size())
        reasons = dict(cap.unsupported_reasons)
        for n in not_planned:
            reasons.setdefault(n, "the copied window is not a box of the source tensor")
        if reasons:
            first = next(iter(reasons))
            raise RuntimeError(f"reshard refit cannot plan {len(reasons)} source(s), e.g. "
                               f"{first!r}: {reasons[first]}")
        self.close()
        self._table = self.ctx.table(table, self._dev) if len(table) else None
        self._sources, self._converts, self._staging, self._dests = sources, converts, staging, dests
        self._staged = [c for c in converts if not isinstance(c, DirectCast)]
        direct = [b for c in converts if isinstance(c, DirectCast) for b in c.boxes]
        self._direct = self.ctx.convert_array(direct) if direct else None   # marshalled once, replayed every step
        planned = {c.param_name for c in cap.copies}
        total = sum(t.numel() * t.element_size() for t in
                    {id(p): p for p in self.model.parameters()}.values())
        moved = int((table[:, 2] * table[:, 3]).sum()) if len(table) else 0
        moved += sum(c.nbytes for c in converts if isinstance(c, DirectCast))
        used = {c.src_name for c in cap.copies}
        all_params = {id(p): n for n, p in self.model.named_parameters()}
        missed = sorted(set(all_params.values()) - planned)
        self.plan = {
            "copies": len(cap.copies), "records": int(len(table)), "bytes_per_step": moved,
            "converts": [c.param_name for c in converts],
            "fused_casts": [c.param_name for c in converts if isinstance(c, DirectCast)],
            "params_written": len(planned),
            "coverage": (moved / total) if total else 1.0,
            "sources_unused": sorted(set(sources) - used),
            "engine": self._table.engine() if self._table is not None else "none",
            "prepare_capture_s": round(t_capture, 6),
            "params_missed": missed,
            "prepare_total_s": round(time.perf_counter() - t0, 6)}
        try:
            check_coverage(self.plan["coverage"], moved, total, missed, len(all_params))
        except IncompleteRefit:
            self.close()
            raise
        return self.plan

    # ------------------------------------------------------------------- verify
    def verify_published(self) -> int:
        """Digest every published shard in place (one launch) and compare with the
        digest its publisher attached; raises ``RuntimeError`` naming the first
        shard that is missing a digest or differs.  Returns the shards checked."""
        from .digest import digest_hex, scalars_from_record
        from .runtime import DIGEST_ROWS

        spans, labels, wants = [], [], []
        for name, src in self._sources.items():
            for sh in src.shards:
                if not sh.digest:
                    raise RuntimeError(f"source {name!r} did not publish a verification digest")
                n = int(src.elsize)
                for extent in sh.shape:
                    n *= int(extent)
                spans.append((int(sh.addr) if n else 0, n))
                labels.append(f"{name}@{tuple(sh.shard_offset)}")
                wants.append(sh.digest)
        if not spans:
            return 0
        recs = self.ctx.digest(spans, DIGEST_ROWS, self._dev)
        for label, want, rec in zip(labels, wants, recs):
            have = digest_hex(scalars_from_record(rec))
            if have != want:
                raise RuntimeError(f"digest mismatch for shard {label}: published {want}, read {have}")
        return len(spans)

    # ------------------------------------------------------------------- update
    def update_weights(self, step: int, *, verify: bool = False) -> dict:
        """Pull this step's weights: one replay of the resident table (plus the
        casts and the caller's install hook).  The trainers must have finished
        writing their shards (the caller's barrier, as in the reference).  Returns
        the stage record of the step."""
        import torch

        if self._table is None and not self.plan:
            raise RuntimeError("prepare() has not been called")
        stages = {"step": int(step)}
        t0 = time.perf_counter()
        torch.cuda.current_stream(self.device).synchronize()
        if verify:
            stages["shards_verified"] = self.verify_published()
            stages["verify_s"] = time.perf_counter() - t0
        t1 = time.perf_counter()
        if self._table is not None:
            self._table.launch()
        if self._direct is not None:
            # casts read in place from the shards: part of the pull, on the same stream
            self.ctx.convert_boxes(self._direct, self._dev)
        if self._table is not None or self._direct is not None:
            # the launches only queue kernels on the library's own stream: wait for them (and
            # learn of a device-side wait that ran out) before anything reads what they wrote
            self.ctx.sync(self._dev)
        stages["read_s"] = time.perf_counter() - t1
        # before anything reads or installs what the step wrote
        check_throughput_ceiling(int(step), int(self.plan.get("bytes_per_step", 0)), stages["read_s"])
        t2 = time.perf_counter()
        if self._staged:
            apply_converts(self._staged, self._staging, self._dests, self.ctx)
        if self._install is not None:
            self._install(self.model)
        torch.cuda.current_stream(self.device).synchronize()
        stages["install_s"] = time.perf_counter() - t2
        stages["total_s"] = time.perf_counter() - t0
        stages["bytes"] = self.plan.get("bytes_per_step", 0)
        stages["gbps"] = stages["bytes"] / stages["read_s"] / 1e9 if stages["read_s"] > 0 else 0.0
        return stages

    def close(self) -> None:
        self._direct = None
        if self._table is not None:
            self._table.close()
            self._table = None
