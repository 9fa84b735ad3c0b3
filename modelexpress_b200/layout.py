"""Tensor-parallel placement rules: checkpoint tensors -> per-rank parameters.

This is the host-staged path's shard arithmetic, stated as geometry instead of
as per-tensor ``narrow`` + ``copy_`` calls.  The reference reaches it through
engines/vllm/adapter.py:316-329 (vLLM's column / merged-column / QKV / row /
vocab-parallel ``weight_loader``s) and states the same splits itself in
engines/vllm/refit/installer.py:72-78 (stacked groups and their pack order),
:292-317 (narrow on the one axis where loaded == expected * tp), :566-616
(running offsets of fused members) and :695-771 (expert slots).

``plan_checkpoint`` turns a checkpoint index into ``Placement`` records; each
one is a single-axis slice of a source tensor landing at an offset of a
destination parameter, which is exactly one 2-D scatter record
(``Placement.record``).
"""

from __future__ import annotations

import re
from dataclasses import dataclass, field

from .safetensors_index import SAFETENSORS_DTYPES

VOCAB_PAD = 64  # vLLM pads the vocabulary to a multiple of 64 and zero-fills the pad rows


@dataclass
class ParamSpec:
    name: str
    shape: tuple
    dtype: str  # safetensors dtype tag
    zero_fill: bool = False  # has bytes no checkpoint tensor covers (vocab padding)

    @property
    def nbytes(self) -> int:
        n = SAFETENSORS_DTYPES[self.dtype][0]
        for s in self.shape:
            n *= int(s)
        return n


@dataclass
class Placement:
    """``src[axis: start..start+size]`` -> ``dst`` at ``dst_start`` on the same axis."""

    src_name: str
    src_shape: tuple
    dtype: str
    axis: int
    start: int
    size: int
    dst_name: str
    dst_shape: tuple
    dst_start: int
    dst_extra: int = 0  # further element offset into the destination (a slot of a stacked parameter)

    def geometry(self) -> tuple:
        """(src_byte_off, dst_byte_off, rows, row_bytes, src_pitch, dst_pitch)."""
        el = SAFETENSORS_DTYPES[self.dtype][0]
        shape = self.src_shape if self.src_shape else (1,)
        dshape = self.dst_shape if self.dst_shape else (1,)
        outer = 1
        for s in shape[: self.axis]:
            outer *= int(s)
        inner = 1
        for s in shape[self.axis + 1:]:
            inner *= int(s)
        row_bytes = self.size * inner * el
        src_pitch = int(shape[self.axis]) * inner * el
        dst_pitch = int(dshape[self.axis]) * inner * el
        dst_off = (self.dst_start * inner + self.dst_extra) * el
        if outer == 1 or (src_pitch == row_bytes and dst_pitch == row_bytes):
            return (self.start * inner * el, dst_off, 1, outer * row_bytes,
                    outer * row_bytes, outer * row_bytes)
        return (self.start * inner * el, dst_off, outer, row_bytes, src_pitch, dst_pitch)

    def record(self, src_base: int, dst_base: int) -> tuple:
        so, do, rows, rb, sp, dp = self.geometry()
        return (src_base + so, dst_base + do, rows, rb, sp, dp)

    @property
    def nbytes(self) -> int:
        _so, _do, rows, rb, _sp, _dp = self.geometry()
        return rows * rb


@dataclass
class CheckpointPlan:
    params: dict = field(default_factory=dict)  # name -> ParamSpec
    placements: list = field(default_factory=list)

    @property
    def bytes_placed(self) -> int:
        return sum(p.nbytes for p in self.placements)


_QKV = ("q_proj", "k_proj", "v_proj")  # pack order, installer.py:72-78
_GATE_UP = ("gate_proj", "up_proj")


def _split(extent: int, tp: int, what: str) -> int:
    if extent % tp:
        raise ValueError(f"{what}: extent {extent} does not divide by tp={tp}")
    return extent // tp


def plan_dense(index: dict, tp_rank: int, tp_size: int) -> CheckpointPlan:
    """Llama / Qwen2-style dense decoder: q,k,v -> qkv_proj and gate,up ->
    gate_up_proj (column-parallel members stacked in pack order), o_proj and
    down_proj row-parallel, embed_tokens and lm_head vocab-parallel, everything
    else replicated.  ``index`` maps HF names to {"shape", "dtype"}."""
    if not 0 <= tp_rank < tp_size:
        raise ValueError("tp_rank out of range")
    plan = CheckpointPlan()
    groups: dict = {}
    for name, info in index.items():
        shape, dtype = tuple(int(s) for s in info["shape"]), info["dtype"]
        m = re.match(r"(.*\.)(q_proj|k_proj|v_proj|gate_proj|up_proj)\.(weight|bias|weight_scale_inv)$", name)
        if m:
            fused = "qkv_proj" if m.group(2) in _QKV else "gate_up_proj"
            groups.setdefault((m.group(1), fused, m.group(3)), {})[m.group(2)] = (name, shape, dtype)
            continue
        if re.search(r"\.gate_up_proj\.(weight|weight_scale_inv)$", name) and len(shape) >= 1:
            # a checkpoint that ships [gate; up] already merged (GLM-4 style): the two
            # partitions are column-parallel independently, so rank r takes rows
            # [r*L, (r+1)*L) of each half and stacks them (installer.py:670-693)
            parts = 2
            if shape[0] % (parts * tp_size):
                raise ValueError(f"{name}: {shape[0]} rows do not split into {parts} x tp={tp_size}")
            part_src = shape[0] // parts
            loc = part_src // tp_size
            dshape = (parts * loc,) + tuple(shape[1:])
            plan.params[name] = ParamSpec(name, dshape, dtype)
            for p in range(parts):
                plan.placements.append(Placement(name, shape, dtype, 0, p * part_src + tp_rank * loc,
                                                 loc, name, dshape, p * loc))
            continue
        if re.search(r"\.(o_proj|down_proj)\.(weight|weight_scale_inv)$", name) and len(shape) == 2:
            loc = _split(shape[1], tp_size, name)
            plan.params[name] = ParamSpec(name, (shape[0], loc), dtype)
            plan.placements.append(Placement(name, shape, dtype, 1, tp_rank * loc, loc, name,
                                             (shape[0], loc), 0))
            continue
        if re.search(r"(embed_tokens|lm_head)\.weight$", name) and len(shape) == 2:
            vocab = shape[0]
            padded = (vocab + VOCAB_PAD - 1) // VOCAB_PAD * VOCAB_PAD
            loc = _split(padded, tp_size, name)
            lo = tp_rank * loc
            hi = min(vocab, lo + loc)
            dshape = (loc, shape[1])
            plan.params[name] = ParamSpec(name, dshape, dtype, zero_fill=(hi - lo) < loc)
            if hi > lo:
                plan.placements.append(Placement(name, shape, dtype, 0, lo, hi - lo, name, dshape, 0))
            continue
        plan.params[name] = ParamSpec(name, shape, dtype)
        plan.placements.append(Placement(name, shape, dtype, 0, 0, shape[0] if shape else 1, name,
                                         shape, 0))
    for (prefix, fused, kind), members in groups.items():
        order = _QKV if fused == "qkv_proj" else _GATE_UP
        missing = [m for m in order if m not in members]
        if missing:
            raise KeyError(f"{prefix}{fused}.{kind}: checkpoint lacks {missing}")
        dtype = members[order[0]][2]
        locs = [_split(members[m][1][0], tp_size, members[m][0]) for m in order]
        trailing = members[order[0]][1][1:]
        dshape = (sum(locs),) + tuple(trailing)
        dst = f"{prefix}{fused}.{kind}"
        plan.params[dst] = ParamSpec(dst, dshape, dtype)
        off = 0
        for m, loc in zip(order, locs):
            name, shape, _dt = members[m]
            if tuple(shape[1:]) != tuple(trailing):
                raise ValueError(f"{name}: trailing dims differ inside {dst}")
            plan.placements.append(Placement(name, shape, dtype, 0, tp_rank * loc, loc, dst, dshape, off))
            off += loc
    return plan


_EXPERT = re.compile(r"(.*\.mlp\.)experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.(weight|weight_scale_inv)$")
_SHARED = re.compile(r"(.*\.mlp\.shared_experts\.)(gate_proj|up_proj|down_proj)\.(weight|weight_scale_inv)$")
_MLA_COL = re.compile(r"\.self_attn\.(q_b_proj|kv_b_proj)\.(weight|weight_scale_inv)$")
_MLA_ROW = re.compile(r"\.self_attn\.o_proj\.(weight|weight_scale_inv)$")
_MLA_A = re.compile(r"(.*\.self_attn\.)(q_a_proj|kv_a_proj_with_mqa)\.(weight|weight_scale_inv)$")


def plan_moe(index: dict, tp_rank: int, tp_size: int, ep_rank: int | None = None,
             ep_size: int | None = None, expert_tp: tuple = (0, 1)) -> CheckpointPlan:
    """DeepSeek-V3-style block-FP8 MoE: routed experts expert-parallel into
    ``experts.w13_weight[slot, half]`` / ``w2_weight[slot]`` with their
    ``weight_scale_inv`` blocks alongside (installer.py:695-771: gate is the low
    half of w13, up the high half, slot = global id - first local id); the shared
    expert and MLA projections tensor-parallel with scale rows/cols split in
    step (128-blocks); q_a/kv_a fused and replicated; the rest replicated.
    ``expert_tp = (rank, size)`` additionally splits every routed expert
    tensor-parallel (gate/up rows, down columns; installer.py:737-768), for
    engines that do not run their experts expert-parallel."""
    ep_rank = tp_rank if ep_rank is None else ep_rank
    ep_size = tp_size if ep_size is None else ep_size
    et_rank, et_size = int(expert_tp[0]), int(expert_tp[1])
    plan = CheckpointPlan()
    experts: dict = {}
    dense_part: dict = {}
    mla_a: dict = {}
    for name, info in index.items():
        shape, dtype = tuple(int(s) for s in info["shape"]), info["dtype"]
        m = _EXPERT.match(name)
        if m:
            experts.setdefault((m.group(1), m.group(4)), {})[(int(m.group(2)), m.group(3))] = (name, shape, dtype)
            continue
        m = _SHARED.match(name)
        if m:
            # same rules as a dense MLP under a different prefix
            dense_part[name] = info
            continue
        if _MLA_COL.search(name) and len(shape) == 2:
            loc = _split(shape[0], tp_size, name)
            plan.params[name] = ParamSpec(name, (loc, shape[1]), dtype)
            plan.placements.append(Placement(name, shape, dtype, 0, tp_rank * loc, loc, name,
                                             (loc, shape[1]), 0))
            continue
        if _MLA_ROW.search(name) and len(shape) == 2:
            loc = _split(shape[1], tp_size, name)
            plan.params[name] = ParamSpec(name, (shape[0], loc), dtype)
            plan.placements.append(Placement(name, shape, dtype, 1, tp_rank * loc, loc, name,
                                             (shape[0], loc), 0))
            continue
        m = _MLA_A.match(name)
        if m:
            mla_a.setdefault((m.group(1), m.group(3)), {})[m.group(2)] = (name, shape, dtype)
            continue
        plan.params[name] = ParamSpec(name, shape, dtype)
        plan.placements.append(Placement(name, shape, dtype, 0, 0, shape[0] if shape else 1, name,
                                         shape, 0))
    sub = plan_dense(dense_part, tp_rank, tp_size)
    plan.params.update(sub.params)
    plan.placements.extend(sub.placements)
    for (prefix, kind), members in mla_a.items():
        order = [m for m in ("q_a_proj", "kv_a_proj_with_mqa") if m in members]
        dtype = members[order[0]][2]
        trailing = members[order[0]][1][1:]
        dshape = (sum(members[m][1][0] for m in order),) + tuple(trailing)
        dst = f"{prefix}fused_qkv_a_proj.{kind}"
        plan.params[dst] = ParamSpec(dst, dshape, dtype)
        off = 0
        for m in order:
            name, shape, _dt = members[m]
            plan.placements.append(Placement(name, shape, dtype, 0, 0, shape[0], dst, dshape, off))
            off += shape[0]
    for (prefix, kind), members in experts.items():
        n_experts = 1 + max(e for e, _ in members)
        per = _split(n_experts, ep_size, f"{prefix}experts")
        first = ep_rank * per
        g = members[(first, "gate_proj")]
        dn = members[(first, "down_proj")]
        dtype = g[2]
        suffix = "weight" if kind == "weight" else "weight_scale_inv"
        w13 = f"{prefix}experts.w13_{suffix}"
        w2 = f"{prefix}experts.w2_{suffix}"
        half = _split(g[1][0], et_size, f"{prefix}experts gate rows")
        down_cols = _split(dn[1][1], et_size, f"{prefix}experts down columns") if len(dn[1]) > 1 else 1
        w13_shape = (per, 2 * half) + tuple(g[1][1:])
        w2_shape = (per, dn[1][0], down_cols) + tuple(dn[1][2:]) if len(dn[1]) > 1 else (per,) + tuple(dn[1])
        plan.params[w13] = ParamSpec(w13, w13_shape, dtype)
        plan.params[w2] = ParamSpec(w2, w2_shape, dn[2])
        for slot in range(per):
            e = first + slot
            for proj, lo in (("gate_proj", 0), ("up_proj", half)):
                name, shape, _dt = members[(e, proj)]
                # the slot is a [2*half, ...] matrix inside the 3-D parameter: address it
                # as axis 0 of a flattened (per*2*half, ...) view
                flat = (per * 2 * half,) + tuple(shape[1:])
                plan.placements.append(Placement(name, shape, dtype, 0, et_rank * half, half, w13, flat,
                                                 slot * 2 * half + lo))
            name, shape, _dt = members[(e, "down_proj")]
            if et_size == 1 or len(shape) < 2:
                flat = (per * shape[0],) + tuple(shape[1:])
                plan.placements.append(Placement(name, shape, dn[2], 0, 0, shape[0], w2, flat,
                                                 slot * shape[0]))
            else:
                # a column block of every row, landing in slot `slot` of [per, rows, cols/size]
                inner = 1
                for extent in shape[2:]:
                    inner *= int(extent)
                plan.placements.append(Placement(name, shape, dn[2], 1, et_rank * down_cols, down_cols, w2,
                                                 (shape[0], down_cols) + tuple(shape[2:]), 0,
                                                 slot * shape[0] * down_cols * inner))
    return plan


def plan_checkpoint(index: dict, tp_rank: int, tp_size: int, family: str = "auto") -> CheckpointPlan:
    if family == "auto":
        family = "moe" if any(".mlp.experts." in n for n in index) else "dense"
    if family == "dense":
        return plan_dense(index, tp_rank, tp_size)
    if family == "moe":
        return plan_moe(index, tp_rank, tp_size)
    raise ValueError(f"unknown model family {family!r}")
