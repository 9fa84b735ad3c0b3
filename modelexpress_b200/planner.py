"""Descriptor compiler: captured copies + published shards -> 2-D scatter records.

The reference plans a refit as a list of 1-D byte runs
(refit/reshard/slice_plan.py:297-339 ``plan_pull``; one run per row of a strided
slice, built by ``itertools.product`` in Python).  This module resolves the same
geometry — the view chain a loader applied to a full source tensor, intersected
with each published shard box — but emits the closed form the scatter kernel
consumes: one ``(src, dst, rows, row_bytes, src_pitch, dst_pitch)`` record per
innermost strided dimension.  Expanding a record row by row gives exactly the
reference's run list, in the reference's order.

Objects are duck-typed on the reference's field names, so its ``RecordedCopy``
(types.py:57-70) and ``Shard`` (slice_plan.py:54-70) instances can be passed
straight in; ``CopySpec`` / ``ShardSpec`` are equivalents for callers that do
not have the reference package.
"""

from __future__ import annotations

import copy as _copy
from dataclasses import dataclass
from typing import Any

import numpy as np


class UnsupportedReshard(NotImplementedError):
    """The loader's op-chain is not a pure permuted box view, or the copy needs
    a dtype conversion; the caller must fail the update (types.py:21-24)."""


@dataclass
class CopySpec:
    src_name: str
    op_chain: tuple
    param_name: str
    dest_offset: int
    dest_shape: tuple
    dest_stride: tuple
    dest_dtype: Any


@dataclass
class ShardSpec:
    shard_offset: tuple
    shape: tuple
    session: str
    addr: int
    elsize: int
    digest: str | None = None


@dataclass
class SourceSpec:
    """Everything known about one full source tensor (transfer_plan.py:39-46)."""

    global_shape: tuple
    dtype: Any
    elsize: int
    shards: list


def _strides_of(shape):
    st, acc = [], 1
    for extent in reversed(shape):
        st.append(acc)
        acc *= int(extent)
    return st[::-1]


class _View:
    """A strided window into a row-major tensor, moved by view ops only."""

    def __init__(self, shape):
        self.shape = [int(x) for x in shape]
        self.stride = _strides_of(self.shape)
        self.offset = 0

    def _dense(self):
        expect = 1
        for extent, st in zip(reversed(self.shape), reversed(self.stride)):
            if extent != 1 and st != expect:
                return False
            expect *= extent
        return True

    def apply(self, op, args):
        nd = len(self.shape)
        if op == "narrow":
            dim, start, size = (int(a) for a in args)
            dim %= nd
            if start < 0 or size < 0 or start + size > self.shape[dim]:
                raise UnsupportedReshard(f"narrow({dim},{start},{size}) leaves the tensor")
            self.offset += start * self.stride[dim]
            self.shape[dim] = size
        elif op == "__getitem__":
            key = args[0] if args else slice(None)
            for dim, k in enumerate(key if isinstance(key, tuple) else (key,)):
                if not isinstance(k, slice) or k.step not in (None, 1):
                    raise UnsupportedReshard(f"index {k!r} changes rank or stride")
                lo, hi, _ = k.indices(self.shape[dim])
                self.offset += lo * self.stride[dim]
                self.shape[dim] = max(0, hi - lo)
        elif op in ("transpose", "t"):
            if op == "t":
                if nd != 2:
                    raise UnsupportedReshard("t() needs a matrix")
                a, b = 0, 1
            else:
                a, b = int(args[0]) % nd, int(args[1]) % nd
            for seq in (self.shape, self.stride):
                seq[a], seq[b] = seq[b], seq[a]
        elif op == "permute":
            order = args[0] if len(args) == 1 and not isinstance(args[0], int) else args
            order = [int(d) % nd for d in order]
            if sorted(order) != list(range(nd)):
                raise UnsupportedReshard("permute is not a permutation")
            self.shape = [self.shape[d] for d in order]
            self.stride = [self.stride[d] for d in order]
        elif op == "contiguous":
            if not self._dense():
                raise UnsupportedReshard("contiguous() would materialise a copy")
        else:
            raise UnsupportedReshard(f"op {op!r} is not a pure view")


def window_box(offset, shape, stride, global_shape, dest_stride, keep_rank: bool = True,
               with_perm: bool = False):
    """A strided window of a row-major tensor -> (box in source coordinates,
    destination strides in source-dim order); slice_plan.py:170-225.

    Every window dim of extent > 1 must walk exactly one source dim (its stride
    equals that dim's row-major stride) and the offset must be a corner of the
    box.  With ``keep_rank`` the window must have the source's rank, as the
    reference requires; without it, size-1 window dims are ignored and source
    dims the window does not walk have extent 1 (an integer index, ``select``,
    ``unbind`` or ``squeeze`` of the source)."""
    gshape = [int(g) for g in global_shape]
    nd = len(gshape)
    if keep_rank and len(shape) != nd:
        raise UnsupportedReshard("rank change")
    gst = _strides_of(gshape)
    dim_of_stride = {}
    for s in range(nd):
        dim_of_stride.setdefault(gst[s], s)
    perm = [None] * len(shape)
    for d in range(len(shape)):
        if shape[d] == 1:
            continue
        s = dim_of_stride.get(int(stride[d]))
        if s is None:
            raise UnsupportedReshard(f"stride {stride[d]} is not a source dim (merged dims)")
        perm[d] = s
    used = [p for p in perm if p is not None]
    if len(set(used)) != len(used):
        raise UnsupportedReshard("view is not a permutation of the source dims")
    lo = [(int(offset) // gst[s]) % gshape[s] if gshape[s] else 0 for s in range(nd)]
    hi = [x + 1 if gshape[s] else x for s, x in enumerate(lo)]
    for d, s in enumerate(perm):
        if s is not None:
            hi[s] = lo[s] + int(shape[d])
    if any(hi[s] > gshape[s] for s in range(nd)):
        raise UnsupportedReshard("box leaves the source")
    if sum(lo[s] * gst[s] for s in range(nd)) != int(offset):
        raise UnsupportedReshard("offset is not a box corner")
    dst_stride = [0] * nd
    for d, s in enumerate(perm):
        if s is not None:
            dst_stride[s] = int(dest_stride[d])
    if with_perm:
        return [(lo[s], hi[s]) for s in range(nd)], dst_stride, perm
    return [(lo[s], hi[s]) for s in range(nd)], dst_stride


def resolve_slice(copy, global_shape):
    """(needed box in source coordinates, destination strides in source-dim
    order) for one captured copy; slice_plan.py:227-245.  ``copy`` carries
    either the reference's op-chain, which is replayed here, or the resolved
    window of a ``geometry.ViewCopy``."""
    if hasattr(copy, "src_stride"):
        offset, shape, stride, keep_rank = copy.src_offset, copy.src_shape, copy.src_stride, False
    else:
        view = _View(global_shape)
        for op, args, _kw in copy.op_chain:
            view.apply(op, args)
        offset, shape, stride, keep_rank = view.offset, view.shape, view.stride, True
    if len(shape) == len(copy.dest_shape) and tuple(copy.dest_shape) != tuple(shape):
        raise UnsupportedReshard(
            f"{copy.param_name}: destination {tuple(copy.dest_shape)} != view {tuple(shape)}")
    if len(shape) != len(copy.dest_shape):
        raise UnsupportedReshard("rank change")
    return window_box(offset, shape, stride, global_shape, copy.dest_stride, keep_rank)


def box_records(overlap, src_origin, src_strides, dst_origin, dst_strides, elsize,
                src_base, dst_base):
    """2-D records covering ``overlap`` (full-tensor coordinates).

    Trailing dims are merged while both layouts are unit-packed (the same rule
    as slice_plan.py:278-284); the next dim out becomes the row dimension with
    its two pitches; dims further out are enumerated.  Returns an (m, 6) uint64
    array in row-major order of the outer dims, i.e. the reference's run order."""
    nd = len(overlap)
    sizes = [hi - lo for lo, hi in overlap]
    run, p = 1, nd
    while p > 0 and src_strides[p - 1] == run and dst_strides[p - 1] == run:
        run *= sizes[p - 1]
        p -= 1
    s0 = sum((lo - o) * st for (lo, _), o, st in zip(overlap, src_origin, src_strides))
    d0 = sum((lo - o) * st for (lo, _), o, st in zip(overlap, dst_origin, dst_strides))
    row_bytes = run * elsize
    if p == 0:
        return np.array([[src_base + s0 * elsize, dst_base + d0 * elsize, 1, row_bytes,
                          row_bytes, row_bytes]], dtype=np.uint64)
    rows = sizes[p - 1]
    sp, dp = src_strides[p - 1] * elsize, dst_strides[p - 1] * elsize
    if rows > 1 and (sp < row_bytes or dp < row_bytes):
        # overlapping rows cannot be one record; fall back to one record per row
        p_outer, rows, sp, dp = p, 1, row_bytes, row_bytes
    else:
        p_outer = p - 1
    outer = [sizes[d] for d in range(p_outer)]
    n_outer = int(np.prod(outer)) if outer else 1
    out = np.empty((n_outer, 6), dtype=np.uint64)
    if n_outer == 1:
        so, do = np.zeros(1, dtype=np.int64), np.zeros(1, dtype=np.int64)
    else:
        grids = np.indices(outer, dtype=np.int64).reshape(len(outer), -1)
        so = sum(grids[d] * src_strides[d] for d in range(p_outer))
        do = sum(grids[d] * dst_strides[d] for d in range(p_outer))
    out[:, 0] = src_base + (s0 + so) * elsize
    out[:, 1] = dst_base + (d0 + do) * elsize
    out[:, 2] = rows
    out[:, 3] = row_bytes
    out[:, 4] = sp if rows > 1 else row_bytes
    out[:, 5] = dp if rows > 1 else row_bytes
    return out


def copy_window(copy, global_shape) -> tuple:
    """(offset, shape, stride, keep_rank) of the source window ``copy`` reads: the
    reference's op-chain replayed (slice_plan.py:136-168), or the window a
    ``geometry.ViewCopy`` already carries."""
    if hasattr(copy, "src_stride"):
        offset, shape, stride, keep_rank = copy.src_offset, copy.src_shape, copy.src_stride, False
    else:
        view = _View(global_shape)
        for op, args, _kw in copy.op_chain:
            view.apply(op, args)
        offset, shape, stride, keep_rank = view.offset, view.shape, view.stride, True
    if len(shape) == len(copy.dest_shape) and tuple(copy.dest_shape) != tuple(shape):
        raise UnsupportedReshard(
            f"{copy.param_name}: destination {tuple(copy.dest_shape)} != view {tuple(shape)}")
    if len(shape) != len(copy.dest_shape):
        raise UnsupportedReshard("rank change")
    return int(offset), [int(x) for x in shape], [int(x) for x in stride], keep_rank


def plan_pull_2d(copy, global_shape, src_dtype, elsize, shards, dst_base: int):
    """Records that read exactly the slice ``copy`` needs out of ``shards`` and
    write it at ``dst_base`` (the parameter's data pointer).  Returns a list of
    ``(session, records)`` in shard order; raises ``UnsupportedReshard`` for a
    dtype mismatch or a non-view op-chain, ``ValueError`` for rank-mismatched
    shard geometry (as the reference does).  The geometry is compiled by the
    library (``mxb_plan_pull``); ``plan_pull_2d_py`` is the same in Python."""
    from . import _lib
    from .runtime import plan_pull

    if src_dtype != copy.dest_dtype:
        raise UnsupportedReshard(f"{copy.param_name}: dtype conversion required")
    offset, shape, stride, keep_rank = copy_window(copy, global_shape)
    nd = len(global_shape)
    if max(nd, len(shape)) > _lib.MAX_DIMS:
        return plan_pull_2d_py(copy, global_shape, src_dtype, elsize, shards, dst_base)
    for sh in shards:
        if not len(sh.shard_offset) == len(sh.shape) == nd:
            raise ValueError("shard rank does not match the source rank")
    try:
        recs, which = plan_pull(global_shape, int(elsize), offset, shape, stride, int(copy.dest_offset),
                                [int(x) for x in copy.dest_stride],
                                [(sh.shard_offset, sh.shape, int(sh.addr)) for sh in shards],
                                int(dst_base), keep_rank)
    except _lib.MxbError as e:
        if e.code == -9:
            raise UnsupportedReshard(str(e)) from e
        raise
    out = []
    for k in sorted(set(which.tolist())):
        out.append((shards[k].session, recs[which == k]))
    return out


def plan_pull_2d_py(copy, global_shape, src_dtype, elsize, shards, dst_base: int):
    """``plan_pull_2d`` without the library (the planner's Python statement)."""
    if src_dtype != copy.dest_dtype:
        raise UnsupportedReshard(f"{copy.param_name}: dtype conversion required")
    needed, dst_strides = resolve_slice(copy, global_shape)
    origin = [lo for lo, _ in needed]
    out = []
    for sh in shards:
        if not len(sh.shard_offset) == len(sh.shape) == len(needed):
            raise ValueError("shard rank does not match the source rank")
        overlap = []
        for (a0, a1), o, s in zip(needed, sh.shard_offset, sh.shape):
            lo, hi = max(a0, int(o)), min(a1, int(o) + int(s))
            if lo >= hi:
                overlap = None
                break
            overlap.append((lo, hi))
        if overlap is None:
            continue
        recs = box_records(overlap, [int(o) for o in sh.shard_offset], _strides_of(sh.shape),
                           origin, dst_strides, int(elsize), int(sh.addr),
                           int(dst_base) + int(copy.dest_offset) * int(elsize))
        out.append((sh.session, recs))
    return out


def expand_records(records) -> list:
    """(src, dst, nbytes) runs of a record array, row by row (for checking)."""
    runs = []
    for src, dst, rows, rb, sp, dp in np.asarray(records, dtype=np.uint64).tolist():
        for r in range(rows):
            runs.append((src + r * sp, dst + r * dp, rb))
    return runs


@dataclass
class ConvertSpec:
    """A copy whose served dtype differs from the destination's: its bytes are
    pulled into ``staging`` (served dtype, contiguous, ``dest_shape``) and cast
    into the live parameter afterwards (transfer_plan.py:49-60, 226-256)."""

    param_name: str
    dest_shape: tuple
    dest_stride: tuple
    dest_offset: int
    src_dtype: Any
    staging_offset: int  # byte offset in the convert staging buffer
    nbytes: int
    # a transposing copy is staged as the box it reads, in the source's own dim order:
    box_shape: tuple | None = None   # shape of that box in staging (None: staged in dest_shape)
    box_perm: tuple | None = None    # per destination dim, the staging dim it walks (None: extent 1)


@dataclass
class DirectCast:
    """A dtype-changing copy whose sources are device memory this GPU can read (local or a
    mapped peer): every record of the pull becomes one box of the convert kernel, read in place
    from the shard and written cast into the live parameter.  No staging buffer, no second pass
    (the reference stages the served dtype and casts afterwards, transfer_plan.py:49-60)."""

    param_name: str
    boxes: list   # (src, dst, extents, dst_strides, src_kind, dst_kind, elem_bytes, src_strides)
    nbytes: int   # source bytes read


TRANSPOSE_MIN_ELEMENTS = 4096   # below this a transposing copy stays a list of narrow records


def transposed_box(copy, global_shape):
    """``(box_shape, box_perm, corner_offset)`` when ``copy`` walks its source against the
    grain: the source's innermost walked dim does not land with stride 1, so its records
    would be one element wide.  ``None`` for every other copy (and for small ones)."""
    try:
        offset, shape, stride, keep_rank = copy_window(copy, global_shape)
        box, dst_strides, perm = window_box(offset, shape, stride, global_shape, copy.dest_stride,
                                            keep_rank, with_perm=True)
    except UnsupportedReshard:
        return None
    sizes = [hi - lo for lo, hi in box]
    walked = [s for s in range(len(sizes)) if sizes[s] > 1]
    if not walked or dst_strides[walked[-1]] == 1:
        return None
    n = 1
    for extent in sizes:
        n *= extent
    if n < TRANSPOSE_MIN_ELEMENTS:
        return None
    return tuple(sizes), tuple(perm), int(offset)


def _box_copy(copy, src, box_shape, corner: int):
    """The same source box landing contiguously, in source dim order, at offset 0."""
    staged = _copy.copy(copy)
    staged.src_offset = corner
    staged.src_shape = tuple(box_shape)
    staged.src_stride = tuple(_strides_of(src.global_shape))
    staged.dest_offset = 0
    staged.dest_shape = tuple(box_shape)
    staged.dest_stride = tuple(_strides_of(box_shape))
    staged.dest_dtype = src.dtype
    if hasattr(staged, "op_chain"):
        staged.op_chain = ()
    return staged


def direct_cast(copy, src, param_ptr: int, dst_elsize: int) -> DirectCast | None:
    """``copy`` (served dtype != destination dtype, walking its source with the grain) as boxes
    read straight from the shards; ``None`` when the pair of dtypes is outside the convert
    kernel's table.  The pull is planned as for a same-dtype copy against a destination at
    address 0 measured in source elements, then every record's destination is rescaled to the
    parameter's element size."""
    sk, dk = _FLOAT_KINDS.get(str(src.dtype)), _FLOAT_KINDS.get(str(copy.dest_dtype))
    if sk is None or dk is None:
        return None
    ssz = int(src.elsize)
    virtual = _copy.copy(copy)
    virtual.dest_dtype = src.dtype
    parts = plan_pull_2d(virtual, src.global_shape, src.dtype, ssz, src.shards, 0)
    boxes, nbytes = [], 0
    for _sess, recs in parts:
        for s_addr, d_virtual, rows, row_bytes, sp, dp in np.asarray(recs, dtype=np.uint64).tolist():
            if row_bytes % ssz or d_virtual % ssz or sp % ssz or dp % ssz:
                raise UnsupportedReshard(f"{copy.param_name}: a record is not element-granular")
            boxes.append((int(s_addr), int(param_ptr) + d_virtual // ssz * int(dst_elsize),
                          [int(rows), row_bytes // ssz], [dp // ssz, 1], sk, dk, ssz, [sp // ssz, 1]))
            nbytes += int(rows) * int(row_bytes)
    return DirectCast(copy.param_name, boxes, nbytes)


def plan_transfer_2d(copies, sources: dict, resolve_param_ptr, convert_base: int | None = None,
                     fuse_casts: bool = False, dst_elsize=None) -> tuple:
    """All copies of a capture -> one record array.

    Returns ``(records, unsupported, converts)``.  Same-dtype copies write
    straight into the live parameters.  A copy whose source dtype differs from
    the destination's is planned into a contiguous staging buffer at
    ``convert_base`` (served dtype, row-major) and listed in ``converts`` for
    the caller to cast, as the reference does; without ``convert_base`` such
    copies are reported unsupported.  With ``fuse_casts`` (sources in device memory;
    ``dst_elsize(param_name)`` gives the parameter's element size) a cast that walks its
    source with the grain is not staged at all: it comes back as a ``DirectCast`` whose
    boxes the convert kernel reads in place.  Sources that are missing or not
    box-shaped are returned by name so the caller can fail closed
    (transfer_plan.py:192-299 keeps the same outcomes; there is no descriptor
    bound here because a strided slice costs one record, not one per row)."""
    recs, unsupported, converts = [], [], []
    staged = 0
    for copy in copies:
        src = sources.get(copy.src_name)
        if src is None:
            unsupported.append(copy.src_name)
            continue
        try:
            tbox = transposed_box(copy, src.global_shape) if convert_base is not None else None
            if tbox is not None:
                # staged as the box it reads (wide rows), transposed (and cast) on the device
                box_shape, box_perm, corner = tbox
                n = int(np.prod(box_shape))
                off = (staged + 255) // 256 * 256
                parts = plan_pull_2d(_box_copy(copy, src, box_shape, corner), src.global_shape, src.dtype,
                                     src.elsize, src.shards, int(convert_base) + off)
                converts.append(ConvertSpec(copy.param_name, tuple(copy.dest_shape),
                                            tuple(copy.dest_stride), int(copy.dest_offset), src.dtype,
                                            off, n * int(src.elsize), box_shape, box_perm))
                staged = off + n * int(src.elsize)
            elif src.dtype != copy.dest_dtype and fuse_casts and dst_elsize is not None and (
                    fused := direct_cast(copy, src, resolve_param_ptr(copy.param_name),
                                         dst_elsize(copy.param_name))) is not None:
                converts.append(fused)
                parts = []
            elif src.dtype != copy.dest_dtype:
                if convert_base is None:
                    raise UnsupportedReshard("dtype conversion required and no staging given")
                n = int(np.prod(copy.dest_shape)) if len(copy.dest_shape) else 1
                # the same window, landing contiguously in staging at the served dtype
                staging_copy = _copy.copy(copy)
                staging_copy.dest_offset = 0
                staging_copy.dest_stride = tuple(_strides_of(copy.dest_shape))
                staging_copy.dest_dtype = src.dtype
                off = (staged + 255) // 256 * 256
                parts = plan_pull_2d(staging_copy, src.global_shape, src.dtype, src.elsize,
                                     src.shards, int(convert_base) + off)
                converts.append(ConvertSpec(copy.param_name, tuple(copy.dest_shape),
                                            tuple(copy.dest_stride), int(copy.dest_offset), src.dtype,
                                            off, n * int(src.elsize)))
                staged = off + n * int(src.elsize)
            else:
                parts = plan_pull_2d(copy, src.global_shape, src.dtype, src.elsize, src.shards,
                                     resolve_param_ptr(copy.param_name))
        except UnsupportedReshard:
            unsupported.append(copy.src_name)
            continue
        recs.extend(r for _sess, r in parts)
    table = np.concatenate(recs) if recs else np.zeros((0, 6), dtype=np.uint64)
    return table, unsupported, converts


def convert_staging_bytes(copies, sources: dict, fuse_casts: bool = False) -> int:
    """Size of the staging buffer ``plan_transfer_2d`` needs for dtype converts
    (``fuse_casts``: casts between the convert kernel's float dtypes are read in place)."""
    total = 0
    for copy in copies:
        src = sources.get(copy.src_name)
        if src is None:
            continue
        tbox = transposed_box(copy, src.global_shape)
        if tbox is not None:
            total = (total + 255) // 256 * 256 + int(np.prod(tbox[0])) * int(src.elsize)
        elif src.dtype != copy.dest_dtype and fuse_casts and str(src.dtype) in _FLOAT_KINDS and str(
                copy.dest_dtype) in _FLOAT_KINDS:
            continue
        elif src.dtype != copy.dest_dtype:
            n = int(np.prod(copy.dest_shape)) if len(copy.dest_shape) else 1
            total = (total + 255) // 256 * 256 + n * int(src.elsize)
    return total


_FLOAT_KINDS = {"torch.float32": "f32", "torch.float16": "f16", "torch.bfloat16": "bf16"}


def convert_box(c, staging_ptr: int, param) -> tuple | None:
    """The ``mxb_convert`` box of one ConvertSpec: ``(src, dst, extents, dst_strides, src_kind,
    dst_kind, elem_bytes)``, or ``None`` when the pair of dtypes is outside the kernel's table."""
    sk, dk = _FLOAT_KINDS.get(str(c.src_dtype)), _FLOAT_KINDS.get(str(param.dtype))
    elem = int(param.element_size())
    if c.src_dtype == param.dtype:
        if elem not in (1, 2, 4, 8):
            return None
        sk = dk = "raw"
    elif sk is None or dk is None:
        return None
    if c.box_shape is None:
        extents, strides = list(c.dest_shape), list(c.dest_stride)
    else:
        # the staged box keeps the source's dim order; destination dim d walks staging dim box_perm[d]
        extents = list(c.box_shape)
        strides = [0] * len(extents)
        for d, s_dim in enumerate(c.box_perm):
            if s_dim is not None:
                strides[s_dim] = int(c.dest_stride[d])
    if len(extents) > 8:
        return None
    return (staging_ptr + int(c.staging_offset), param.data_ptr() + int(c.dest_offset) * elem,
            extents, strides, sk, dk, elem)


def apply_converts(converts, staging, params: dict, ctx=None) -> None:
    """Cast (and, for staged boxes, transpose) the staged sources into their parameters
    (receiver.py:964-971).  On the GPU all of them go through one call of the box-convert
    kernel (one launch per pair of dtypes present); a pair of dtypes outside its table (and host tensors, which only the planner's own
    tests use) takes torch's strided copy."""
    import torch

    leftover = list(converts)
    if converts and staging.is_cuda:
        from ._lib import MxbError
        from .runtime import default_context

        ctx = ctx or default_context(staging.device.index)
        boxes, leftover = [], []
        for c in converts:
            if isinstance(c, DirectCast):
                boxes += [(c, b) for b in c.boxes]
                continue
            box = convert_box(c, staging.data_ptr(), params[c.param_name])
            if box is None:
                leftover.append(c)
            else:
                boxes.append((c, box))
        try:
            if boxes:
                torch.cuda.current_stream(staging.device).synchronize()   # the parameters may be torch's
                ctx.convert_boxes([b for _c, b in boxes], staging.device.index)
        except MxbError as e:
            if getattr(e, "code", None) != -9:   # MXB_ERR_UNSUPPORTED: more than four dims after merging
                raise
            for c, b in boxes:
                try:
                    ctx.convert_boxes([b], staging.device.index)
                except MxbError as e1:
                    if getattr(e1, "code", None) != -9 or isinstance(c, DirectCast):
                        raise
                    leftover.append(c)
    for c in leftover:
        src = staging[c.staging_offset: c.staging_offset + c.nbytes].view(c.src_dtype)
        if c.box_shape is None:
            src = src.reshape(c.dest_shape)
        else:
            # the staged box in the source's dim order -> the destination's: walked dims in
            # destination order first, the box's extent-1 dims last, then only size-1 dims differ
            walked = [s for s in c.box_perm if s is not None]
            rest = [d for d in range(len(c.box_shape)) if d not in walked]
            src = src.reshape(c.box_shape).permute(walked + rest).reshape(c.dest_shape)
        p = params[c.param_name]
        dst = torch.as_strided(p, c.dest_shape, c.dest_stride, p.storage_offset() + c.dest_offset)
        dst.copy_(src)
