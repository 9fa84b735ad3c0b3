"""The C-ABI library loads without a GPU and exports every declared symbol."""

import ctypes
import os
import re

import numpy as np
import pytest

from modelexpress_b200 import _lib, build
from modelexpress_b200.runtime import coalesce_runs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def _declared():
    text = open(os.path.join(ROOT, "include", "mxb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mxb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = _declared()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in mxb200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes table and header disagree"


def test_struct_sizes_match_the_header(lib):
    assert ctypes.sizeof(_lib.Run) == 24
    assert ctypes.sizeof(_lib.Desc2D) == 48
    assert ctypes.sizeof(_lib.Span) == 16
    assert ctypes.sizeof(_lib.DigestOut) == 64
    assert lib.mxb_version() == 1


def test_compute_entry_points_fail_loudly_without_a_device(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    h = ctypes.c_void_p()
    ids = (ctypes.c_int32 * 1)(0)
    rc = lib.mxb_ctx_create(ids, 1, ctypes.byref(h))
    assert rc == -4  # MXB_ERR_CUDA, never a silent CPU path
    assert lib.mxb_last_error()


def test_coalesce_folds_strided_runs_and_round_trips():
    rng = np.random.default_rng(0)
    runs = []
    # a row-parallel slice: 64 runs of 48 bytes, src pitch 384, dst pitch 48 -> one record
    runs += [(10_000 + r * 384, 50_000 + r * 48, 48) for r in range(64)]
    # fused destination with a wider pitch
    runs += [(90_000 + r * 100, 70_000 + r * 160, 100) for r in range(5)]
    # a lone run, an empty run, an irregular pair
    runs += [(1, 2, 3), (7, 7, 0), (500, 900, 8), (520, 940, 8), (555, 1000, 8)]
    recs = coalesce_runs(runs)
    expanded = []
    for src, dst, rows, rb, sp, dp in recs.tolist():
        expanded += [(src + r * sp, dst + r * dp, rb) for r in range(rows)]
    flat = []
    for s, d, n in expanded:
        flat.append((s, d, n))
    want = [r for r in runs if r[2]]
    # records may merge back-to-back rows into one longer row: compare byte maps
    def byte_map(rs):
        m = {}
        for s, d, n in rs:
            for k in range(n):
                m[d + k] = s + k
        return m
    assert byte_map(flat) == byte_map(want)
    assert len(recs) < len(want)
    assert tuple(recs[0]) == (10_000, 50_000, 64, 48, 384, 48)
    # random stress
    for _ in range(20):
        n = int(rng.integers(1, 40))
        rr = [(int(rng.integers(1, 1 << 20)), int(rng.integers(1, 1 << 20)), int(rng.integers(0, 64)))
              for _ in range(n)]
        recs = coalesce_runs(rr)
        exp = []
        for src, dst, rows, rb, sp, dp in recs.tolist():
            exp += [(src + r * sp, dst + r * dp, rb) for r in range(rows)]
        assert sorted(exp) == sorted(x for x in rr if x[2])


def test_vllm_import_path_shim_exposes_the_loader_class():
    """vLLM imports modelexpress.engines.vllm.loader:MxModelLoader; the shim directory
    must expose our class there with the reference's entry points."""
    import importlib
    import sys

    shim = os.path.join(ROOT, "modelexpress_b200", "shim")
    sys.path.insert(0, shim)
    try:
        mod = importlib.import_module("modelexpress.engines.vllm.loader")
        cls = mod.MxModelLoader
        for name in ("load_model", "download_model", "load_weights", "nixl_manager", "tensors"):
            assert hasattr(cls, name), name
        assert cls.__module__ == "modelexpress_b200.engines.vllm.loader"
    finally:
        sys.path.remove(shim)
        for k in [k for k in sys.modules if k == "modelexpress" or k.startswith("modelexpress.")]:
            del sys.modules[k]


# ---------------------------------------------------------------------------
# the descriptor compiler behind the C ABI (mxb_plan_pull / mxb_plan_reshard)
# ---------------------------------------------------------------------------


def _window_of(case):
    """Replay the case's op-chain (host side, as a binding would) into a strided window."""
    from modelexpress_b200 import planner
    from test_oracle_golden import _chain

    view = planner._View(case["global_shape"])
    for op, args, _kw in _chain(case["op_chain"]):
        view.apply(op, args)
    return view.offset, view.shape, view.stride


def _golden_cases():
    from test_oracle_golden import _load

    return _load("slice_plan.json")


@pytest.mark.parametrize("case", _golden_cases(), ids=lambda c: c["tag"])
def test_plan_pull_through_the_abi_expands_to_the_reference_runs(lib, case):
    """tests/golden/slice_plan.json holds the reference's own plan_pull output (62 cases,
    the reference tests' hand-computed ones among them): the C planner's records,
    expanded row by row, must be those runs in that order."""
    from modelexpress_b200 import planner
    from modelexpress_b200._lib import MxbError
    from modelexpress_b200.runtime import plan_pull

    try:
        off, shape, stride = _window_of(case)
    except planner.UnsupportedReshard:
        assert case["error"]          # the op-chain itself is not a view: nothing reaches the ABI
        return
    shards = [(tuple(o), tuple(s), addr) for o, s, _sess, addr in case["shards"]]
    sessions = [sess for _o, _s, sess, _a in case["shards"]]
    rank_ok = len(shape) == len(case["dest_shape"]) and tuple(shape) == tuple(case["dest_shape"])
    if case["error"]:
        if rank_ok:
            with pytest.raises(MxbError) as e:
                plan_pull(case["global_shape"], case["elsize"], off, shape, stride, case["dest_offset"],
                          case["dest_stride"], shards, 0)
            assert e.value.code == -9
        return
    recs, which = plan_pull(case["global_shape"], case["elsize"], off, shape, stride, case["dest_offset"],
                            case["dest_stride"], shards, 0)
    got = []
    for rec, k in zip(recs.tolist(), which.tolist()):
        src, dst, rows, rb, sp, dp = rec
        got += [[sessions[k], src + r * sp, dst + r * dp, rb] for r in range(rows)]
    assert got == case["segments"]


def test_plan_pull_agrees_with_the_python_planner_on_random_windows(lib):
    from modelexpress_b200 import planner
    from modelexpress_b200._lib import MxbError
    from modelexpress_b200.runtime import plan_pull

    rng = np.random.default_rng(7)
    checked = refused = 0
    for _ in range(400):
        nd = int(rng.integers(1, 5))
        gshape = [int(rng.integers(1, 7)) for _ in range(nd)]
        view = planner._View(gshape)
        for _op in range(int(rng.integers(0, 4))):
            kind = rng.integers(0, 3)
            if kind == 0:
                d = int(rng.integers(0, nd))
                if view.shape[d] == 0:
                    continue
                start = int(rng.integers(0, view.shape[d]))
                size = int(rng.integers(1, view.shape[d] - start + 1))
                view.apply("narrow", (d, start, size))
            elif kind == 1 and nd >= 2:
                a, b = (int(x) for x in rng.choice(nd, 2, replace=False))
                view.apply("transpose", (a, b))
            elif kind == 2:
                view.apply("permute", (tuple(int(x) for x in rng.permutation(nd)),))
        dest_shape = tuple(view.shape)
        dstride = planner._strides_of([s + int(rng.integers(0, 3)) for s in dest_shape])
        dest_off = int(rng.integers(0, 5))
        el = int(rng.choice([1, 2, 4]))
        # shards: split dim 0 of the source in two (or one shard)
        cut = int(rng.integers(0, gshape[0] + 1))
        boxes = [((0,) * nd, tuple([cut] + gshape[1:]), 4096), ((cut,) + (0,) * (nd - 1),
                 tuple([gshape[0] - cut] + gshape[1:]), 1 << 20)]
        boxes = [b for b in boxes if b[1][0] > 0]
        copy = planner.CopySpec("s", (), "p", dest_off, dest_shape, tuple(dstride), "dt")
        copy.src_offset, copy.src_shape, copy.src_stride = view.offset, tuple(view.shape), tuple(view.stride)
        shard_specs = [planner.ShardSpec(o, s, f"s{k}", a, el) for k, (o, s, a) in enumerate(boxes)]
        try:
            want = planner.plan_pull_2d(copy, gshape, "dt", el, shard_specs, 1 << 30)
        except planner.UnsupportedReshard:
            with pytest.raises(MxbError):
                plan_pull(gshape, el, view.offset, view.shape, view.stride, dest_off, dstride, boxes,
                          1 << 30, keep_rank=False)
            refused += 1
            continue
        recs, _which = plan_pull(gshape, el, view.offset, view.shape, view.stride, dest_off, dstride, boxes,
                                 1 << 30, keep_rank=False)
        flat = np.concatenate([r for _s, r in want]) if want else np.zeros((0, 6), dtype=np.uint64)
        assert planner.expand_records(recs) == planner.expand_records(flat)
        checked += 1
    assert checked > 200


def test_plan_reshard_agrees_with_the_python_clip(lib):
    from modelexpress_b200 import reshard
    from modelexpress_b200.runtime import plan_reshard

    rng = np.random.default_rng(11)
    for _ in range(500):
        rows = int(rng.integers(1, 40))
        rb = int(rng.integers(1, 300))
        sp = rb + int(rng.integers(0, 200)) if rows > 1 else rb
        dp = rb + int(rng.integers(0, 64)) if rows > 1 else rb
        so = int(rng.integers(0, 500))
        total = so + (rows - 1) * sp + rb + int(rng.integers(0, 100))
        lo = int(rng.integers(0, total))
        hi = int(rng.integers(lo, total + 1))
        dst0 = 1 << 20
        want = reshard.clip_records(so, 0, rows, rb, sp, dp, lo, hi, 5000, dst0)
        got = plan_reshard([(so, dst0, rows, rb, sp, dp)], lo, hi, 5000)
        from modelexpress_b200.planner import expand_records

        assert expand_records(got) == expand_records(np.array(want, dtype=np.uint64).reshape(-1, 6)), \
            (so, rows, rb, sp, dp, lo, hi)
    # splitting keeps the byte map
    big = plan_reshard([(0, 1 << 20, 1, 1 << 22, 1 << 22, 1 << 22), (64, 1 << 30, 100, 4096, 8192, 4096)],
                       0, 1 << 23, 0, max_record_bytes=1 << 20)
    whole = plan_reshard([(0, 1 << 20, 1, 1 << 22, 1 << 22, 1 << 22), (64, 1 << 30, 100, 4096, 8192, 4096)],
                         0, 1 << 23, 0)
    assert len(big) > len(whole) and int((big[:, 2] * big[:, 3]).max()) <= 1 << 20
    assert int((big[:, 2] * big[:, 3]).sum()) == int((whole[:, 2] * whole[:, 3]).sum())


def test_fanout_plan_piece_sizes():
    """``mxb_fanout_plan_pieces`` (host only): pieces tile every range exactly once, stay inside
    the chunk they start in (but for a 16-byte alignment piece) and within the piece size, start on 16-byte boundaries inside their range, and only a
    range's last piece is ragged; the plan depends on the sizes alone."""
    import pytest

    from modelexpress_b200 import _lib
    from modelexpress_b200.fanout import plan_pieces

    sizes = [3 << 20, 4096 + 16, 100, 333 * 16, 1 << 20, 52, 700_000, 0, 48]
    for chunk, piece in ((1 << 20, 64 << 10), (1 << 20, 256 << 10), (256 << 10, 256 << 10), (64 << 10, 64 << 10),
                         (64 << 10, 256 << 10), (4096, 4096)):
        pieces, per_chunk = plan_pieces(sizes, chunk, piece)
        assert sum(per_chunk) == len(pieces)
        at, vpos = [0] * len(sizes), 0
        for rng, off, n, ch in pieces:
            assert off == at[rng] and 0 < n <= min(piece, chunk) and off % 16 == 0
            # a piece belongs to the chunk it starts in; only a 16-byte piece that keeps a range's
            # 16-byte phase may reach past the chunk's end
            assert vpos // chunk == ch and ((vpos + n - 1) // chunk == ch or n <= 16)
            assert n % 16 == 0 or off + n == sizes[rng]                     # only a last piece is ragged
            at[rng] += n
            vpos += n
        assert at == sizes
        if piece >= chunk:
            assert all(c >= 1 for c in per_chunk)
    assert plan_pieces(sizes, 1 << 20) == plan_pieces(sizes, 1 << 20, 64 << 10)   # the default piece
    for bad in (100, 2 << 20, 65536 + 8):
        with pytest.raises(_lib.MxbError):
            plan_pieces(sizes, 1 << 20, bad)
