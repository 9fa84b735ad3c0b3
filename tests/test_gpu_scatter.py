"""Scatter kernel (through the C ABI) against the oracle's memmove loops."""

import ctypes

import numpy as np
import pytest

from make_golden import golden_bytes
from oracle import c_port as C
from oracle import ref_port as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch

    from modelexpress_b200.runtime import Context

    assert torch.cuda.is_available()
    ctx = Context([0])
    yield ctx, torch
    ctx.close()


def _run_both(ctx, torch, src_np, dst_size, recs_rel, flags=0):
    """recs_rel: records with offsets relative to src/dst buffers.  Runs the
    CUDA path on device copies and the oracle on host copies; returns both."""
    src_d = torch.from_numpy(src_np.copy()).cuda()
    dst_d = torch.full((dst_size,), 0xA5, dtype=torch.uint8, device="cuda")
    dst_h = np.full(dst_size, 0xA5, dtype=np.uint8)
    torch.cuda.synchronize()
    dev = [(src_d.data_ptr() + s, dst_d.data_ptr() + d, r, rb, sp, dp) for s, d, r, rb, sp, dp in recs_rel]
    host = [(src_np.ctypes.data + s, dst_h.ctypes.data + d, r, rb, sp, dp) for s, d, r, rb, sp, dp in recs_rel]
    ctx.scatter(dev, 0, flags)
    C.scatter2d(host)
    return dst_d.cpu().numpy(), dst_h


def test_row_parallel_slice_is_byte_exact(env):
    ctx, torch = env
    rows, cols, tp, rank = 512, 4096, 8, 3
    src = golden_bytes(1, rows * cols * 2)
    loc = cols // tp * 2
    recs = [(rank * loc, 0, rows, loc, cols * 2, loc)]
    got, want = _run_both(ctx, torch, src, rows * loc, recs)
    assert np.array_equal(got, want)
    full = src.view(np.uint16).reshape(rows, cols)
    assert np.array_equal(got.view(np.uint16).reshape(rows, cols // tp),
                          full[:, rank * cols // tp:(rank + 1) * cols // tp])


def test_fused_qkv_destination_offsets(env):
    ctx, torch = env
    h = 1024
    q, k, v = 512, 128, 128
    src = golden_bytes(2, (q + k + v) * 8 * h * 2)  # full q|k|v stacked, tp=8
    rank, el = 5, 2
    recs, off, soff = [], 0, 0
    for n in (q, k, v):
        recs.append((soff + rank * n * h * el, off, 1, n * h * el, n * h * el, n * h * el))
        off += n * h * el
        soff += n * 8 * h * el
    got, want = _run_both(ctx, torch, src, (q + k + v) * h * el, recs)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("seed", range(6))
def test_random_tables_any_alignment(env, seed):
    """Ragged sizes, odd offsets, pitches that are not multiples of 16, empty
    records, rows longer than a tile, single-byte rows."""
    ctx, torch = env
    rng = np.random.default_rng(seed)
    src = golden_bytes(100 + seed, 6 << 20)
    recs, dpos = [], 0
    for _ in range(60):
        kind = int(rng.integers(0, 6))
        if kind == 0:   # long contiguous, arbitrary alignment
            rows, rb = 1, int(rng.integers(1, 300_000))
            sp = dp = rb
        elif kind == 1:  # short strided rows
            rows, rb = int(rng.integers(1, 400)), int(rng.integers(1, 700))
            sp, dp = rb + int(rng.integers(0, 50)), rb + int(rng.integers(0, 50))
        elif kind == 2:  # aligned strided rows
            rows, rb = int(rng.integers(1, 200)), 16 * int(rng.integers(1, 300))
            sp, dp = rb + 16 * int(rng.integers(0, 9)), rb + 16 * int(rng.integers(0, 9))
        elif kind == 3:  # empty
            rows, rb, sp, dp = int(rng.integers(0, 2)), 0, 0, 0
        elif kind == 4:  # rows between 8 KiB and a tile
            rows, rb = int(rng.integers(1, 6)), int(rng.integers(8193, 70_000))
            sp, dp = rb + int(rng.integers(0, 33)), rb + int(rng.integers(0, 33))
        else:            # bytes
            rows, rb = int(rng.integers(1, 40)), int(rng.integers(1, 4))
            sp, dp = rb + int(rng.integers(0, 3)), rb + int(rng.integers(0, 3))
        span_s = (rows - 1) * sp + rb if rows and rb else 0
        span_d = (rows - 1) * dp + rb if rows and rb else 0
        s0 = int(rng.integers(0, src.size - span_s - 1)) if span_s else 0
        d0 = dpos + int(rng.integers(0, 17))
        recs.append((s0, d0, rows, rb, sp, dp))
        dpos = d0 + span_d
    got, want = _run_both(ctx, torch, src, dpos + 64, recs)
    assert np.array_equal(got, want)


def test_transport_read_matches_reference_memmove(env):
    """Transport.read(descriptors) seam: same bytes as the reference's ctypes loop."""
    ctx, torch = env
    from modelexpress_b200.transport import MxbTransport, ReadDescriptor, Transport

    src = golden_bytes(5, 1 << 20)
    src_d = torch.from_numpy(src.copy()).cuda()
    dst_d = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    dst_h = np.zeros(1 << 20, dtype=np.uint8)
    rng = np.random.default_rng(5)
    rel, pos = [], 0
    for _ in range(300):
        n = int(rng.integers(0, 3000))
        s = int(rng.integers(0, src.size - n))
        rel.append((s, pos, n))
        pos += n + int(rng.integers(0, 9))
    # plus a strided slice as the reference emits it: one run per row
    rel += [(4096 + r * 512, pos + r * 64, 64) for r in range(256)]
    torch.cuda.synchronize()
    t = MxbTransport(ctx, 0)
    assert isinstance(t, Transport)
    t.read([ReadDescriptor("s", src_d.data_ptr() + s, dst_d.data_ptr() + d, n) for s, d, n in rel])
    R.memmove_read([R.ReadDescriptor("s", src.ctypes.data + s, dst_h.ctypes.data + d, n) for s, d, n in rel])
    assert np.array_equal(dst_d.cpu().numpy(), dst_h)
    assert t.bytes_moved == sum(n for _s, _d, n in rel)
    assert t.reads_issued == sum(1 for _s, _d, n in rel if n)
    t.read([])  # empty batch is a no-op
    with pytest.raises(KeyError):
        MxbTransport(ctx, 0, sessions={"a": 1}).read([ReadDescriptor("b", 1, 2, 3)])


def test_toy_model_reshard_through_the_transport(env):
    """The reference's strongest check (tests/test_reshard_refit_transfer.py:71-124):
    parameters rebuilt from shards alone equal the loader's ground truth — here with
    the reference's captured copies (fixture), planned as 2-D records and moved by
    the CUDA transport."""
    import json
    import os

    ctx, torch = env
    from modelexpress_b200 import planner
    from test_oracle_golden import _chain

    g = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "toy_reshard.json")))
    shapes = {n: tuple(s) for n, s in g["manifest"]}
    srcs, base = {}, 0.0
    for name, shape in shapes.items():
        n = int(np.prod(shape))
        srcs[name] = (base + torch.arange(n, dtype=torch.float32)).reshape(shape).cuda()
        base += n
    for nsplit in (1, 2):
        params = {n: torch.zeros(s, dtype=torch.float32, device="cuda") for n, s in g["param_shapes"].items()}
        sources, keep = {}, []
        for name, t in srcs.items():
            per = t.shape[0] // nsplit
            shards = []
            for s in range(nsplit):
                piece = t[s * per:(s + 1) * per].contiguous()
                keep.append(piece)
                shards.append(planner.ShardSpec((s * per,) + (0,) * (t.dim() - 1), tuple(piece.shape),
                                                f"{name}#{s}", piece.data_ptr(), 4))
            sources[name] = planner.SourceSpec(tuple(t.shape), "f32", 4, shards)
        copies = [planner.CopySpec(c["src_name"], _chain(c["op_chain"]), c["param_name"], c["dest_offset"],
                                   tuple(c["dest_shape"]), tuple(c["dest_stride"]), "f32") for c in g["copies"]]
        table, unsupported, converts = planner.plan_transfer_2d(copies, sources, lambda n: params[n].data_ptr())
        assert converts == []
        assert unsupported == []
        torch.cuda.synchronize()
        ctx.scatter(table, 0)
        for n, truth in g["truth"].items():
            assert params[n].reshape(-1).cpu().tolist() == truth, n


def test_bad_tables_are_rejected_before_launch(env):
    ctx, torch = env
    from modelexpress_b200._lib import MxbError

    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    with pytest.raises(MxbError, match="null address"):
        ctx.scatter([(0, p, 1, 16, 16, 16)], 0)
    with pytest.raises(MxbError, match="pitch"):
        ctx.scatter([(p, p + 2048, 4, 64, 32, 64)], 0)
    ctx.register_extent(p, 1024)
    try:
        with pytest.raises(MxbError, match="outside the registered extents"):
            ctx.scatter([(p, p + 1000, 1, 64, 64, 64)], 0)
        ctx.scatter([(p + 2048, p, 1, 64, 64, 64)], 0)  # inside: accepted
    finally:
        ctx.clear_extents()
    ctx.scatter([], 0)  # empty table


def test_resident_table_replays(env):
    ctx, torch = env
    src = torch.from_numpy(golden_bytes(3, 1 << 20)).cuda()
    dst = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    tb = ctx.table([(src.data_ptr(), dst.data_ptr(), 256, 2048, 4096, 2048)], 0)
    assert tb.nbytes == 256 * 2048
    ctx.event_record(0, 0)
    for _ in range(3):
        tb.launch()
    ctx.event_record(1, 0)
    assert ctx.event_elapsed_ms(0, 1, 0) > 0
    ctx.sync(0)
    want = src.cpu().numpy().reshape(256, 4096)[:, :2048].reshape(-1)
    assert np.array_equal(dst.cpu().numpy()[: want.size], want)
    tb.close()


def test_convert_sources_are_staged_then_cast(env):
    """A bf16-served source feeding an fp32 parameter (the router case of
    refit/reshard/receiver.py:964-971): bytes move as bf16 into staging through the
    kernel, the cast is the only step left to torch; result equals a direct cast."""
    ctx, torch = env
    from modelexpress_b200 import planner

    src = torch.randn(8, 16, dtype=torch.float32, device="cuda").to(torch.bfloat16)
    halves = [src[:4].contiguous(), src[4:].contiguous()]
    shards = [planner.ShardSpec((i * 4, 0), (4, 16), f"t{i}", h.data_ptr(), 2) for i, h in enumerate(halves)]
    sources = {"gate.weight": planner.SourceSpec((8, 16), torch.bfloat16, 2, shards)}
    param = torch.zeros(6, 16, dtype=torch.float32, device="cuda")
    copy = planner.CopySpec("gate.weight", (("narrow", (0, 1, 6), ()),), "gate", 0, (6, 16), (16, 1),
                            torch.float32)
    nbytes = planner.convert_staging_bytes([copy], sources)
    staging = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    table, unsupported, converts = planner.plan_transfer_2d(
        [copy], sources, lambda n: param.data_ptr(), convert_base=staging.data_ptr())
    assert unsupported == [] and len(converts) == 1
    ctx.scatter(table, 0)
    planner.apply_converts(converts, staging, {"gate": param})
    assert torch.equal(param, src[1:7].to(torch.float32))  # a widening cast is exact
