"""The cp.async.bulk tile engine of the scatter kernel against the oracle."""

import numpy as np
import pytest

from make_golden import golden_bytes
from test_gpu_scatter import _run_both, env  # noqa: F401  (fixture)

pytestmark = pytest.mark.gpu


def test_bulk_engine_matches_vector_engine(env):
    ctx, torch = env
    from modelexpress_b200.runtime import SCATTER_DEFAULT, SCATTER_VECTOR

    rng = np.random.default_rng(9)
    src = golden_bytes(77, 24 << 20)
    recs, dpos = [], 0
    for _ in range(40):
        if rng.integers(0, 2):
            rows, rb = 1, 16 * int(rng.integers(64, 40_000))
            sp = dp = rb
        else:
            rows, rb = int(rng.integers(1, 300)), 16 * int(rng.integers(64, 600))
            sp, dp = rb + 16 * int(rng.integers(0, 40)), rb + 16 * int(rng.integers(0, 40))
        span_s, span_d = (rows - 1) * sp + rb, (rows - 1) * dp + rb
        s0 = 16 * int(rng.integers(0, (src.size - span_s) // 16))
        recs.append((s0, dpos, rows, rb, sp, dp))
        dpos += (span_d + 255) // 256 * 256
    got, want = _run_both(ctx, torch, src, dpos, recs, SCATTER_DEFAULT)
    assert np.array_equal(got, want)
    got2, _ = _run_both(ctx, torch, src, dpos, recs, SCATTER_VECTOR)
    assert np.array_equal(got2, want)
    tb = ctx.table([(1 << 20, 2 << 20, 4, 2048, 4096, 2048)])  # addresses only classified, never launched
    assert tb.engine(SCATTER_DEFAULT) == "bulk" and tb.engine(SCATTER_VECTOR) == "vector"
    tb.close()
    # a mixed table: most records qualify for bulk copies, some do not (odd offsets, short rows)
    mixed, pos = list(recs), dpos
    for k in range(12):
        rows, rb = int(rng.integers(1, 50)), int(rng.integers(1, 900))
        mixed.append((int(rng.integers(0, 1 << 20)) | 1, pos + 3, rows, rb, rb + 5, rb + 7))
        pos += 3 + rows * (rb + 7) + 64
    got3, want3 = _run_both(ctx, torch, src, pos, mixed, SCATTER_DEFAULT)
    assert np.array_equal(got3, want3)
    tb = ctx.table([(1 << 20, 2 << 20, 4, 2048, 4096, 2048), ((1 << 20) + 1, 3 << 20, 1, 64, 64, 64)])
    assert tb.engine(SCATTER_DEFAULT) == "bulk+vector"
    tb.close()
    assert ctx.launch_count > 0




def test_both_engines_side_by_side(env):
    """MXB_SCATTER_OVERLAP: a table with hundreds of tiles for each engine runs the
    bulk kernel and the vector kernel as two concurrent launches; same bytes."""
    ctx, torch = env
    from modelexpress_b200.runtime import SCATTER_DEFAULT, SCATTER_OVERLAP

    rng = np.random.default_rng(21)
    src = golden_bytes(78, 96 << 20)
    recs, dpos = [], 0
    for k in range(24):      # 24 x 2 MiB aligned (bulk engine) + 24 x ~2 MiB at odd offsets (vector engine)
        rows, rb = 512, 4096
        s0 = 16 * int(rng.integers(0, (src.size - rows * 8192) // 16))
        recs.append((s0, dpos, rows, rb, 8192, 4096))
        dpos += rows * 4096
        rows, rb = 500, 4099
        s1 = int(rng.integers(0, src.size - rows * 8200)) | 1
        recs.append((s1, dpos + 5, rows, rb, 8200, 4112))
        dpos += (5 + rows * 4112 + 255) // 256 * 256
    want = None
    for flags in (SCATTER_DEFAULT, SCATTER_OVERLAP, SCATTER_OVERLAP):
        got, want = _run_both(ctx, torch, src, dpos, recs, flags)
        assert np.array_equal(got, want)
