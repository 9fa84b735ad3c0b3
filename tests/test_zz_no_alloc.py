"""The allocation-free digest entry point against the ordinary one.

Some hosts of this library may not allocate device memory at all (an inference
engine whose KV cache already owns every free byte of HBM, for one), so
``mxb_digest_noalloc`` works out of a fixed array inside the library.  This
test calls it through the C ABI twice in a row on different data and checks
every field against ``mxb_digest``; the second call also proves that what the
first call left in the shared array does not leak into the next result.  The
second round also reads the device's free memory immediately before and after
the allocation-free calls (the first round has loaded every kernel they use):
the figure must not move.  It is collected last on purpose."""

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _records_equal(a, b):
    fields = ("nbytes", "row_sum", "row_sum_w", "tail_sum", "tail_sum_w", "ragged_sum", "block_hash",
              "safe_checksum")
    return all(int(getattr(a, f)) == int(getattr(b, f)) for f in fields)


def test_noalloc_digest_matches_the_allocating_entry_point():
    import torch

    from make_golden import golden_bytes
    from modelexpress_b200 import _lib
    from modelexpress_b200.runtime import Context

    assert torch.cuda.is_available()
    lib = _lib.load()
    ctx = Context([0])
    for call, seed in enumerate((301, 302)):
        sizes = [5 << 20, 4096 * 3 + 7, 65536, 1, 0, (1 << 20) + 4 * 511 + 2, 100_000 + call]
        bufs = [torch.from_numpy(golden_bytes(seed + i, n)).cuda() for i, n in enumerate(sizes)]
        views = bufs + [bufs[0][3:70_003]]  # an unaligned view as well
        torch.cuda.synchronize()
        spans = [(v.data_ptr() if v.numel() else 0, v.numel()) for v in views]
        want = ctx.digest(spans, 7, 0)
        arr, n = _lib.span_array(spans)
        out = (_lib.DigestOut * n)()
        out2 = (_lib.DigestOut * n)()
        s = torch.cuda.Stream()
        torch.cuda.synchronize()
        # nothing between the two readings allocates on the host side of this test either
        free_before = torch.cuda.mem_get_info(0)[0]
        rc = lib.mxb_digest_noalloc(0, arr, n, 7, out, None)
        # on a caller-provided stream too
        rc2 = lib.mxb_digest_noalloc(0, arr, n, 2, out2, ctypes.c_void_p(s.cuda_stream))
        free_after = torch.cuda.mem_get_info(0)[0]
        assert rc == 0 and rc2 == 0, lib.mxb_last_error()
        if call == 1:   # the first call loaded the kernels; from here on the device's free memory must not move
            assert free_after == free_before, (free_before, free_after)
        for i in range(n):
            assert _records_equal(out[i], want[i]), (call, i, sizes[i] if i < len(sizes) else "view")
        for i in range(n):
            assert int(out2[i].row_sum) == int(want[i].row_sum)
            assert int(out2[i].row_sum_w) == int(want[i].row_sum_w)
    # sizes beyond the fixed scratch are refused with a clear message, nothing is queued
    big = torch.empty(1, dtype=torch.uint8, device="cuda")
    arr, n = _lib.span_array([(big.data_ptr(), (1 << 30) + 65536)])
    out = (_lib.DigestOut * 1)()
    assert lib.mxb_digest_noalloc(0, arr, 1, 1, out, None) == -1
    assert b"exceed the fixed scratch" in lib.mxb_last_error()
    arr, n = _lib.span_array([(big.data_ptr(), 1)] * 257)
    out = (_lib.DigestOut * 257)()
    assert lib.mxb_digest_noalloc(0, arr, 257, 1, out, None) == -1
    assert b"at most 256" in lib.mxb_last_error()
    del bufs, views, big
    torch.cuda.synchronize()
    ctx.close()
