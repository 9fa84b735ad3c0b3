"""Sizes past 2^32 bytes: 64-bit offsets in the tile tables, the digest's row
index weights and the safe_checksum byte index (which wraps mod 2^32 by
definition).  Checked against the oracle's C loops."""

import numpy as np
import pytest

from oracle import c_port as C
from oracle import ref_port as R

pytestmark = pytest.mark.gpu

BIG = (4 << 30) + (300 << 20) + 4096 * 5 + 7  # 4.3 GiB, ragged


def test_digest_and_scatter_beyond_4_gib():
    import torch

    from modelexpress_b200.runtime import Context

    free, _total = torch.cuda.mem_get_info(0)
    if free < 3 * BIG:
        pytest.skip("not enough free device memory")
    ctx = Context([0])
    g = torch.Generator(device="cuda")
    g.manual_seed(11)
    src = torch.randint(0, 256, (BIG,), dtype=torch.uint8, device="cuda", generator=g)
    torch.cuda.synchronize()
    host = src.cpu().numpy()
    rec = ctx.digest([(src.data_ptr(), BIG)], 7, 0)[0]
    assert format(int(rec.safe_checksum), "08x") == C.safe_checksum(host, mt=True)
    sc = C.digest_scalars(host, mt=True)
    assert [int(rec.nbytes), int(rec.row_sum), int(rec.row_sum_w), int(rec.tail_sum),
            int(rec.tail_sum_w), int(rec.ragged_sum), BIG % 4] == sc
    assert int(rec.block_hash) == C.block_hash64(host)

    # one contiguous record of 4.3 GiB and one strided record whose rows sum past 2^32
    dst = torch.zeros(BIG, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    ctx.scatter([(src.data_ptr(), dst.data_ptr(), 1, BIG, BIG, BIG)], 0)
    got = ctx.digest([(dst.data_ptr(), BIG)], 4, 0)[0]
    assert int(got.block_hash) == int(rec.block_hash)
    dst.zero_()
    torch.cuda.synchronize()  # the library runs on its own stream: order the fill before it
    rows, rb, sp = 70_000, 32_768, 65_536           # 2.3 GB moved, source span 4.6 GB > BIG? keep inside
    rows = min(rows, (BIG - rb) // sp)
    ctx.scatter([(src.data_ptr(), dst.data_ptr(), rows, rb, sp, rb)], 0)
    want = host[: rows * sp].reshape(rows, sp)[:, :rb].reshape(-1)
    assert np.array_equal(dst[: rows * rb].cpu().numpy(), want)
    del src, dst
    ctx.close()
