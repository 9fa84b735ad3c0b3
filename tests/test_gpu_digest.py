"""Digest kernel against the reference-generated golden values and the oracle."""

import json
import os

import numpy as np
import pytest

from make_golden import golden_bytes
from oracle import c_port as C
from oracle import ref_port as R
from test_oracle_golden import digest_case_bytes

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def torch_mod():
    import torch

    assert torch.cuda.is_available()
    return torch


@pytest.mark.parametrize("engine", ["vector", "bulk"])
def test_golden_digests_through_the_kernel(torch_mod, engine, monkeypatch):
    """Both tile engines (the default vector one and the shared-memory-staged one
    that MXB_DIGEST_ENGINE=bulk selects for full tiles of aligned ranges)."""
    torch = torch_mod
    from modelexpress_b200 import digest

    monkeypatch.setenv("MXB_DIGEST_ENGINE", engine)

    cases = json.load(open(os.path.join(G, "digests.json")))
    tensors = [torch.from_numpy(digest_case_bytes(c).copy()).cuda() for c in cases]
    res = digest.digest_many(tensors)  # one launch for all of them
    for c, r, t in zip(cases, res, tensors):
        b = digest_case_bytes(c)
        assert r["safe_checksum"] == c["safe_checksum"], c
        if c["tensor_digest"] is not None:
            assert r["tensor_digest"] == c["tensor_digest"], c
        else:  # the reference raises below one word; the kernel follows the oracle's extension
            assert r["tensor_digest"] == R.tensor_digest(b)
        assert r["block_hash64"] == R.block_hash64(b) == C.block_hash64(b), c
    # single-tensor entry points, same names and return types as the reference
    assert digest.safe_checksum(torch.arange(16, dtype=torch.bfloat16).cuda()) == "59cd2bf4"
    assert digest.tensor_digest(torch.arange(4096, dtype=torch.int32).cuda()) == \
        "b80e42d0aa211223be9669385be8976b"
    with pytest.raises(RuntimeError):
        digest.safe_checksum(torch.zeros(4))  # CPU tensor: no fallback


@pytest.mark.parametrize("engine", ["vector", "bulk"])
def test_large_seeded_tensor_matches_oracle(torch_mod, engine, monkeypatch):
    torch = torch_mod
    from modelexpress_b200 import digest

    monkeypatch.setenv("MXB_DIGEST_ENGINE", engine)

    b = golden_bytes(42, (64 << 20) + 4096 * 3 + 1234 * 4 + 3)
    t = torch.from_numpy(b).cuda()
    r = digest.digest_many([t])[0]
    assert r["safe_checksum"] == C.safe_checksum(b, mt=True)
    assert r["tensor_digest"] == R.digest_from_scalars(C.digest_scalars(b, mt=True))
    assert r["block_hash64"] == C.block_hash64(b)


def test_reference_digest_properties(torch_mod):
    """tests/test_reshard_refit_verify.py:43-171 of the reference, on the kernel."""
    torch = torch_mod
    from modelexpress_b200.digest import tensor_digest

    a = torch.arange(4096, dtype=torch.int32).cuda()
    assert tensor_digest(a) == tensor_digest(a.clone())
    b = a.clone()
    b[1234] += 1
    assert tensor_digest(a) != tensor_digest(b)
    a = torch.arange(8192, dtype=torch.int32).cuda()
    b = a.clone()
    b[0:1024], b[1024:2048] = a[1024:2048].clone(), a[0:1024].clone()
    assert a.sum() == b.sum()
    assert tensor_digest(a) != tensor_digest(b)
    a = torch.arange(1024 + 7, dtype=torch.int16).cuda()
    b = a.clone()
    b[-1] += 1
    assert tensor_digest(a) != tensor_digest(b)
    dense = torch.arange(64, dtype=torch.int32).reshape(8, 8).cuda()
    assert tensor_digest(dense[:, ::2]) == tensor_digest(dense[:, ::2].contiguous())


@pytest.mark.parametrize("half", [1409, 17])
def test_unaligned_views_digest_like_their_copies(torch_mod, half):
    """Odd bf16 splits start 2 bytes off a word boundary: the kernel reads them in
    place and must agree with the rebased copy the reference makes."""
    torch = torch_mod
    from modelexpress_b200 import digest

    fused = torch.arange(2 * half, dtype=torch.bfloat16).cuda()
    view = fused.narrow(0, half, half)
    assert (view.storage_offset() * view.element_size()) % 4
    r_view, r_copy = digest.digest_many([view, view.clone()])
    assert r_view == r_copy
    want = R.tensor_digest(view.cpu().view(torch.int16).numpy())
    assert r_view["tensor_digest"] == want
    # every byte offset, checked against the oracle
    raw = torch.from_numpy(golden_bytes(8, 70_000)).cuda()
    host = raw.cpu().numpy()
    views = [raw[o:o + 65_000 + o] for o in range(0, 8)]
    for o, r in enumerate(digest.digest_many(views)):
        hb = host[o:o + 65_000 + o]
        assert r["safe_checksum"] == R.safe_checksum(hb)
        assert r["tensor_digest"] == R.tensor_digest(hb)
        assert r["block_hash64"] == R.block_hash64(hb)


def test_block_hash_array(torch_mod):
    torch = torch_mod
    from modelexpress_b200.runtime import default_context

    b = golden_bytes(9, 10 * 4096 + 100)
    t = torch.from_numpy(b).cuda()
    out = torch.zeros(11, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    default_context(0).block_hashes(t.data_ptr(), t.numel(), out.data_ptr(), 0)
    got = out.cpu().numpy().view(np.uint64)
    assert np.array_equal(got, R.block_hashes64(b))
