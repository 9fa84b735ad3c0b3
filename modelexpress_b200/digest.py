"""Integrity digests computed by the sm_100a digest kernel.

``safe_checksum`` and ``tensor_digest`` take a CUDA tensor and return exactly
the strings the reference's functions of the same names return for the same
bytes (tensor_utils.py:27-44, refit/reshard/verify.py:79-155): the kernel
produces the integer reductions, the host formats them (``%08x``, blake2b-128
of the little-endian scalars).  ``digest_many`` does a whole list of tensors in
one launch, which is what a refit with thousands of shards needs.
"""

from __future__ import annotations

import hashlib

from .runtime import DIGEST_BLOCK64, DIGEST_ROWS, DIGEST_SAFE32, Context, default_context

_U64 = (1 << 64) - 1
ROW_WORDS = 1024


def _flat_cuda(tensor):
    import torch

    t = tensor.detach()
    if not t.is_cuda:
        raise RuntimeError("modelexpress_b200.digest works on CUDA tensors only (no CPU fallback)")
    if t.dim() == 0:
        t = t.unsqueeze(0)
    flat = t.reshape(-1)
    if not flat.is_contiguous():
        flat = flat.contiguous()
    return flat.view(torch.uint8) if flat.numel() else flat


def scalars_from_record(rec) -> list:
    """The scalar list verify.py:113-150 feeds to blake2b, from a kernel record."""
    n = int(rec.nbytes)
    words = (n - n % 4) // 4
    rows = words // ROW_WORDS
    s = [n]
    if rows:
        s += [int(rec.row_sum), int(rec.row_sum_w)]
    if words - rows * ROW_WORDS:
        s += [int(rec.tail_sum), int(rec.tail_sum_w)]
    if n % 4:
        s += [int(rec.ragged_sum), n % 4]
    return s


def digest_hex(scalars) -> str:
    h = hashlib.blake2b(digest_size=16)
    for v in scalars:
        h.update((int(v) & _U64).to_bytes(8, "little"))
    return h.hexdigest()


def _ctx_for(flat, ctx):
    return ctx if ctx is not None else default_context(flat.device.index or 0)


def digest_many(tensors, modes: int = DIGEST_SAFE32 | DIGEST_ROWS | DIGEST_BLOCK64,
                ctx: Context | None = None) -> list:
    """One launch over all tensors; returns a dict per tensor with the keys
    ``safe_checksum`` (str), ``tensor_digest`` (str), ``block_hash64`` (int) that
    the mode bits ask for."""
    flats = [_flat_cuda(t) for t in tensors]
    if not flats:
        return []
    c = _ctx_for(flats[0], ctx)
    dev = flats[0].device.index or 0
    import torch

    torch.cuda.current_stream(dev).synchronize()
    spans = [(f.data_ptr() if f.numel() else 0, f.numel()) for f in flats]
    recs = c.digest(spans, modes, dev)
    out = []
    for rec in recs:
        d = {}
        if modes & DIGEST_SAFE32:
            d["safe_checksum"] = format(int(rec.safe_checksum) & 0xFFFFFFFF, "08x")
        if modes & DIGEST_ROWS:
            d["tensor_digest"] = digest_hex(scalars_from_record(rec))
        if modes & DIGEST_BLOCK64:
            d["block_hash64"] = int(rec.block_hash)
        out.append(d)
    return out


def safe_checksum(tensor, ctx: Context | None = None) -> str:
    """Drop-in for ``modelexpress.tensor_utils.safe_checksum`` on CUDA tensors."""
    return digest_many([tensor], DIGEST_SAFE32, ctx)[0]["safe_checksum"]


def tensor_digest(tensor, ctx: Context | None = None) -> str:
    """Drop-in for ``modelexpress.refit.reshard.verify.tensor_digest``; any byte
    offset of the view is handled in the kernel, so no rebasing copy is made."""
    return digest_many([tensor], DIGEST_ROWS, ctx)[0]["tensor_digest"]


def block_hash64(tensor, ctx: Context | None = None) -> int:
    """64-bit hash over 4 KiB blocks (no counterpart in the reference)."""
    return digest_many([tensor], DIGEST_BLOCK64, ctx)[0]["block_hash64"]
