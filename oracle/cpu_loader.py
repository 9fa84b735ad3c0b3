"""The reference's host-staged load-and-shard, timed on CPU cores. TEST/BENCH
INFRASTRUCTURE ONLY (the benchmark's ``cpu_baseline`` leg and reference arm).

What the reference runs for this path (engines/vllm/adapter.py:316-329) is
vLLM's DefaultModelLoader: for every checkpoint tensor, ``safe_open(...)
.get_tensor(name)`` hands out the full tensor (a view of the memory-mapped
file, paged in on first touch), the layer's ``weight_loader`` narrows it to the
rank's slice and ``param.copy_`` writes the slice into the parameter, one
tensor at a time.  This port does exactly those
three steps with torch CPU tensors; the slice rules are the oracle's
(``ref_port._classify`` / ``load_and_shard``), which the CPU tests pin against
real vLLM layers.  Destinations are host tensors, so no PCIe copy is included:
the number is an upper bound on what the reference's CPU side can feed a GPU.
"""

from __future__ import annotations

import os
import time

from . import ref_port

VOCAB_PAD = ref_port.VOCAB_PAD


def _alloc_params(index: dict, tp_rank: int, tp_size: int):
    """Destination host tensors with the per-rank shapes (zero-filled)."""
    import torch

    from modelexpress_b200.layout import plan_checkpoint  # shapes only; no compute
    from modelexpress_b200.loader import torch_dtype

    plan = plan_checkpoint(index, tp_rank, tp_size, "dense")
    return {n: torch.zeros(tuple(s.shape), dtype=torch_dtype(s.dtype)) for n, s in plan.params.items()}


def load_and_shard_torch(model_dir: str, tp_rank: int, tp_size: int, params: dict | None = None,
                         max_bytes: int | None = None) -> tuple:
    """One pass of the reference's loop.  Returns (params, bytes_placed, seconds).
    ``max_bytes`` stops after that many placed bytes (a bounded sample)."""
    import torch
    from safetensors import safe_open

    files = sorted(os.path.join(model_dir, f) for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    if params is None:
        index = {}
        for path in files:
            for n, i in ref_port.parse_safetensors_header(path).items():
                index[n] = {"shape": i["shape"], "dtype": i["dtype"]}
        params = _alloc_params(index, tp_rank, tp_size)
    offsets: dict = {}
    placed = 0
    t0 = time.perf_counter()
    for path in files:
        with safe_open(path, framework="pt", device="cpu") as f:
            for name in f.keys():
                loaded = f.get_tensor(name)  # the full tensor, mapped from the file, as the reference does
                dest, kind, member = ref_port._classify(name)
                p = params[dest]
                if kind in ("qkv", "gate_up"):
                    order = ref_port._QKV_ORDER if kind == "qkv" else ref_port._GATE_UP_ORDER
                    loc = loaded.shape[0] // tp_size
                    # running offset of the member inside the fused parameter
                    key = (dest, member)
                    if key not in offsets:
                        prefix = name[: name.rfind(member)]
                        suffix = name[name.rfind(member) + len(member):]
                        off = 0
                        for m in order:
                            offsets[(dest, m)] = off
                            off += f_shape(files, prefix + m + suffix)[0] // tp_size
                    src = loaded.narrow(0, tp_rank * loc, loc)
                    p.narrow(0, offsets[key], loc).copy_(src)
                    placed += src.numel() * src.element_size()
                elif kind == "row":
                    loc = loaded.shape[1] // tp_size
                    src = loaded.narrow(1, tp_rank * loc, loc)
                    p.copy_(src)
                    placed += src.numel() * src.element_size()
                elif kind == "vocab":
                    loc = p.shape[0]
                    lo = tp_rank * loc
                    hi = min(loaded.shape[0], lo + loc)
                    if hi > lo:
                        p[: hi - lo].copy_(loaded[lo:hi])
                        placed += (hi - lo) * loaded.shape[1] * loaded.element_size()
                else:
                    p.copy_(loaded)
                    placed += loaded.numel() * loaded.element_size()
                if max_bytes is not None and placed >= max_bytes:
                    return params, placed, time.perf_counter() - t0
    return params, placed, time.perf_counter() - t0


_SHAPES: dict = {}


def f_shape(files, name):
    """Shape of a checkpoint tensor by name (header lookup, cached)."""
    if not _SHAPES:
        for path in files:
            for n, i in ref_port.parse_safetensors_header(path).items():
                _SHAPES[n] = tuple(i["shape"])
    if name not in _SHAPES:
        _SHAPES.clear()
        for path in files:
            for n, i in ref_port.parse_safetensors_header(path).items():
                _SHAPES[n] = tuple(i["shape"])
    return _SHAPES[name]
