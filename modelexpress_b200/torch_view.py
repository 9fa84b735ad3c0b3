"""View a raw device allocation as a torch tensor (tests and benchmarks use it
to fill and inspect library-owned arenas; the data path never needs it)."""

from __future__ import annotations


class _Holder:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


def as_tensor(ptr: int, nbytes: int, device: int):
    """uint8 tensor over ``[ptr, ptr+nbytes)`` on ``cuda:device``; the caller keeps
    the allocation alive."""
    import torch

    return torch.as_tensor(_Holder(int(ptr), int(nbytes)), device=f"cuda:{device}")
