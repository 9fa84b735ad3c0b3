"""ctypes access to the C restatement (``ref_port.c``). TEST INFRASTRUCTURE ONLY."""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class Run(ctypes.Structure):
    _fields_ = [("src", ctypes.c_uint64), ("dst", ctypes.c_uint64), ("nbytes", ctypes.c_uint64)]


class Desc2D(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64)
                for n in ("src", "dst", "rows", "row_bytes", "src_pitch", "dst_pitch")]


def build(force: bool = False) -> str:
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "ref_port.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"],
                              stdout=subprocess.DEVNULL)
    return so


def lib():
    global _LIB
    if _LIB is None:
        L = ctypes.CDLL(build())
        u8p, u64, u64p = ctypes.c_void_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_uint64)
        L.orc_memmove_runs.argtypes = [ctypes.POINTER(Run), u64]
        L.orc_scatter2d.argtypes = [ctypes.POINTER(Desc2D), u64]
        L.orc_scatter2d_mt.argtypes = [ctypes.POINTER(Desc2D), u64]
        for f in (L.orc_safe_checksum, L.orc_safe_checksum_mt):
            f.argtypes, f.restype = [u8p, u64], ctypes.c_uint32
        for f in (L.orc_digest_scalars, L.orc_digest_scalars_mt):
            f.argtypes, f.restype = [u8p, u64, u64p], ctypes.c_uint32
        L.orc_block_hashes64.argtypes = [u8p, u64, u64p]
        L.orc_block_hash64.argtypes, L.orc_block_hash64.restype = [u8p, u64], ctypes.c_uint64
        _LIB = L
    return _LIB


def _ptr(a: np.ndarray):
    return ctypes.c_void_p(a.ctypes.data)


def safe_checksum(a: np.ndarray, mt: bool = False) -> str:
    b = np.ascontiguousarray(a).reshape(-1).view(np.uint8)
    f = lib().orc_safe_checksum_mt if mt else lib().orc_safe_checksum
    return format(f(_ptr(b), b.size), "08x")


def digest_scalars(a: np.ndarray, mt: bool = False) -> list:
    b = np.ascontiguousarray(a).reshape(-1).view(np.uint8)
    out = (ctypes.c_uint64 * 7)()
    f = lib().orc_digest_scalars_mt if mt else lib().orc_digest_scalars
    mask = f(_ptr(b), b.size, out)
    s = [out[0]]
    if mask & 1:
        s += [out[1], out[2]]
    if mask & 2:
        s += [out[3], out[4]]
    if mask & 4:
        s += [out[5], out[6]]
    return [int(v) for v in s]


def block_hashes64(a: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(a).reshape(-1).view(np.uint8)
    out = np.zeros((b.size + 4095) // 4096, dtype=np.uint64)
    lib().orc_block_hashes64(_ptr(b), b.size, out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64)))
    return out


def block_hash64(a: np.ndarray) -> int:
    b = np.ascontiguousarray(a).reshape(-1).view(np.uint8)
    return int(lib().orc_block_hash64(_ptr(b), b.size))


def scatter2d(descs, mt: bool = False) -> None:
    """descs: iterable of (src, dst, rows, row_bytes, src_pitch, dst_pitch) host addresses."""
    descs = list(descs)
    arr = (Desc2D * len(descs))(*[Desc2D(*[int(x) for x in d]) for d in descs])
    (lib().orc_scatter2d_mt if mt else lib().orc_scatter2d)(arr, len(descs))


def memmove_runs(runs) -> None:
    runs = list(runs)
    arr = (Run * len(runs))(*[Run(*[int(x) for x in r]) for r in runs])
    lib().orc_memmove_runs(arr, len(runs))
