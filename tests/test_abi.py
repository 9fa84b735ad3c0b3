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
