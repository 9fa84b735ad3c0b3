"""Load-strategy contract without a GPU: the misses that must be reported as
``StrategyFailed(mutated=False)`` before anything is touched
(load_strategy/base.py:37-76, adapter.py:24-34), and that there is no CPU fallback."""

import pytest
import torch

from modelexpress_b200.loader import (B200CapturedStrategy, B200ScatterStrategy, LoadResult,
                                      StrategyFailed, place_captured, place_checkpoint)


class _Cfg:
    def __init__(self, model):
        self.model = model


class _Ctx:
    def __init__(self, model_dir, adapter=object()):
        self.model_config, self.device_id, self.adapter = _Cfg(model_dir), 0, adapter


class _WithLoader(torch.nn.Module):
    def load_weights(self, weights):
        return set()


@pytest.mark.parametrize("strategy", [B200CapturedStrategy, B200ScatterStrategy])
def test_missing_checkpoint_directory_is_an_expected_miss(strategy, tmp_path):
    s = strategy()
    assert s.requires == () and s.name in ("b200_captured", "b200_scatter")
    for bad in (None, "", str(tmp_path / "nowhere")):
        with pytest.raises(StrategyFailed) as e:
            s.load(LoadResult(value=None, model=_WithLoader()), _Ctx(bad))
        assert e.value.mutated is False
    s.rollback(_Ctx(None))


def test_captured_strategy_needs_a_loader_to_dry_run(tmp_path):
    with pytest.raises(StrategyFailed, match="load_weights") as e:
        B200CapturedStrategy().load(LoadResult(value=None, model=torch.nn.Linear(2, 2)), _Ctx(str(tmp_path)))
    assert e.value.mutated is False


def test_scatter_strategy_names_the_adapter_hook_it_lacks(tmp_path):
    with pytest.raises(StrategyFailed, match="adapter") as e:
        B200ScatterStrategy().load(LoadResult(value=None, model=_WithLoader()), _Ctx(str(tmp_path)))
    assert e.value.mutated is False


def test_strategies_are_unavailable_without_an_adapter():
    assert B200ScatterStrategy().is_available(_Ctx("x", adapter=None)) is False


def test_no_cpu_fallback():
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        place_checkpoint("/nonexistent", 0, 1, "cpu")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        place_captured(_WithLoader(), "/nonexistent", "cpu")


def test_truncated_shard_is_an_expected_miss(tmp_path):
    """A half-written safetensors file must fail before any copy is planned
    (ValueError -> StrategyFailed(mutated=False)), not run past the mapping."""
    import os

    import pytest

    from modelexpress_b200 import synth
    from modelexpress_b200.loader import FileImage, check_index
    from modelexpress_b200.safetensors_index import checkpoint_index

    cfg = synth.DenseConfig("trunc", 1, 64, 128, 2, 2, 32, 256, False, 5, 1)
    d = str(tmp_path)
    synth.write_checkpoint(d, synth.dense_tensors(cfg), cfg.seed, 1)
    idx = checkpoint_index(d)
    path = next(iter({i["file"] for i in idx.values()}))
    check_index(idx, {path: os.path.getsize(path)})
    with open(path, "r+b") as f:
        f.truncate(os.path.getsize(path) - 100)
    im = FileImage(path)
    try:
        with pytest.raises(ValueError, match="truncated"):
            check_index(idx, {path: im.size})
    finally:
        im.close()
    bad = {n: dict(i) for n, i in idx.items()}
    first = next(iter(bad))
    bad[first]["size"] = bad[first]["size"] + 2
    with pytest.raises(ValueError, match="header gives"):
        check_index(bad, {path: 1 << 40})


def test_prepared_plan_is_cached_until_the_files_change(tmp_path):
    """HostImages.prepared: the parsed headers and the rank's plan are kept while the
    checkpoint files keep their size and modification time, rebuilt when one changes;
    its record arrays are what placement_items computes tensor by tensor."""
    import os
    import time

    import numpy as np

    from modelexpress_b200 import synth
    from modelexpress_b200.loader import HostImages, Prepared, placement_items

    cfg = synth.DenseConfig("prep", 2, 64, 128, 4, 4, 16, 256, False, 9, 2)
    d = str(tmp_path)
    synth.write_checkpoint(d, synth.dense_tensors(cfg), cfg.seed, cfg.files)
    images = HostImages()
    a = images.prepared(d, 1, 2, "auto")
    assert images.prepared(d, 1, 2, "auto") is a and images.prepared(d, 0, 2, "auto") is not a
    assert a.fresh() and len(a.files) == 2 and a.geometry.shape == (len(a.plan.placements), 6)

    class FakeTensor:          # only what items() asks of a destination
        def __init__(self, spec, ptr):
            self.shape, self._ptr = tuple(spec.shape), ptr
            self._el = {"BF16": 2, "F32": 4}[spec.dtype]

        def is_contiguous(self):
            return True

        def element_size(self):
            return self._el

        def data_ptr(self):
            return self._ptr

    params = {n: FakeTensor(s, 1 << 40 | (k << 24)) for k, (n, s) in enumerate(a.plan.params.items())}
    addresses = {p: (7 << 32) + 4096 * k for k, p in enumerate(a.files)}
    assert np.array_equal(a.items(addresses, params), placement_items(a.plan, a.index, addresses, params))
    # a rewritten file (same size, later mtime) invalidates the plan
    path = a.files[0]
    st = os.stat(path)
    os.utime(path, ns=(st.st_atime_ns, st.st_mtime_ns + 5_000_000_000))
    assert not a.fresh()
    b = images.prepared(d, 1, 2, "auto")
    assert b is not a and b.fresh()
    images.close()
