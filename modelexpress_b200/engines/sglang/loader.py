"""``MxModelLoader`` for SGLang (signature of engines/sglang/loader.py:44-86).

SGLang instantiates the class from its ``remote_instance`` loader and hands it
an ALREADY INITIALISED model: ``load_model(*, model, model_config,
device_config) -> nn.Module``.  Here the weights are placed into that model's
parameters by the scatter path: planned from the model's own ``load_weights``
when it has one (``B200CapturedStrategy``), else from the built-in layout rules
(``B200ScatterStrategy``).  SGLang is not installed where this library was
developed, so this adapter is covered only by a test with stand-in objects; the
placement underneath is the same code the vLLM adapter exercises.
"""

from __future__ import annotations

import logging

from ...loader import B200CapturedStrategy, B200ScatterStrategy, LoadResult, StrategyFailed

logger = logging.getLogger("modelexpress_b200.engines.sglang")


class SglangScatterAdapter:
    def __init__(self, tp_rank: int | None = None, tp_size: int | None = None):
        self._tp = (tp_rank, tp_size)

    def tp_layout(self, result) -> tuple:
        if self._tp[0] is not None:
            return int(self._tp[0]), int(self._tp[1])
        from sglang.srt.distributed import (get_tensor_model_parallel_rank,
                                            get_tensor_model_parallel_world_size)

        return int(get_tensor_model_parallel_rank()), int(get_tensor_model_parallel_world_size())

    def named_destinations(self, result) -> dict:
        return {name: p.data for name, p in result.model.named_parameters()}


class _Ctx:
    def __init__(self, model_config, device_id, adapter):
        self.model_config, self.device_id, self.adapter = model_config, device_id, adapter


class MxModelLoader:
    """Drop-in for the reference's SGLang loader class."""

    def __init__(self, load_config, tp_rank: int | None = None, tp_size: int | None = None):
        self.load_config = load_config
        self._adapter = SglangScatterAdapter(tp_rank, tp_size)
        self._tensors: dict = {}
        self.last_strategy: str | None = None

    def load_model(self, *, model, model_config, device_config):
        """Place the checkpoint at ``model_config.model_path`` (SGLang's field; ``model``
        is accepted too) into ``model``; raises ``RuntimeError`` when the scatter path
        cannot serve it, as the reference's chain does when no strategy succeeds
        (load_strategy/__init__.py:114-117)."""
        import torch

        path = getattr(model_config, "model_path", None) or getattr(model_config, "model", None)

        class _Cfg:
            model = path

        gpu_id = getattr(device_config, "gpu_id", None)
        device_id = torch.cuda.current_device() if gpu_id in (None, -1) else int(gpu_id)
        ctx = _Ctx(_Cfg(), device_id, self._adapter)
        if not B200ScatterStrategy().is_available(ctx):
            raise RuntimeError("No loading strategy succeeded: CUDA library or device unavailable")
        errors = []
        self.last_strategy = None
        for strategy in (B200CapturedStrategy(), B200ScatterStrategy()):
            try:
                strategy.load(LoadResult(value=model, model=model), ctx)
                self.last_strategy = strategy.name
                break
            except StrategyFailed as e:
                strategy.rollback(ctx)
                errors.append(f"{strategy.name}: {e}")
        if self.last_strategy is None:
            raise RuntimeError(f"No loading strategy succeeded for model {path!r}: " + "; ".join(errors))
        self._tensors = {n: p.data for n, p in model.named_parameters()}
        return model.eval()

    @property
    def tensors(self) -> dict:
        return self._tensors
