"""``MxModelLoader`` for vLLM, weights placed by the B200 scatter path.

vLLM's ``--load-format modelexpress`` imports
``modelexpress.engines.vllm.loader:MxModelLoader`` and calls three methods on it
(vllm/model_executor/model_loader/modelexpress_loader.py:15-68).  The
reference's class (engines/vllm/loader.py:62-183) initialises the model, runs
its strategy chain and returns ``model.eval()``.  This class keeps that surface
— ``__init__(load_config)``, ``load_model(vllm_config, model_config, prefix)``,
``download_model(model_config)``, ``load_weights(model, model_config)``, the
``nixl_manager`` / ``tensors`` properties — and runs a chain of strategies:
``B200FanoutStrategy`` (a serving peer on the same box has published its weights
in the rendezvous directory ``MXB_FANOUT_DIR``: they arrive over NVLink, the
checkpoint is not read at all), ``B200CapturedStrategy`` (the model's own ``load_weights`` dry-run over
byte-less placeholders tells which window of which checkpoint tensor lands
where, for any architecture vLLM can load; safetensors -> pinned ring -> PCIe
-> scatter kernel, straight into the engine's parameters), then
``B200ScatterStrategy`` (the same data path planned from built-in layout
rules), then vLLM's own ``DefaultModelLoader`` when the checkpoint is not a
local safetensors directory.  The ``shim/`` directory next to this package
exposes the class at the dotted path vLLM imports.
"""

from __future__ import annotations

import copy
import logging
import os

from ...fanout import B200FanoutStrategy
from ...loader import B200CapturedStrategy, B200ScatterStrategy, LoadResult, StrategyFailed

logger = logging.getLogger("modelexpress_b200.engines.vllm")

try:  # vLLM is the host engine; without it the class still imports for inspection
    from vllm.model_executor.model_loader.base_loader import BaseModelLoader
except Exception:  # pragma: no cover - exercised only where vLLM is absent
    class BaseModelLoader:  # type: ignore[no-redef]
        def __init__(self, load_config):
            self.load_config = load_config


class VllmScatterAdapter:
    """The two hooks ``B200ScatterStrategy`` needs from an engine adapter, for vLLM
    (the reference's adapter contract is adapter.py:54-196)."""

    def tp_layout(self, result) -> tuple:
        from vllm.distributed import (get_tensor_model_parallel_rank,
                                      get_tensor_model_parallel_world_size)

        return int(get_tensor_model_parallel_rank()), int(get_tensor_model_parallel_world_size())

    def named_destinations(self, result) -> dict:
        return {name: p.data for name, p in result.model.named_parameters()}


class _Ctx:
    def __init__(self, model_config, device_id: int, reinit=None):
        self.model_config = model_config
        self.device_id = device_id
        self.adapter = VllmScatterAdapter()
        if reinit is not None:
            # adapter.py:24-34 of the reference: after a strategy failed having written into
            # the model, the next one starts from a freshly initialised model
            self.adapter.reinit_for_retry = reinit


class MxModelLoader(BaseModelLoader):
    """Drop-in for the reference's vLLM loader class."""

    def __init__(self, load_config):
        super().__init__(load_config)
        self._tensors: dict = {}
        self.last_strategy: str | None = None
        self.last_metadata: dict | None = None

    # -- BaseModelLoader surface ------------------------------------------------
    def download_model(self, model_config) -> None:
        """A local checkpoint directory needs nothing; anything else goes through
        vLLM's own downloader, as the reference does (loader.py:138-158)."""
        if os.path.isdir(str(model_config.model)):
            return
        self._native().download_model(model_config)

    def load_weights(self, model, model_config, reinit=None):
        """Load weights into an already-initialised model (standalone API).  ``reinit``
        (``LoadResult -> LoadResult``) re-initialises the model after a strategy failed
        having written into it (load_strategy/__init__.py:95-131); without it the next
        strategy starts from the model as the failed one left it, which is safe only
        because every strategy after the first writes every parameter it loads.
        Returns the model that holds the weights (another object after a reinit)."""
        import torch

        device_id = torch.cuda.current_device()
        result = LoadResult(value=model, model=model)
        ctx = _Ctx(model_config, device_id, reinit)
        self.last_strategy = None
        for strategy in (B200FanoutStrategy(), B200CapturedStrategy(), B200ScatterStrategy()):
            try:
                if not strategy.is_available(ctx):
                    raise StrategyFailed("not available here", mutated=False)
                result = strategy.load(result, ctx) or result
                self.last_strategy = strategy.name
                self.last_metadata = result.metadata.get(strategy.name)
                logger.info("weights placed by %s: %s", strategy.name, result.metadata.get(strategy.name))
                break
            except StrategyFailed as e:
                strategy.rollback(ctx)
                level = logger.warning if e.mutated else logger.info
                level("%s did not load the model (%s); trying the next strategy", strategy.name, e)
                if e.mutated and reinit is not None:
                    result = reinit(result)
        if self.last_strategy is None:
            self._native().load_weights(result.model, model_config)
            self.last_strategy = "default"
        self._tensors = {n: p.data for n, p in result.model.named_parameters()}
        return result.model

    def load_model(self, vllm_config, model_config, prefix: str = ""):
        import torch
        from vllm.model_executor.model_loader.utils import (initialize_model,
                                                            process_weights_after_loading)
        from vllm.utils.torch_utils import set_default_torch_dtype

        from ...arena import maybe_enter_arena

        device_config = vllm_config.device_config
        target_device = torch.device(device_config.device)
        dev_index = target_device.index if target_device.index is not None else (
            torch.cuda.current_device() if target_device.type == "cuda" else 0)
        # MXB_VMM_ARENA=1: the model is allocated in one arena that peers can map through a single
        # descriptor exchange (the load envelope of the reference's loader.py:107-127)
        with maybe_enter_arena(dev_index, os.environ.get("MXB_FANOUT_DIR")), \
                set_default_torch_dtype(model_config.dtype):
            def fresh_model():
                with target_device:
                    return initialize_model(vllm_config=vllm_config, model_config=model_config, prefix=prefix)

            def reinit(result):
                model = fresh_model()
                return LoadResult(value=model, model=model, metadata=result.metadata)

            model = self.load_weights(fresh_model(), model_config, reinit)
            process_weights_after_loading(model, model_config, target_device)
        return model.eval()

    # -- reference-compatible extras ---------------------------------------------
    @property
    def nixl_manager(self):
        """There is no NIXL agent on this path (peers are reached over NVLink)."""
        return None

    @property
    def tensors(self) -> dict:
        return self._tensors

    def _native(self):
        from vllm.model_executor.model_loader.default_loader import DefaultModelLoader

        disk_config = copy.copy(self.load_config)
        try:
            disk_config.load_format = "auto"
        except AttributeError:
            object.__setattr__(disk_config, "load_format", "auto")
        return DefaultModelLoader(disk_config)
