"""Drop-in check at the real engine boundary: a vLLM ``LlamaForCausalLM`` built on
the GPU, loaded once by vLLM's own ``load_weights`` (what the reference's
host-staged path ends in, engines/vllm/adapter.py:223-231, 316-329) and once by
``place_checkpoint`` writing into the same ``named_parameters()``; every
parameter must be bit-identical.  Skips (never fails) when vLLM cannot build a
model in this environment."""

import json
import os

import pytest

pytestmark = pytest.mark.gpu

CFG = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 256,
       "intermediate_size": 512, "num_hidden_layers": 2, "num_attention_heads": 8,
       "num_key_value_heads": 4, "head_dim": 32, "vocab_size": 1024, "max_position_embeddings": 512,
       "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "tie_word_embeddings": False,
       "torch_dtype": "bfloat16", "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2}


def _build_vllm_model(model_dir):
    import torch
    from vllm.config import DeviceConfig, LoadConfig, ModelConfig, VllmConfig, set_current_vllm_config
    from vllm.distributed import parallel_state as ps
    from vllm.model_executor.model_loader.utils import initialize_model
    from vllm.utils.torch_utils import set_default_torch_dtype

    mc = ModelConfig(model=model_dir, skip_tokenizer_init=True, dtype="bfloat16", enforce_eager=True)
    vc = VllmConfig(model_config=mc, device_config=DeviceConfig(device="cuda"),
                    load_config=LoadConfig(load_format="dummy"))
    ctx = set_current_vllm_config(vc)
    ctx.__enter__()
    if not ps.model_parallel_is_initialized():
        port = 29700 + os.getpid() % 200
        ps.init_distributed_environment(world_size=1, rank=0, local_rank=0, backend="nccl",
                                        distributed_init_method=f"tcp://127.0.0.1:{port}")
        ps.initialize_model_parallel(1, 1)
    with set_default_torch_dtype(torch.bfloat16), torch.device("cuda"):
        model = initialize_model(vllm_config=vc)
    return model, ctx, vc, mc


def test_place_checkpoint_equals_vllm_load_weights(tmp_path):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from modelexpress_b200 import synth
    from modelexpress_b200.loader import place_checkpoint

    d = str(tmp_path)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(CFG, f)
    cfg = synth.DenseConfig("tiny-vllm", layers=2, hidden=256, intermediate=512, q_heads=8, kv_heads=4,
                            head_dim=32, vocab=1024, qkv_bias=False, seed=21, files=1)
    synth.write_checkpoint(d, synth.dense_tensors(cfg), cfg.seed, 1)
    try:
        model, ctx, vc, mc = _build_vllm_model(d)
    except Exception as e:  # vLLM internals differ between versions / environments
        pytest.skip(f"vLLM could not build a model here: {type(e).__name__}: {e}")
    try:
        from safetensors import safe_open

        with safe_open(os.path.join(d, "model.safetensors"), framework="pt", device="cpu") as f:
            weights = [(k, f.get_tensor(k)) for k in f.keys()]
        model.load_weights(iter(weights))            # the engine's own loader: ground truth
        torch.cuda.synchronize()
        params = dict(model.named_parameters())
        truth = {n: p.detach().clone() for n, p in params.items()}
        for p in params.values():
            p.data.zero_()
        torch.cuda.synchronize()
        dests = {n: p.data for n, p in params.items()}
        placed = place_checkpoint(d, 0, 1, "cuda:0", params=dests, ring_bytes=16 << 20, ring_slots=4,
                                  host_threads=2)
        assert set(placed.plan.params) <= set(params), sorted(set(placed.plan.params) - set(params))
        for n, t in truth.items():
            assert torch.equal(params[n].detach().view(torch.int16), t.view(torch.int16)), n
        assert placed.stats.bytes_placed == sum(t.numel() * t.element_size() for t in truth.values())

        # the outermost seam: vLLM's own `--load-format modelexpress` wrapper importing
        # modelexpress.engines.vllm.loader:MxModelLoader (here: the shim directory)
        import sys

        from vllm.config import LoadConfig

        shim = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                            "modelexpress_b200", "shim")
        sys.path.insert(0, shim)
        try:
            from vllm.model_executor.model_loader.modelexpress_loader import ModelExpressModelLoader

            from vllm.config import DeviceConfig, VllmConfig, set_current_vllm_config

            wrapper = ModelExpressModelLoader(LoadConfig(load_format="auto"))
            # a second model needs its own config object (layer names are registered per config)
            vc2 = VllmConfig(model_config=mc, device_config=DeviceConfig(device="cuda"),
                             load_config=LoadConfig(load_format="auto"))
            with set_current_vllm_config(vc2):
                model2 = wrapper.load_model(vllm_config=vc2, model_config=mc)
            inner = wrapper._loader
            assert type(inner).__name__ == "MxModelLoader" and inner.last_strategy == "b200_scatter"
            assert inner.nixl_manager is None and set(inner.tensors) == set(truth)
            assert not model2.training
            for n, p in model2.named_parameters():
                assert torch.equal(p.detach().view(torch.int16), truth[n].view(torch.int16)), n
            # standalone API on the already-initialised first model
            for p in params.values():
                p.data.zero_()
            inner.load_weights(model, mc)
            for n, t in truth.items():
                assert torch.equal(params[n].detach().view(torch.int16), t.view(torch.int16)), n
        finally:
            sys.path.remove(shim)
            for k in [k for k in sys.modules if k == "modelexpress" or k.startswith("modelexpress.")]:
                del sys.modules[k]
    finally:
        ctx.__exit__(None, None, None)
