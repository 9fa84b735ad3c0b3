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
    elif getattr(mc, "is_moe", False) and getattr(ps, "_EP", None) is None:
        # the groups were made for a dense model earlier in this process: an expert-parallel
        # group only exists when they are made under a MoE config
        ps.destroy_model_parallel()
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

        # the same load planned from vLLM's own load_weights instead of layout rules
        from modelexpress_b200.loader import place_captured

        for p in params.values():
            p.data.zero_()
        got = place_captured(model, d, "cuda:0", ring_bytes=16 << 20, ring_slots=4, host_threads=2)
        assert got.engine_loaded == [] and not got.converted, got.reasons
        assert got.stats.bytes_placed == placed.stats.bytes_placed
        assert got.written_params == set(truth)
        for n, t in truth.items():
            assert torch.equal(params[n].detach().view(torch.int16), t.view(torch.int16)), n

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
            assert type(inner).__name__ == "MxModelLoader" and inner.last_strategy == "b200_captured"
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
            # MXB_VMM_ARENA=1 (the reference's MX_VMM_ARENA envelope, engines/vllm/loader.py:107-127):
            # the same load with the model allocated in an arena that is published for peers
            from modelexpress_b200 import arena as arena_mod

            os.environ["MXB_VMM_ARENA"] = "1"
            try:
                vc3 = VllmConfig(model_config=mc, device_config=DeviceConfig(device="cuda"),
                                 load_config=LoadConfig(load_format="auto"))
                with set_current_vllm_config(vc3):
                    model3 = wrapper.load_model(vllm_config=vc3, model_config=mc)
            finally:
                del os.environ["MXB_VMM_ARENA"]
            hits = [arena_mod.lookup(p.data_ptr(), p.numel() * p.element_size()) for p in model3.parameters()]
            assert all(h is not None for h in hits) and len({h[0] for h in hits}) == 1
            for n, p in model3.named_parameters():
                assert torch.equal(p.detach().view(torch.int16), truth[n].view(torch.int16)), n
            served = arena_mod._published[hits[0][0]][0]
            assert served.live_allocation_count >= 1 and served.mapped_bytes >= sum(
                p.numel() * p.element_size() for p in model3.parameters())
            arena_mod.withdraw_arena(hits[0][0])
        finally:
            sys.path.remove(shim)
            for k in [k for k in sys.modules if k == "modelexpress" or k.startswith("modelexpress.")]:
                del sys.modules[k]
    finally:
        ctx.__exit__(None, None, None)


MOE_CFG = {"architectures": ["Qwen3MoeForCausalLM"], "model_type": "qwen3_moe", "hidden_size": 256,
           "intermediate_size": 512, "moe_intermediate_size": 128, "num_hidden_layers": 2,
           "num_attention_heads": 8, "num_key_value_heads": 4, "head_dim": 32, "vocab_size": 1024,
           "num_experts": 8, "num_experts_per_tok": 2, "decoder_sparse_step": 1, "norm_topk_prob": True,
           "mlp_only_layers": [], "max_position_embeddings": 512, "rms_norm_eps": 1e-6,
           "rope_theta": 10000.0, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
           "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2}


def _qwen3_moe_tensors(c):
    h, hd = c["hidden_size"], c["head_dim"]
    out = [("model.embed_tokens.weight", (c["vocab_size"], h), "BF16", "matrix")]
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        out += [(p + "input_layernorm.weight", (h,), "BF16", "matrix"),
                (p + "self_attn.q_proj.weight", (c["num_attention_heads"] * hd, h), "BF16", "matrix"),
                (p + "self_attn.k_proj.weight", (c["num_key_value_heads"] * hd, h), "BF16", "matrix"),
                (p + "self_attn.v_proj.weight", (c["num_key_value_heads"] * hd, h), "BF16", "matrix"),
                (p + "self_attn.q_norm.weight", (hd,), "BF16", "matrix"),
                (p + "self_attn.k_norm.weight", (hd,), "BF16", "matrix"),
                (p + "self_attn.o_proj.weight", (h, c["num_attention_heads"] * hd), "BF16", "matrix"),
                (p + "post_attention_layernorm.weight", (h,), "BF16", "matrix"),
                (p + "mlp.gate.weight", (c["num_experts"], h), "BF16", "matrix")]
        for e in range(c["num_experts"]):
            q = f"{p}mlp.experts.{e}."
            out += [(q + "gate_proj.weight", (c["moe_intermediate_size"], h), "BF16", "matrix"),
                    (q + "up_proj.weight", (c["moe_intermediate_size"], h), "BF16", "matrix"),
                    (q + "down_proj.weight", (h, c["moe_intermediate_size"]), "BF16", "matrix")]
    out += [("model.norm.weight", (h,), "BF16", "matrix"),
            ("lm_head.weight", (c["vocab_size"], h), "BF16", "matrix")]
    return out


def test_place_captured_loads_a_vllm_moe_model_with_no_layout_rules(tmp_path):
    """An architecture the built-in placement rules do not describe (per-expert
    checkpoint tensors stacked into vLLM's fused expert parameters): the capture
    of vLLM's own ``load_weights`` plans it, and every parameter ends up
    bit-identical to what ``load_weights`` itself produces."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from modelexpress_b200 import synth
    from modelexpress_b200.loader import place_captured

    d = str(tmp_path)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(MOE_CFG, f)
    synth.write_checkpoint(d, _qwen3_moe_tensors(MOE_CFG), 33, 2)
    try:
        model, ctx, vc, mc = _build_vllm_model(d)
    except Exception as e:
        pytest.skip(f"vLLM could not build a MoE model here: {type(e).__name__}: {e}")
    try:
        from safetensors import safe_open

        weights = []
        for fn in sorted(os.listdir(d)):
            if fn.endswith(".safetensors"):
                with safe_open(os.path.join(d, fn), framework="pt", device="cpu") as f:
                    weights += [(k, f.get_tensor(k)) for k in f.keys()]
        model.load_weights(iter(weights))
        torch.cuda.synchronize()
        params = dict(model.named_parameters())
        truth = {n: p.detach().clone() for n, p in params.items()}
        for p in params.values():
            p.data.zero_()
        torch.cuda.synchronize()
        got = place_captured(model, d, "cuda:0", ring_bytes=16 << 20, ring_slots=4, host_threads=2)
        ckpt_bytes = sum(t.numel() * t.element_size() for _n, t in weights)
        engine_bytes = sum(t.numel() * t.element_size() for n, t in weights if n in got.engine_loaded)
        # everything but at most a handful of small tensors goes through the scatter kernel
        assert engine_bytes <= ckpt_bytes // 100, got.reasons
        assert got.stats.bytes_placed >= ckpt_bytes - engine_bytes - sum(
            t.numel() * t.element_size() for n, t in weights if "rotary" in n)
        experts = [n for n in truth if "experts" in n]
        assert experts and set(experts) <= got.written_params
        for n, t in truth.items():
            assert torch.equal(params[n].detach().view(torch.uint8), t.view(torch.uint8)), n
    finally:
        ctx.__exit__(None, None, None)


GPT2_CFG = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_embd": 256, "n_head": 8,
            "n_layer": 2, "n_positions": 512, "n_inner": 1024, "vocab_size": 1024,
            "layer_norm_epsilon": 1e-5, "activation_function": "gelu_new", "tie_word_embeddings": True,
            "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2}


def _gpt2_tensors():
    """Conv1D weights are stored (in, out); vLLM's loader transposes them on the way in."""
    out = [("wte.weight", (1024, 256), "BF16", "matrix"), ("wpe.weight", (512, 256), "BF16", "matrix")]
    for i in range(2):
        p = f"h.{i}."
        out += [(p + "ln_1.weight", (256,), "BF16", "matrix"), (p + "ln_1.bias", (256,), "BF16", "matrix"),
                (p + "attn.c_attn.weight", (256, 768), "BF16", "matrix"),
                (p + "attn.c_attn.bias", (768,), "BF16", "matrix"),
                (p + "attn.c_proj.weight", (256, 256), "BF16", "matrix"),
                (p + "attn.c_proj.bias", (256,), "BF16", "matrix"),
                (p + "ln_2.weight", (256,), "BF16", "matrix"), (p + "ln_2.bias", (256,), "BF16", "matrix"),
                (p + "mlp.c_fc.weight", (256, 1024), "BF16", "matrix"),
                (p + "mlp.c_fc.bias", (1024,), "BF16", "matrix"),
                (p + "mlp.c_proj.weight", (1024, 256), "BF16", "matrix"),
                (p + "mlp.c_proj.bias", (256,), "BF16", "matrix")]
    return out + [("ln_f.weight", (256,), "BF16", "matrix"), ("ln_f.bias", (256,), "BF16", "matrix")]


def test_transposed_checkpoint_weights_go_through_the_convert_kernel(tmp_path):
    """vLLM's ``GPT2LMHeadModel`` on the GPU: its loader transposes every Conv1D weight.  The
    capture stages those sources as the boxes they read, the box-convert kernel turns them, and
    every parameter equals what vLLM's own ``load_weights`` produces; nothing is left to it."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from modelexpress_b200 import synth
    from modelexpress_b200.loader import place_captured
    from modelexpress_b200.runtime import default_context

    d = str(tmp_path)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(GPT2_CFG, f)
    synth.write_checkpoint(d, _gpt2_tensors(), 44, 2)
    try:
        model, ctx, vc, mc = _build_vllm_model(d)
    except Exception as e:
        pytest.skip(f"vLLM could not build a GPT-2 model here: {type(e).__name__}: {e}")
    try:
        from safetensors import safe_open

        weights = []
        for fn in sorted(os.listdir(d)):
            if fn.endswith(".safetensors"):
                with safe_open(os.path.join(d, fn), framework="pt", device="cpu") as f:
                    weights += [(k, f.get_tensor(k)) for k in f.keys()]
        model.load_weights(iter(weights))
        torch.cuda.synchronize()
        params = dict(model.named_parameters())
        truth = {n: p.detach().clone() for n, p in params.items()}
        for p in params.values():
            p.data.zero_()
        torch.cuda.synchronize()
        before = default_context(0).launch_count
        got = place_captured(model, d, "cuda:0", ring_bytes=16 << 20, ring_slots=4, host_threads=2)
        assert got.engine_loaded == [], got.reasons
        turned = [n for n in got.converted if n.endswith(("c_attn.weight", "c_proj.weight", "c_fc.weight"))]
        assert len(turned) >= 8, got.converted       # four Conv1D weights per layer
        assert default_context(0).launch_count > before
        for n, t in truth.items():
            assert torch.equal(params[n].detach().view(torch.uint8), t.view(torch.uint8)), n
    finally:
        ctx.__exit__(None, None, None)
