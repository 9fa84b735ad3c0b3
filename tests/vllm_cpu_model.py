"""Helper run as a child process by test_geometry_capture.py: whole vLLM models on
the CPU with a faked tensor-parallel layout.

For each architecture and TP rank: build the real vLLM model (its attention
class replaced by an empty module: attention owns no checkpoint tensor and needs
a GPU platform to construct), load a seeded synthetic checkpoint with vLLM's own
``load_weights`` (the ground truth), zero the parameters, then compile the dry
run of the same ``load_weights`` into records, move the bytes with the CPU
scatter of the oracle, and compare every parameter bit for bit.  Prints one JSON
object.  Runs in its own process because vLLM's parallel state is global.
"""

import importlib
import json
import os
import sys
import tempfile
from unittest import mock

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

def _dense(bias):
    from modelexpress_b200 import synth

    cfg = synth.DenseConfig("tiny", layers=2, hidden=256, intermediate=512, q_heads=8, kv_heads=4,
                            head_dim=32, vocab=1000, qkv_bias=bias, seed=21, files=1)
    # random values for the norms too, so that a misplaced norm cannot pass
    return [(n, s, dt, "matrix") for n, s, dt, _k in synth.dense_tensors(cfg)]


def _phi3():
    """Checkpoint with q/k/v and gate/up already fused on disk."""
    out = [("model.embed_tokens.weight", (1000, 256), "BF16", "matrix")]
    for i in range(2):
        p = f"model.layers.{i}."
        out += [(p + "input_layernorm.weight", (256,), "BF16", "matrix"),
                (p + "self_attn.qkv_proj.weight", ((8 + 2 * 4) * 32, 256), "BF16", "matrix"),
                (p + "self_attn.o_proj.weight", (256, 256), "BF16", "matrix"),
                (p + "post_attention_layernorm.weight", (256,), "BF16", "matrix"),
                (p + "mlp.gate_up_proj.weight", (2 * 512, 256), "BF16", "matrix"),
                (p + "mlp.down_proj.weight", (256, 512), "BF16", "matrix")]
    return out + [("model.norm.weight", (256,), "BF16", "matrix"),
                  ("lm_head.weight", (1000, 256), "BF16", "matrix")]


def _gpt2():
    """Conv1D weights are stored (in, out): the loader transposes them; embeddings tied."""
    out = [("wte.weight", (1000, 256), "BF16", "matrix"), ("wpe.weight", (512, 256), "BF16", "matrix")]
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


_LLAMA_LIKE = {"hidden_size": 256, "intermediate_size": 512, "num_hidden_layers": 2,
               "num_attention_heads": 8, "num_key_value_heads": 4, "vocab_size": 1000,
               "max_position_embeddings": 512, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
               "tie_word_embeddings": False, "hidden_act": "silu"}
ARCHS = {
    "llama": ({**_LLAMA_LIKE, "architectures": ["LlamaForCausalLM"], "model_type": "llama", "head_dim": 32},
              lambda: _dense(False)),
    "qwen2": ({**_LLAMA_LIKE, "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2"},
              lambda: _dense(True)),
    "phi3": ({**_LLAMA_LIKE, "architectures": ["Phi3ForCausalLM"], "model_type": "phi3",
              "pad_token_id": 0, "original_max_position_embeddings": 512}, _phi3),
    "gpt2": ({"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_embd": 256, "n_head": 8,
              "n_layer": 2, "n_positions": 512, "n_inner": 1024, "vocab_size": 1000,
              "layer_norm_epsilon": 1e-5, "activation_function": "gelu_new",
              "tie_word_embeddings": True}, _gpt2),
}
TP = 4


class NoAttention(torch.nn.Module):
    def __init__(self, *args, **kwargs):
        super().__init__()


PATCHED = ("vllm.model_executor.layers.linear", "vllm.model_executor.layers.vocab_parallel_embedding",
           "vllm.model_executor.parameter", "vllm.model_executor.utils",
           "vllm.distributed.parallel_state", "vllm.model_executor.models.llama",
           "vllm.model_executor.models.qwen2", "vllm.model_executor.models.phi3",
           "vllm.model_executor.models.gpt2")


def run_arch(arch, cfg_json, make_tensors, out):
    from vllm.config import (DeviceConfig, LoadConfig, ModelConfig, VllmConfig,
                             set_current_vllm_config)
    from vllm.distributed import parallel_state as ps
    from vllm.model_executor.model_loader.utils import initialize_model
    from vllm.utils.torch_utils import set_default_torch_dtype
    from safetensors import safe_open

    from modelexpress_b200 import synth
    from modelexpress_b200.loader import FileImage, captured_table
    from modelexpress_b200.safetensors_index import checkpoint_index
    from oracle import c_port

    d = tempfile.mkdtemp(prefix=f"mxb_{arch}_")
    cfg_json = {"torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2, **cfg_json}
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg_json, f)
    synth.write_checkpoint(d, make_tensors(), 21, 1)
    path = os.path.join(d, "model.safetensors")
    with safe_open(path, framework="pt", device="cpu") as f:
        weights = [(k, f.get_tensor(k)) for k in f.keys()]
    index = checkpoint_index(d)
    image = FileImage(path)
    mc = ModelConfig(model=d, skip_tokenizer_init=True, dtype="bfloat16", enforce_eager=True)
    for rank in range(TP):
        vc = VllmConfig(model_config=mc, device_config=DeviceConfig(device="cpu"),
                        load_config=LoadConfig(load_format="dummy"))
        with set_current_vllm_config(vc):
            if not ps.model_parallel_is_initialized():
                ps.init_distributed_environment(
                    world_size=1, rank=0, local_rank=0, backend="gloo",
                    distributed_init_method=f"tcp://127.0.0.1:{29800 + os.getpid() % 150}")
                ps.initialize_model_parallel(1, 1)
            patches = []
            for m in PATCHED:
                mod = importlib.import_module(m)
                for fn, val in (("get_tensor_model_parallel_rank", rank),
                                ("get_tensor_model_parallel_world_size", TP)):
                    if hasattr(mod, fn):
                        patches.append(mock.patch.object(mod, fn, lambda v=val: v))
                if hasattr(mod, "Attention"):
                    patches.append(mock.patch.object(mod, "Attention", NoAttention))
            for p in patches:
                p.start()
            try:
                with set_default_torch_dtype(torch.bfloat16), torch.device("cpu"):
                    model = initialize_model(vllm_config=vc)
                model.load_weights(iter(weights))
                truth = {n: p.detach().clone() for n, p in model.named_parameters()}
                for p in model.parameters():
                    p.data.zero_()
                # min_row_bytes=0: transposed sources stay in the records, to check their geometry
                cap = captured_table(model, index, {path: image.address}, device=torch.device("cpu"),
                                     min_row_bytes=0)
                policy = captured_table(model, index, {path: image.address}, device=torch.device("cpu"))
                c_port.scatter2d(cap.records)
                twin_same = None
                if rank == 0:
                    # the refit receiver captures on a throw-away twin on `meta`
                    # (engines/vllm/refit/receiver.py:61-119): same copies as on the live model
                    from modelexpress_b200.geometry import capture_geometry
                    from modelexpress_b200.loader import torch_dtype

                    vc2 = VllmConfig(model_config=mc, device_config=DeviceConfig(device="cpu"),
                                     load_config=LoadConfig(load_format="dummy"))
                    with set_current_vllm_config(vc2):
                        with set_default_torch_dtype(torch.bfloat16), torch.device("meta"):
                            twin = initialize_model(vllm_config=vc2)
                    man = [(n, torch_dtype(i["dtype"]), tuple(i["shape"])) for n, i in index.items()]
                    live, meta = capture_geometry(model, man), capture_geometry(twin, man)
                    twin_same = (live.copies == meta.copies and live.unsupported == meta.unsupported
                                 and all(p.device.type == "meta" for p in twin.parameters()))
                if cap.reasons:  # what the loader computes on goes through the loader itself
                    model.load_weights((n, w) for n, w in weights if n in cap.reasons)
                # the same load with a staging buffer: transposing copies are staged as wide boxes
                from modelexpress_b200.planner import apply_converts

                twin_params = {n: p.detach().clone() for n, p in model.named_parameters()}
                for p in model.parameters():
                    p.data.zero_()
                held = []

                def alloc(nbytes):
                    held.append(torch.zeros(nbytes, dtype=torch.uint8))
                    return held[0].data_ptr()

                staged = captured_table(model, index, {path: image.address}, device=torch.device("cpu"),
                                        alloc_staging=alloc)
                c_port.scatter2d(staged.records)
                if staged.converts:
                    apply_converts(staged.converts, held[0], {n: p.data for n, p in model.named_parameters()})
                if staged.reasons:
                    model.load_weights((n, w) for n, w in weights if n in staged.reasons)
                staged_bad = [n for n, p in model.named_parameters()
                              if not torch.equal(p.data.view(torch.int16), truth[n].view(torch.int16))]
                for n, p in model.named_parameters():
                    p.data.copy_(twin_params[n])
            finally:
                for p in patches:
                    p.stop()
        bad = [n for n, p in model.named_parameters()
               if not torch.equal(p.data.view(torch.int16), truth[n].view(torch.int16))]
        recs = cap.records
        out[f"{arch}/rank{rank}"] = {
            "class": type(model).__name__, "params": len(truth), "copies": cap.copies,
            "records": int(len(recs)), "engine": sorted(cap.reasons), "mismatch": bad,
            "bytes": int(sum(int(r[2]) * int(r[3]) for r in recs)),
            "smallest_row": int(min((int(r[3]) for r in recs), default=0)),
            "left_to_engine_by_default": sorted(policy.reasons), "meta_twin_same": twin_same,
            "staged_mismatch": staged_bad, "staged_engine": sorted(staged.reasons),
            "staged_transposes": len([c for c in staged.converts if c.box_shape is not None]),
            "staged_smallest_row": int(min((int(r[3]) for r in staged.records), default=0))}
    image.close()


def main():
    out = {}
    for arch, (cfg_json, make_tensors) in ARCHS.items():
        try:
            run_arch(arch, cfg_json, make_tensors, out)
        except Exception as e:  # an architecture vLLM cannot build on the CPU here
            out[arch] = {"skipped": f"{type(e).__name__}: {e}"[:300]}
    print("RESULT " + json.dumps(out))


if __name__ == "__main__":
    main()
