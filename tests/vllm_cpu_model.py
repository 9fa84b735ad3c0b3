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

ARCHS = {
    "llama": ({"architectures": ["LlamaForCausalLM"], "model_type": "llama", "head_dim": 32}, False),
    "qwen2": ({"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2"}, True),
}
TP = 4


class NoAttention(torch.nn.Module):
    def __init__(self, *args, **kwargs):
        super().__init__()


def main():
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

    out = {}
    started = False
    for arch, (extra, bias) in ARCHS.items():
        d = tempfile.mkdtemp(prefix=f"mxb_{arch}_")
        cfg_json = {"hidden_size": 256, "intermediate_size": 512, "num_hidden_layers": 2,
                    "num_attention_heads": 8, "num_key_value_heads": 4, "vocab_size": 1000,
                    "max_position_embeddings": 512, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
                    "tie_word_embeddings": False, "torch_dtype": "bfloat16", "hidden_act": "silu",
                    "bos_token_id": 1, "eos_token_id": 2, **extra}
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg_json, f)
        cfg = synth.DenseConfig("tiny", layers=2, hidden=256, intermediate=512, q_heads=8, kv_heads=4,
                                head_dim=32, vocab=1000, qkv_bias=bias, seed=21, files=1)
        # random values for the norms too, so that a misplaced norm cannot pass
        tensors = [(n, s, dt, "matrix") for n, s, dt, _k in synth.dense_tensors(cfg)]
        synth.write_checkpoint(d, tensors, cfg.seed, 1)
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
                if not started:
                    ps.init_distributed_environment(
                        world_size=1, rank=0, local_rank=0, backend="gloo",
                        distributed_init_method=f"tcp://127.0.0.1:{29800 + os.getpid() % 150}")
                    ps.initialize_model_parallel(1, 1)
                    started = True
                patches = []
                for m in ("vllm.model_executor.layers.linear",
                          "vllm.model_executor.layers.vocab_parallel_embedding",
                          "vllm.model_executor.parameter", "vllm.model_executor.utils",
                          "vllm.distributed.parallel_state", "vllm.model_executor.models.llama",
                          "vllm.model_executor.models.qwen2"):
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
                    cap = captured_table(model, index, {path: image.address}, device=torch.device("cpu"))
                finally:
                    for p in patches:
                        p.stop()
            c_port.scatter2d(cap.records)
            bad = [n for n, p in model.named_parameters()
                   if not torch.equal(p.data.view(torch.int16), truth[n].view(torch.int16))]
            out[f"{arch}/rank{rank}"] = {
                "class": type(model).__name__, "params": len(truth), "copies": cap.copies,
                "records": int(len(cap.records)), "engine": sorted(cap.reasons), "mismatch": bad,
                "bytes": int(sum(int(r[2]) * int(r[3]) for r in cap.records))}
        image.close()
    print("RESULT " + json.dumps(out))


if __name__ == "__main__":
    main()
