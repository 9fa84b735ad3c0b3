"""Seeded synthetic checkpoints with the shapes of the benchmark configurations.

Real weights are not needed to exercise a byte mover; these stand in for the
Llama-3-8B / Qwen2.5-32B / DeepSeek-V3 checkpoints the reference is run on.
Files are genuine safetensors (8-byte little-endian header length, JSON header
padded with spaces to a multiple of 8, then the tensors back to back), written
in streaming fashion so a 16 GB checkpoint never has to sit in one buffer.
Matrices are N(0, 0.02) in bf16, norm weights are 1.0; the FP8 variant stores
``float8_e4m3fn`` values quantised per 128x128 block with fp32
``weight_scale_inv`` tensors.
"""

from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass

from .safetensors_index import SAFETENSORS_DTYPES


@dataclass(frozen=True)
class DenseConfig:
    name: str
    layers: int
    hidden: int
    intermediate: int
    q_heads: int
    kv_heads: int
    head_dim: int
    vocab: int
    qkv_bias: bool = False
    seed: int = 0
    files: int = 1


SMALL_LLAMA = DenseConfig("small-llama", 4, 1024, 2816, 16, 4, 64, 32000, False, 0, 1)
LLAMA3_8B = DenseConfig("llama3-8b", 32, 4096, 14336, 32, 8, 128, 128256, False, 1, 4)
QWEN25_32B = DenseConfig("qwen2.5-32b", 64, 5120, 27648, 40, 8, 128, 152064, True, 2, 17)


@dataclass(frozen=True)
class MoEConfig:
    name: str = "deepseek-v3-slice"
    layers: int = 4
    hidden: int = 7168
    experts: int = 256
    moe_intermediate: int = 2048
    q_lora: int = 1536
    kv_lora: int = 512
    qk_rope: int = 64
    qk_nope: int = 128
    v_head: int = 128
    heads: int = 128
    seed: int = 3
    files: int = 4
    block: int = 128


DEEPSEEK_V3_SLICE = MoEConfig()


def dense_tensors(cfg: DenseConfig) -> list:
    """[(name, shape, dtype tag, kind)] in HF order; kind is 'matrix' or 'norm' or 'bias'."""
    q, kv = cfg.q_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
    out = [("model.embed_tokens.weight", (cfg.vocab, cfg.hidden), "BF16", "matrix")]
    for i in range(cfg.layers):
        p = f"model.layers.{i}."
        out += [
            (p + "input_layernorm.weight", (cfg.hidden,), "BF16", "norm"),
            (p + "self_attn.q_proj.weight", (q, cfg.hidden), "BF16", "matrix"),
            (p + "self_attn.k_proj.weight", (kv, cfg.hidden), "BF16", "matrix"),
            (p + "self_attn.v_proj.weight", (kv, cfg.hidden), "BF16", "matrix"),
        ]
        if cfg.qkv_bias:
            out += [
                (p + "self_attn.q_proj.bias", (q,), "BF16", "bias"),
                (p + "self_attn.k_proj.bias", (kv,), "BF16", "bias"),
                (p + "self_attn.v_proj.bias", (kv,), "BF16", "bias"),
            ]
        out += [
            (p + "self_attn.o_proj.weight", (cfg.hidden, q), "BF16", "matrix"),
            (p + "post_attention_layernorm.weight", (cfg.hidden,), "BF16", "norm"),
            (p + "mlp.gate_proj.weight", (cfg.intermediate, cfg.hidden), "BF16", "matrix"),
            (p + "mlp.up_proj.weight", (cfg.intermediate, cfg.hidden), "BF16", "matrix"),
            (p + "mlp.down_proj.weight", (cfg.hidden, cfg.intermediate), "BF16", "matrix"),
        ]
    out += [("model.norm.weight", (cfg.hidden,), "BF16", "norm"),
            ("lm_head.weight", (cfg.vocab, cfg.hidden), "BF16", "matrix")]
    return out


def moe_tensors(cfg: MoEConfig) -> list:
    """DeepSeek-V3-style MoE layers: MLA attention + 256 routed experts + 1 shared
    expert, FP8 weights each followed by its fp32 block scale tensor."""
    b = cfg.block

    def fp8(name, shape):
        scale = tuple((s + b - 1) // b for s in shape)
        return [(name + ".weight", shape, "F8_E4M3", "fp8"),
                (name + ".weight_scale_inv", scale, "F32", "scale")]

    qk = cfg.qk_nope + cfg.qk_rope
    out = []
    for i in range(cfg.layers):
        p = f"model.layers.{i}."
        out += [(p + "input_layernorm.weight", (cfg.hidden,), "BF16", "norm")]
        out += fp8(p + "self_attn.q_a_proj", (cfg.q_lora, cfg.hidden))
        out += [(p + "self_attn.q_a_layernorm.weight", (cfg.q_lora,), "BF16", "norm")]
        out += fp8(p + "self_attn.q_b_proj", (cfg.heads * qk, cfg.q_lora))
        out += fp8(p + "self_attn.kv_a_proj_with_mqa", (cfg.kv_lora + cfg.qk_rope, cfg.hidden))
        out += [(p + "self_attn.kv_a_layernorm.weight", (cfg.kv_lora,), "BF16", "norm")]
        out += fp8(p + "self_attn.kv_b_proj", (cfg.heads * (cfg.qk_nope + cfg.v_head), cfg.kv_lora))
        out += fp8(p + "self_attn.o_proj", (cfg.hidden, cfg.heads * cfg.v_head))
        out += [(p + "post_attention_layernorm.weight", (cfg.hidden,), "BF16", "norm"),
                (p + "mlp.gate.weight", (cfg.experts, cfg.hidden), "BF16", "matrix"),
                (p + "mlp.gate.e_score_correction_bias", (cfg.experts,), "F32", "bias")]
        for e in range(cfg.experts):
            q = f"{p}mlp.experts.{e}."
            out += fp8(q + "gate_proj", (cfg.moe_intermediate, cfg.hidden))
            out += fp8(q + "up_proj", (cfg.moe_intermediate, cfg.hidden))
            out += fp8(q + "down_proj", (cfg.hidden, cfg.moe_intermediate))
        q = p + "mlp.shared_experts."
        out += fp8(q + "gate_proj", (cfg.moe_intermediate, cfg.hidden))
        out += fp8(q + "up_proj", (cfg.moe_intermediate, cfg.hidden))
        out += fp8(q + "down_proj", (cfg.hidden, cfg.moe_intermediate))
    return out


def tensor_nbytes(shape, dtype: str) -> int:
    n = SAFETENSORS_DTYPES[dtype][0]
    for s in shape:
        n *= int(s)
    return n


def _make(shape, dtype: str, kind: str, gen, device):
    """One synthetic tensor as a torch tensor on ``device`` in its storage dtype."""
    import torch

    if kind == "norm":
        return torch.ones(shape, dtype=torch.bfloat16, device=device)
    if kind == "scale":
        # amax of a 128x128 block of N(0, 0.02) sits near 0.08; scale = amax / 448
        return (torch.rand(shape, generator=gen, device=device, dtype=torch.float32) * 4e-5 + 1.6e-4)
    if kind == "fp8":
        w = torch.empty(shape, dtype=torch.float32, device=device).normal_(0.0, 0.02, generator=gen)
        return (w / 1.8e-4).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn)
    tdt = getattr(torch, SAFETENSORS_DTYPES[dtype][1])
    if tdt in (torch.float32, torch.bfloat16, torch.float16):
        return torch.empty(shape, dtype=torch.float32, device=device).normal_(
            0.0, 0.02, generator=gen).to(tdt)
    raise ValueError(f"no generator for {dtype}")


def write_checkpoint(out_dir: str, tensors: list, seed: int, files: int = 1, device="cpu") -> dict:
    """Write ``tensors`` ([(name, shape, dtype, kind)]) as ``files`` safetensors
    files plus ``model.safetensors.index.json``.  Returns {name: file path}.
    Values depend on (seed, position in the list, device type)."""
    import torch

    os.makedirs(out_dir, exist_ok=True)
    total = sum(tensor_nbytes(s, d) for _n, s, d, _k in tensors)
    per_file = (total + files - 1) // files
    groups, cur, acc = [], [], 0
    for t in tensors:
        cur.append(t)
        acc += tensor_nbytes(t[1], t[2])
        if acc >= per_file and len(groups) < files - 1:
            groups.append(cur)
            cur, acc = [], 0
    if cur:
        groups.append(cur)
    weight_map = {}
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    for fi, group in enumerate(groups):
        fname = ("model.safetensors" if len(groups) == 1
                 else f"model-{fi + 1:05d}-of-{len(groups):05d}.safetensors")
        header, off = {}, 0
        for name, shape, dtype, _kind in group:
            n = tensor_nbytes(shape, dtype)
            header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [off, off + n]}
            off += n
            weight_map[name] = fname
        hj = json.dumps(header, separators=(",", ":")).encode()
        hj += b" " * ((8 - len(hj) % 8) % 8)
        with open(os.path.join(out_dir, fname), "wb") as f:
            f.write(struct.pack("<Q", len(hj)))
            f.write(hj)
            for _name, shape, dtype, kind in group:
                t = _make(shape, dtype, kind, gen, device)
                raw = t.contiguous().view(torch.uint8).reshape(-1).cpu().numpy()
                f.write(memoryview(raw))
    if len(groups) > 1:
        with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f)
    return {n: os.path.join(out_dir, fn) for n, fn in weight_map.items()}


def ensure_checkpoint(out_dir: str, tensors: list, seed: int, files: int, device="cpu") -> str:
    """Write the checkpoint unless a complete one (marked by ``.complete``) is there."""
    marker = os.path.join(out_dir, ".complete")
    if not os.path.exists(marker):
        write_checkpoint(out_dir, tensors, seed, files, device)
        with open(marker, "w") as f:
            f.write("ok\n")
    return out_dir


def scaled(cfg: DenseConfig, layers: int | None = None, vocab: int | None = None) -> DenseConfig:
    """The same architecture with fewer layers / a smaller vocabulary (test sizes)."""
    from dataclasses import replace

    return replace(cfg, layers=layers if layers is not None else cfg.layers,
                   vocab=vocab if vocab is not None else cfg.vocab)
