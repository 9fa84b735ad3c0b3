"""Safetensors header and shard-index handling (host side, no tensor bytes).

Follows gds_loader.py:36-49 (dtype map), :189-243 (file discovery) and :245-282
(header parse) of the reference: same return shape, same rejections.
"""

from __future__ import annotations

import json
import struct
from collections import defaultdict
from pathlib import Path

MAX_HEADER_BYTES = 100 * 1024 * 1024

# safetensors dtype tag -> (bytes per element, torch dtype name)
SAFETENSORS_DTYPES = {
    "F64": (8, "float64"), "F32": (4, "float32"), "F16": (2, "float16"), "BF16": (2, "bfloat16"),
    "F8_E4M3": (1, "float8_e4m3fn"), "F8_E5M2": (1, "float8_e5m2"), "I64": (8, "int64"),
    "I32": (4, "int32"), "I16": (2, "int16"), "I8": (1, "int8"), "U8": (1, "uint8"),
    "BOOL": (1, "bool"),
}


def parse_safetensors_header(file_path: str) -> dict:
    """{tensor_name: {"file_offset": int, "size": int, "dtype": str, "shape": list}}"""
    with open(file_path, "rb") as f:
        raw = f.read(8)
        if len(raw) < 8:
            raise RuntimeError(f"Invalid safetensors file: {file_path}")
        (header_size,) = struct.unpack("<Q", raw)
        if header_size > MAX_HEADER_BYTES:
            raise RuntimeError(f"Safetensors header too large ({header_size} bytes): {file_path}")
        header_bytes = f.read(header_size)
    header = json.loads(header_bytes)
    data_start = 8 + header_size
    result = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        offsets = info["data_offsets"]
        dtype = info["dtype"]
        if dtype not in SAFETENSORS_DTYPES:
            raise RuntimeError(f"Unsupported safetensors dtype '{dtype}' for tensor '{name}'")
        result[name] = {
            "file_offset": data_start + offsets[0],
            "size": offsets[1] - offsets[0],
            "dtype": dtype,
            "shape": list(info["shape"]),
        }
    return result


def resolve_safetensors_files(model_path: str) -> dict:
    """{absolute file path: [tensor names]}: sharded index, single file, or glob."""
    model_dir = Path(model_path)
    index_path = model_dir / "model.safetensors.index.json"
    if index_path.exists():
        with open(index_path) as f:
            weight_map = json.load(f).get("weight_map", {})
        if not weight_map:
            raise RuntimeError(f"Empty weight_map in {index_path}")
        files = defaultdict(list)
        for tensor_name, filename in weight_map.items():
            files[str(model_dir / filename)].append(tensor_name)
        return dict(files)
    single = model_dir / "model.safetensors"
    if single.exists():
        return {str(single): list(parse_safetensors_header(str(single)).keys())}
    st_files = sorted(model_dir.glob("*.safetensors"))
    if not st_files:
        raise FileNotFoundError(f"No .safetensors files found in {model_path}")
    return {str(p): list(parse_safetensors_header(str(p)).keys()) for p in st_files}


def checkpoint_index(model_path: str) -> dict:
    """{tensor name: {"file", "file_offset", "size", "dtype", "shape"}} over all files."""
    out = {}
    for path in resolve_safetensors_files(model_path):
        for name, info in parse_safetensors_header(path).items():
            entry = dict(info)
            entry["file"] = path
            out[name] = entry
    return out
