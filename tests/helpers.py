"""Shared test helpers: synthetic checkpoints, oracle loading, record execution on the host."""

import os

import numpy as np

from oracle import c_port, ref_port

NP_OF_TAG = {"BF16": np.uint16, "F16": np.uint16, "F32": np.float32, "F8_E4M3": np.uint8,
             "F8_E5M2": np.uint8, "I32": np.int32, "I64": np.int64, "U8": np.uint8, "I8": np.int8,
             "I16": np.int16, "F64": np.float64, "BOOL": np.uint8}


def read_full_tensors(model_dir: str) -> dict:
    """Every checkpoint tensor as a raw-typed numpy array, through the ORACLE's
    header parser (so the product's parser is not trusted by the checker)."""
    out = {}
    files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    for fn in files:
        path = os.path.join(model_dir, fn)
        hdr = ref_port.parse_safetensors_header(path)
        raw = np.fromfile(path, dtype=np.uint8)
        for name, info in hdr.items():
            dt = NP_OF_TAG[info["dtype"]]
            a = raw[info["file_offset"]: info["file_offset"] + info["size"]].view(dt)
            out[name] = a.reshape(info["shape"]) if info["shape"] else a.reshape(())
    return out


def run_records_on_host(records) -> None:
    """Execute (src, dst, rows, row_bytes, src_pitch, dst_pitch) records whose
    addresses are HOST addresses with the oracle's C loop."""
    c_port.scatter2d([tuple(int(x) for x in r) for r in np.asarray(records).tolist()])


def tiny_dense_config():
    from modelexpress_b200.synth import DenseConfig

    return DenseConfig("tiny", layers=2, hidden=256, intermediate=512, q_heads=8, kv_heads=8,
                       head_dim=32, vocab=1024, qkv_bias=True, seed=7, files=2)
