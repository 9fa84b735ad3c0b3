"""Geometry capture on the CPU: what a loader's dry run records, what it refuses,
and — the parity part — that the compiled records move exactly the bytes the
loader itself moves when it is run for real (reference tests of the same
behaviour: tests/test_reshard_refit_geometry.py:88-240 for capture,
tests/test_reshard_refit_slice_plan.py for the resolved boxes)."""

import importlib
import os
from unittest import mock

import numpy as np
import pytest
import torch

from modelexpress_b200.geometry import (TracedSource, capture_geometry,
                                        summarize_unsupported)
from modelexpress_b200.loader import captured_table
from modelexpress_b200.planner import apply_converts
from oracle import c_port

G = os.path.join(os.path.dirname(__file__), "golden")
TAG = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.int32: "I32",
       torch.uint8: "U8"}


class Toy(torch.nn.Module):
    """Loader patterns met in engines: fused rows, a column slice, a transposed
    expert stack, a slice assignment, a device move, a padded table, a buffer."""

    def __init__(self, rank=1, tp=2):
        super().__init__()
        self.rank, self.tp = rank, tp
        self.qkv = torch.nn.Parameter(torch.zeros(8 + 4 + 4, 16))
        self.down = torch.nn.Parameter(torch.zeros(16, 12))
        self.experts = torch.nn.Parameter(torch.zeros(3, 6, 16))
        self.norm = torch.nn.Parameter(torch.zeros(16))
        self.embed = torch.nn.Parameter(torch.ones(24, 16))
        self.router = torch.nn.Parameter(torch.zeros(3, 16, dtype=torch.float32))
        self.scale = torch.nn.Parameter(torch.zeros(1))
        self.doubled = torch.nn.Parameter(torch.zeros(16))
        self.register_buffer("table", torch.zeros(4, 4))

    def load_weights(self, weights):
        done = set()
        for name, w in weights:
            done.add(name)
            if name in ("q", "k", "v"):
                rows = {"q": 8, "k": 4, "v": 4}[name]
                at = {"q": 0, "k": 8, "v": 12}[name]
                self.qkv.data.narrow(0, at, rows).copy_(w.narrow(0, self.rank * rows, rows))
            elif name == "down":
                self.down.data.copy_(w[:, self.rank * 12:(self.rank + 1) * 12])
            elif name == "experts_t":      # stored (E, hidden, inter): transposed per expert
                for e, we in enumerate(w.unbind(0)):
                    self.experts.data[e].copy_(we.t().narrow(0, self.rank * 6, 6))
            elif name == "norm":
                self.norm.data[:] = w.to(self.norm.device)
            elif name == "embed":          # 20 real rows, 24 padded
                self.embed.data[: w.shape[0]].copy_(w)
                self.embed.data[w.shape[0]:].fill_(0)
            elif name == "router":         # served bf16, kept fp32
                self.router.data.copy_(w)
            elif name == "scale":
                self.scale.data.fill_(w.item())
            elif name == "table":
                self.table.copy_(w.squeeze(0))
            elif name == "cast":
                self.doubled.data.copy_(w.float() * 2)
            elif name == "temp":
                tmp = torch.empty(16)
                tmp.copy_(w)
                self.norm.data.copy_(tmp + 1)
            elif name == "skipme":
                done.discard(name)
        return done


MANIFEST = [("q", torch.float32, (16, 16)), ("k", torch.float32, (8, 16)), ("scale", torch.float32, (1,)),
            ("v", torch.float32, (8, 16)), ("down", torch.float32, (16, 24)),
            ("experts_t", torch.float32, (3, 16, 12)), ("cast", torch.bfloat16, (16,)),
            ("norm", torch.float32, (16,)), ("embed", torch.float32, (20, 16)),
            ("router", torch.bfloat16, (3, 16)), ("table", torch.float32, (1, 4, 4)),
            ("temp", torch.float32, (16,)), ("skipme", torch.float32, (5,))]


def test_capture_records_windows_and_destinations():
    cap = capture_geometry(Toy(), MANIFEST)
    by = {}
    for c in cap.copies:
        by.setdefault(c.src_name, []).append(c)
    q, = by["q"]
    assert (q.src_offset, q.src_shape, q.src_stride) == (8 * 16, (8, 16), (16, 1))
    assert (q.param_name, q.dest_offset, q.dest_shape, q.dest_stride) == ("qkv", 0, (8, 16), (16, 1))
    assert by["k"][0].dest_offset == 8 * 16 and by["v"][0].dest_offset == 12 * 16
    d, = by["down"]
    assert (d.src_offset, d.src_stride, d.dest_stride) == (12, (24, 1), (12, 1))
    ex = by["experts_t"]
    assert [c.src_offset for c in ex] == [e * 16 * 12 + 6 for e in range(3)]
    assert all(c.src_shape == (6, 16) and c.src_stride == (1, 12) for c in ex)
    assert [c.dest_offset for c in ex] == [0, 96, 192]
    assert by["norm"][0].param_name == "norm" and by["embed"][0].dest_shape == (20, 16)
    assert by["router"][0].src_dtype == torch.bfloat16 and by["router"][0].dest_dtype == torch.float32
    assert by["table"][0].param_name == "table" and by["table"][0].src_shape == (4, 4)
    assert "skipme" not in by and "skipme" not in cap.unsupported


def test_unsupported_sources_are_isolated_with_their_cause():
    cap = capture_geometry(Toy(), MANIFEST)
    assert cap.unsupported == ["scale", "cast", "temp"]
    assert "item" in cap.unsupported_reasons["scale"]
    assert "float" in cap.unsupported_reasons["cast"]
    assert "not a parameter" in cap.unsupported_reasons["temp"] and cap.unattributed == 1
    assert not [c for c in cap.copies if c.src_name in cap.unsupported]
    # sources before, between and after the failing ones were all captured, once each
    names = [c.src_name for c in cap.copies]
    assert names.count("q") == names.count("v") == names.count("norm") == names.count("table") == 1
    assert names.count("experts_t") == 3


def test_one_call_and_one_call_per_source_agree():
    a = capture_geometry(Toy(), MANIFEST)
    b = capture_geometry(Toy(), MANIFEST, isolate=True)
    assert a.copies == b.copies and a.unsupported == b.unsupported


def test_summarize_unsupported_groups_causes():
    got = summarize_unsupported({"a": "x", "b": "y", "c": "x"})
    assert got == [("x", 2), ("y", 1)] and summarize_unsupported(None) == []


def test_traced_source_answers_metadata_and_refuses_data():
    t = TracedSource.source("w", (4, 6), torch.bfloat16, "cpu")
    assert t.shape == (4, 6) and t.dtype == torch.bfloat16 and t.dim() == 2 and t.numel() == 24
    assert t.device.type == "cpu" and t.is_contiguous() and t.size(1) == 6
    v = t.t()
    assert isinstance(v, TracedSource) and v.shape == (6, 4) and not v.is_contiguous()
    assert t.to("cpu") is t and t.to(torch.bfloat16) is t
    a, b = t.chunk(2, dim=1)
    assert a.shape == (4, 3) and b._window.storage_offset() == 3
    for bad in (lambda: t + 1, lambda: t.float(), lambda: v.contiguous(), lambda: t.sum().item(),
                lambda: torch.cat([t, t]), lambda: t.view(torch.int16), lambda: t.clone()):
        with pytest.raises(NotImplementedError):
            bad()
    assert v.t().contiguous().shape == (4, 6)   # contiguous() of a dense window is still a view


def _image(manifest, seed=0):
    """An in-memory 'file': tensors back to back at odd offsets, plus an index in
    the shape checkpoint_index returns."""
    rng = np.random.default_rng(seed)
    index, chunks, at = {}, [], 0
    for name, dtype, shape in manifest:
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        pad = int(rng.integers(0, 3)) * 2
        chunks.append(np.zeros(pad, dtype=np.uint8))
        at += pad
        if dtype in (torch.float32,):
            raw = rng.standard_normal(int(np.prod(shape))).astype(np.float32).view(np.uint8)
        else:                          # bf16: any bit pattern without NaN/Inf exponents
            u = rng.integers(0, 0x7F00, size=int(np.prod(shape)), dtype=np.uint16)
            raw = u.view(np.uint8)
        chunks.append(raw)
        index[name] = {"file": "mem", "file_offset": at, "size": n, "dtype": TAG[dtype], "shape": list(shape)}
        at += n
    return np.concatenate(chunks), index


def _real_tensor(image, info, dtype):
    raw = torch.from_numpy(image[info["file_offset"]: info["file_offset"] + info["size"]].copy())
    return raw.view(dtype).reshape(info["shape"])


def _run_records(model, image, index, manifest):
    """Compile the capture and move the bytes with the CPU scatter (the checker)."""
    staging = []

    def alloc(nbytes):
        staging.append(torch.zeros(nbytes, dtype=torch.uint8))
        return staging[0].data_ptr()

    cap = captured_table(model, index, {"mem": image.ctypes.data}, device=torch.device("cpu"),
                         alloc_staging=alloc)
    c_port.scatter2d(cap.records)
    if cap.converts:
        dests = {n: p.data for n, p in model.named_parameters()}
        apply_converts(cap.converts, staging[0], dests)
    left = [(n, _real_tensor(image, index[n], dt)) for n, dt, _s in manifest if n in cap.reasons]
    model.load_weights(iter(left))
    return cap


@pytest.mark.parametrize("rank", [0, 1])
def test_records_move_what_the_loader_moves(rank):
    manifest = [m for m in MANIFEST if m[0] != "temp"]
    image, index = _image(manifest, seed=rank)
    truth = Toy(rank)
    truth.load_weights((n, _real_tensor(image, index[n], dt)) for n, dt, _s in manifest)
    model = Toy(rank)
    cap = _run_records(model, image, index, manifest)
    assert sorted(cap.reasons) == ["cast", "scale"]
    assert [c.param_name for c in cap.converts] == ["router"]
    assert cap.written_params == {"qkv", "down", "experts", "norm", "embed", "router", "table"}
    for (n, a), (_n, b) in zip(model.state_dict().items(), truth.state_dict().items()):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), n


def test_without_staging_a_dtype_change_goes_to_the_engine():
    image, index = _image(MANIFEST[:1] + [m for m in MANIFEST if m[0] == "router"])
    cap = captured_table(Toy(), index, {"mem": image.ctypes.data}, device=torch.device("cpu"))
    assert list(cap.reasons) == ["router"] and not cap.converts and cap.copies == 1


def test_captured_copies_plan_against_row_sharded_sources():
    """The refit case: the same captured copies, but every source tensor is
    published as three row shards living in separate buffers (the trainer's
    layout, slice_plan.py:54-70); the records must still assemble what the
    loader assembles from the full tensors."""
    from modelexpress_b200.planner import ShardSpec, SourceSpec, plan_transfer_2d

    manifest = [m for m in MANIFEST if m[0] in ("q", "k", "v", "down", "experts_t", "norm", "embed", "table")]
    image, index = _image(manifest, seed=7)
    full = {n: _real_tensor(image, index[n], dt) for n, dt, _s in manifest}
    truth = Toy(1)
    truth.load_weights(iter(full.items()))
    model = Toy(1)
    cap = capture_geometry(model, manifest)
    keep, sources = [], {}
    for name, t in full.items():
        rows = t.shape[0]
        cuts = sorted({0, rows // 3, (2 * rows) // 3, rows})
        shards = []
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            part = t[lo:hi].contiguous()
            keep.append(part)
            shards.append(ShardSpec((lo,) + (0,) * (t.dim() - 1), tuple(part.shape), f"{name}@{lo}",
                                    part.data_ptr(), t.element_size()))
        sources[name] = SourceSpec(tuple(t.shape), t.dtype, t.element_size(), shards)
    dests = dict(model.named_parameters())
    dests.update(dict(model.named_buffers()))
    table, unsupported, converts = plan_transfer_2d(cap.copies, sources, lambda n: dests[n].data_ptr())
    assert not unsupported and not converts
    c_port.scatter2d(table)
    for (n, a), (_n, b) in zip(model.state_dict().items(), truth.state_dict().items()):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), n


def test_fused_gqa_trainer_storage_as_many_shards_per_source():
    """Sources published the way a Megatron trainer holds them: ONE fused QKV
    tensor interleaved per KV group ([q_g; k_g; v_g] for each group g), exposed
    as per-group alias shards of the HF q / k / v tensors
    (modelexpress_rl/train/engines/megatron/aliases.py; the reference pins these
    boxes in tests/test_reshard_megatron_gqa.py:195-342).  The captured copies of
    a fused-qkv loader must pull the right group rows straight out of the
    interleaved storage."""
    from modelexpress_b200.planner import ShardSpec, SourceSpec, plan_transfer_2d

    groups, q_rows, kv_rows, cols = 4, 4, 2, 16         # per group: 4 q rows, 2 k rows, 2 v rows
    per_group = q_rows + 2 * kv_rows
    fused = torch.randn(groups * per_group, cols)
    rows = fused.view(groups, per_group, cols)
    full = {"q": rows[:, :q_rows].reshape(-1, cols).contiguous(),
            "k": rows[:, q_rows:q_rows + kv_rows].reshape(-1, cols).contiguous(),
            "v": rows[:, q_rows + kv_rows:].reshape(-1, cols).contiguous()}
    el = fused.element_size()
    sources = {}
    for name, first, n in (("q", 0, q_rows), ("k", q_rows, kv_rows), ("v", q_rows + kv_rows, kv_rows)):
        shards = [ShardSpec((g * n, 0), (n, cols), f"trainer/{name}/{g}",
                            fused.data_ptr() + (g * per_group + first) * cols * el, el)
                  for g in range(groups)]
        sources[name] = SourceSpec((groups * n, cols), torch.float32, el, shards)
    manifest = [(n, torch.float32, tuple(t.shape)) for n, t in full.items()]
    for rank in (0, 1):
        truth = Toy(rank)
        truth.load_weights(iter(full.items()))
        model = Toy(rank)
        cap = capture_geometry(model, manifest)
        table, unsupported, converts = plan_transfer_2d(
            cap.copies, sources, lambda n: dict(model.named_parameters())[n].data_ptr())
        assert not unsupported and not converts
        # rank r keeps q rows [8r, 8r+8) = groups 2r, 2r+1 and k/v rows [4r, 4r+4): two shards each
        assert len(table) == 6 and int(table[:, 2].astype(np.int64).sum()) == 6
        c_port.scatter2d(table)
        assert torch.equal(model.qkv.data, truth.qkv.data), rank


class PostProcessing(torch.nn.Module):
    """Loaders that keep working on a parameter after copying into it."""

    def __init__(self):
        super().__init__()
        self.scaled = torch.nn.Parameter(torch.zeros(8, 8))
        self.plain = torch.nn.Parameter(torch.zeros(8, 8))
        self.derived = torch.nn.Parameter(torch.zeros(8))
        self.padded = torch.nn.Parameter(torch.ones(12, 8))

    def load_weights(self, weights):
        for name, w in weights:
            if name == "scaled":
                self.scaled.data.copy_(w)
                self.scaled.data.mul_(0.5)                 # in place, after the copy
            elif name == "plain":
                self.plain.data.copy_(w)
            elif name == "derived_from_plain":
                self.derived.data.copy_(self.plain.data.sum(0))   # reads what "plain" wrote
            elif name == "padded":
                self.padded.data[:8].copy_(w)
                self.padded.data[8:].fill_(0)              # other rows: harmless


def test_work_on_a_destination_after_the_copy_gives_the_source_up():
    manifest = [("scaled", torch.float32, (8, 8)), ("plain", torch.float32, (8, 8)),
                ("padded", torch.float32, (8, 8)), ("derived_from_plain", torch.float32, (1,))]
    cap = capture_geometry(PostProcessing(), manifest)
    assert sorted(cap.unsupported) == ["derived_from_plain", "plain", "scaled"]
    assert "mul_" in cap.unsupported_reasons["scaled"] and "after the copy" in cap.unsupported_reasons["scaled"]
    assert "sum" in cap.unsupported_reasons["plain"]
    assert "'plain' provides" in cap.unsupported_reasons["derived_from_plain"]
    assert [c.src_name for c in cap.copies] == ["padded"]
    # end to end: records for what was captured, the loader itself for the rest
    image, index = _image(manifest[:3], seed=3)
    truth = PostProcessing()
    truth.load_weights([(n, _real_tensor(image, index[n], dt)) for n, dt, _s in manifest[:3]]
                       + [("derived_from_plain", torch.zeros(1))])
    model = PostProcessing()
    index["derived_from_plain"] = {"file": "mem", "file_offset": 0, "size": 4, "dtype": "F32", "shape": [1]}
    cap = _run_records(model, image, index, manifest)
    # the dependent source is re-run by the loader after the bytes it reads are in place
    assert sorted(cap.reasons) == ["derived_from_plain", "plain", "scaled"]
    for (n, a), (_n, b) in zip(model.state_dict().items(), truth.state_dict().items()):
        assert torch.equal(a, b), n


def test_parts_of_one_checkpoint_share_what_was_recorded():
    """A checkpoint compiled part by part (as the pipelined load does): the loader of
    a later part that reads bytes an earlier part provides is still noticed, and
    the earlier source is reported by the later call."""
    from modelexpress_b200.geometry import CaptureState

    model = PostProcessing()
    state = CaptureState(model)
    first = capture_geometry(model, [("plain", torch.float32, (8, 8)), ("padded", torch.float32, (8, 8))],
                             state=state)
    assert first.unsupported == [] and [c.src_name for c in first.copies] == ["plain", "padded"]
    second = capture_geometry(model, [("derived_from_plain", torch.float32, (1,))], state=state)
    assert sorted(second.unsupported) == ["derived_from_plain", "plain"] and second.copies == []
    # without the shared state the second call cannot know
    alone = capture_geometry(PostProcessing(), [("derived_from_plain", torch.float32, (1,))])
    assert alone.unsupported == []


# ---- real vLLM parallel layers, checked against outputs recorded from vLLM itself --------------

def _vllm_mini(rank, tp, dims):
    """A module made of vLLM's own QKV / merged-column / row-parallel /
    vocab-parallel layers with the usual stacked-parameter ``load_weights``."""
    from vllm.config import DeviceConfig, VllmConfig, set_current_vllm_config
    from vllm.model_executor.layers import linear as L
    from vllm.model_executor.layers import vocab_parallel_embedding as V
    from vllm.model_executor.model_loader.weight_utils import default_weight_loader

    h, qh, kvh, hd, inter, voc = dims
    patches = []
    for m in ("vllm.model_executor.layers.linear", "vllm.model_executor.layers.vocab_parallel_embedding",
              "vllm.model_executor.parameter", "vllm.model_executor.utils",
              "vllm.distributed.parallel_state"):
        mod = importlib.import_module(m)
        for fn, val in (("get_tensor_model_parallel_rank", rank),
                        ("get_tensor_model_parallel_world_size", tp)):
            if hasattr(mod, fn):
                patches.append(mock.patch.object(mod, fn, lambda v=val: v))

    class Mini(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.qkv_proj = L.QKVParallelLinear(h, hd, qh, kvh, bias=True)
            self.gate_up_proj = L.MergedColumnParallelLinear(h, [inter, inter], bias=False)
            self.o_proj = L.RowParallelLinear(qh * hd, h, bias=False)
            self.down_proj = L.RowParallelLinear(inter, h, bias=False)
            self.embed_tokens = V.VocabParallelEmbedding(voc, h)

        def load_weights(self, weights):
            stacked = [("qkv_proj", "q_proj", "q"), ("qkv_proj", "k_proj", "k"), ("qkv_proj", "v_proj", "v"),
                       ("gate_up_proj", "gate_proj", 0), ("gate_up_proj", "up_proj", 1)]
            params = dict(self.named_parameters())
            for name, w in weights:
                for fused, part, shard_id in stacked:
                    if part in name:
                        p = params[name.replace(part, fused)]
                        p.weight_loader(p, w, shard_id)
                        break
                else:
                    p = params[name]
                    getattr(p, "weight_loader", default_weight_loader)(p, w)

    cfg = VllmConfig(device_config=DeviceConfig(device="cpu"))
    return Mini, patches, cfg, set_current_vllm_config


def test_capture_of_real_vllm_layers_matches_recorded_vllm_outputs():
    pytest.importorskip("vllm")
    z = np.load(os.path.join(G, "vllm_layers.npz"))
    tp, h, qh, kvh, hd, inter, voc = (int(x) for x in z["meta"])
    src = {"q_proj.weight": "q_proj", "k_proj.weight": "k_proj", "v_proj.weight": "v_proj",
           "q_proj.bias": "q_bias", "k_proj.bias": "k_bias", "v_proj.bias": "v_bias",
           "gate_proj.weight": "gate_proj", "up_proj.weight": "up_proj", "o_proj.weight": "o_proj",
           "down_proj.weight": "down_proj", "embed_tokens.weight": "embed"}
    chunks, index, at = [], {}, 0
    for name, key in src.items():
        a = np.ascontiguousarray(z[f"src/{key}"].astype(np.uint16))
        chunks.append(a.reshape(-1).view(np.uint8))
        index[name] = {"file": "mem", "file_offset": at, "size": a.nbytes, "dtype": "BF16",
                       "shape": list(a.shape)}
        at += a.nbytes
    image = np.concatenate(chunks)
    want = {"qkv_proj.weight": "qkv_w", "qkv_proj.bias": "qkv_b", "gate_up_proj.weight": "gate_up",
            "o_proj.weight": "o", "down_proj.weight": "down", "embed_tokens.weight": "embed"}
    for rank in range(tp):
        Mini, patches, cfg, use = _vllm_mini(rank, tp, (h, qh, kvh, hd, inter, voc))
        for p in patches:
            p.start()
        try:
            with use(cfg):
                torch.set_default_dtype(torch.bfloat16)
                try:
                    model = Mini()
                finally:
                    torch.set_default_dtype(torch.float32)
                cap = captured_table(model, index, {"mem": image.ctypes.data}, device=torch.device("cpu"))
        finally:
            for p in patches:
                p.stop()
        assert not cap.reasons and cap.copies == len(src)
        c_port.scatter2d(cap.records)
        for pname, key in want.items():
            got = dict(model.named_parameters())[pname].data.contiguous().view(torch.int16).numpy().view(np.uint16)
            assert np.array_equal(got, z[f"rank{rank}/{key}"]), (rank, pname)


def test_whole_vllm_models_on_cpu_every_tp_rank():
    """Real vLLM ``LlamaForCausalLM``, ``Qwen2ForCausalLM`` (q/k/v biases),
    ``Phi3ForCausalLM`` (projections fused on disk) and ``GPT2LMHeadModel`` (transposed
    Conv1D weights, tied embeddings) built on the CPU, tensor-parallel size 4, every rank: records compiled from the dry run
    of the model's own ``load_weights`` reproduce what ``load_weights`` produces,
    bit for bit, with nothing left to the engine.  Runs in a child process (vLLM's
    parallel state is global)."""
    pytest.importorskip("vllm")
    import json
    import subprocess
    import sys

    helper = os.path.join(os.path.dirname(__file__), "vllm_cpu_model.py")
    run = subprocess.run([sys.executable, helper], capture_output=True, text=True, timeout=900)
    lines = [ln for ln in run.stdout.splitlines() if ln.startswith("RESULT ")]
    if run.returncode != 0 or not lines:
        pytest.skip("vLLM could not build a model on the CPU here: " + run.stderr.strip()[-400:])
    res = json.loads(lines[-1][len("RESULT "):])
    archs = ("llama", "qwen2", "phi3", "gpt2")
    built = [a for a in archs if a not in res]          # an arch that could not be built is listed bare
    assert {"llama", "qwen2"} <= set(built), res
    for a in built:
        for r in range(4):
            got = res[f"{a}/rank{r}"]
            assert got["mismatch"] == [] and got["engine"] == [], (a, r, got)
        # a twin of the model on `meta` (what a refit receiver captures on) records the same copies
        assert res[f"{a}/rank0"]["meta_twin_same"] is True, a
    for a, copies in (("llama", 21), ("qwen2", 27), ("phi3", 21)):   # phi3: q/k/v and gate/up fused on disk
        if a in built:
            assert all(res[f"{a}/rank{r}"]["copies"] == res[f"{a}/rank{r}"]["records"] == copies
                       and res[f"{a}/rank{r}"]["left_to_engine_by_default"] == [] for r in range(4)), a
    if "gpt2" in built:
        # Conv1D weights are transposed by the loader: exact as records (two-byte rows), but by
        # default those eight tensors go to the engine's loader instead
        g = res["gpt2/rank0"]
        assert g["smallest_row"] == 2 and g["records"] > 1000
        assert len(g["left_to_engine_by_default"]) == 8
        assert all(n.endswith(("c_attn.weight", "c_proj.weight", "c_fc.weight"))
                   for n in g["left_to_engine_by_default"])
        # with a staging buffer the same eight tensors are staged as wide boxes and transposed on
        # the device: nothing is left to the engine and no narrow record remains
        for r in range(4):
            gs = res[f"gpt2/rank{r}"]
            # 12 copies: c_attn lands as q, k and v, the other three Conv1D weights as one each
            assert gs["staged_mismatch"] == [] and gs["staged_engine"] == [] and gs["staged_transposes"] == 12
            assert gs["staged_smallest_row"] >= 64
    for a in built:
        for r in range(4):
            assert res[f"{a}/rank{r}"]["staged_mismatch"] == [], (a, r)
    # vocabulary 1000 pads to 1024: the last rank's embed and lm_head shards hold 24 real rows
    # fewer (x 256 columns x 2 bytes x 2 tensors) than the other ranks'
    for arch in ("llama", "qwen2"):
        b = [res[f"{arch}/rank{r}"]["bytes"] for r in range(4)]
        assert b[0] == b[1] == b[2] and b[0] - b[3] == 2 * 24 * 256 * 2


def test_capture_resolves_to_the_boxes_the_reference_resolves():
    """Pinned against the reference itself: ``capture_pin.json`` holds what the
    reference's capture_geometry + resolve_slice make of tests/hooked_model.py
    (fused qkv with shard ids, gate/up, a pre-merged tensor split with chunk, row
    and column parallel, a transposed source, per-expert tensors into a stacked
    parameter, a padded vocabulary, a default-loader parameter).  This repository's
    capture of the same model must resolve every copy to the same source box,
    landing place and destination strides."""
    import json
    import sys

    sys.path.insert(0, os.path.dirname(__file__))
    import hooked_model as H
    from modelexpress_b200.planner import resolve_slice

    with open(os.path.join(G, "capture_pin.json")) as f:
        pin = json.load(f)
    assert pin["unsupported"] == [] and pin["unattributed"] == 0
    shapes = {n: s for n, _d, s in H.manifest()}
    for device in ("cpu", "meta"):
        with torch.device(device):
            model = H.HookedModel()
        cap = capture_geometry(model, H.manifest())
        assert cap.unsupported == [] and cap.unattributed == 0
        got = []
        for c in cap.copies:
            box, dstride = resolve_slice(c, shapes[c.src_name])
            got.append({"src": c.src_name, "param": c.param_name, "dest_offset": c.dest_offset,
                        "dest_shape": list(c.dest_shape), "box": [list(b) for b in box],
                        "dest_stride_src": list(dstride)})
        want = [c for c in pin["copies"] if "unsupported" not in c]
        assert len(want) == len(pin["copies"]) == len(got)
        key = lambda r: (r["src"], r["param"], r["dest_offset"])  # noqa: E731
        assert sorted(got, key=key) == sorted(want, key=key), device


@pytest.mark.parametrize("seed", range(6))
def test_random_view_chains_move_what_torch_moves(seed):
    """Fuzz: a random chain of view ops (narrow, slicing, transpose, permute, select,
    unsqueeze/squeeze, chunk, unbind, t) applied to a placeholder and to a real
    tensor, copied into a random strided window of a destination.  Whenever the
    planner accepts the copy, the records executed by the CPU scatter must equal
    torch's own ``copy_``; when it refuses, it must refuse before moving anything."""
    from modelexpress_b200.planner import ShardSpec, SourceSpec, plan_transfer_2d

    rng = np.random.default_rng(1000 + seed)
    accepted = 0
    for _case in range(40):
        nd = int(rng.integers(1, 4))
        shape = tuple(int(rng.integers(1, 7)) for _ in range(nd))
        real = torch.arange(int(np.prod(shape)), dtype=torch.float32).reshape(shape) + 1

        def chain(t):
            ops = []
            for _ in range(int(rng.integers(0, 4))):
                kind = rng.choice(["narrow", "slice", "transpose", "permute", "select", "unsqueeze",
                                   "squeeze", "chunk", "unbind", "t"])
                d = int(rng.integers(0, max(1, t.dim()))) if t.dim() else 0
                if kind == "narrow" and t.dim():
                    lo = int(rng.integers(0, t.shape[d]))
                    ops.append(("narrow", (d, lo, int(rng.integers(1, t.shape[d] - lo + 1)))))
                elif kind == "slice" and t.dim():
                    lo = int(rng.integers(0, t.shape[0]))
                    ops.append(("getitem", (slice(lo, int(rng.integers(lo + 1, t.shape[0] + 1))),)))
                elif kind == "transpose" and t.dim() >= 2:
                    ops.append(("transpose", (d, int(rng.integers(0, t.dim())))))
                elif kind == "permute" and t.dim() >= 2:
                    ops.append(("permute", (tuple(int(x) for x in rng.permutation(t.dim())),)))
                elif kind == "select" and t.dim() >= 2:
                    ops.append(("select", (d, int(rng.integers(0, t.shape[d])))))
                elif kind == "unsqueeze":
                    ops.append(("unsqueeze", (int(rng.integers(0, t.dim() + 1)),)))
                elif kind == "squeeze":
                    ops.append(("squeeze", ()))
                elif kind == "chunk" and t.dim() and t.shape[d] >= 2:
                    ops.append(("chunk", (2, d, int(rng.integers(0, 2)))))
                elif kind == "unbind" and t.dim() >= 2:
                    ops.append(("unbind", (d, int(rng.integers(0, t.shape[d])))))
                elif kind == "t" and t.dim() == 2:
                    ops.append(("t", ()))
                else:
                    continue
                t = apply(t, ops[-1])
            return ops

        def apply(t, op):
            name, args = op
            if name == "getitem":
                return t[args[0]]
            if name == "chunk":
                return t.chunk(args[0], dim=args[1])[args[2]]
            if name == "unbind":
                return t.unbind(args[0])[args[1]]
            return getattr(t, name)(*args)

        ops = chain(real)
        view = real
        for op in ops:
            view = apply(view, op)
        if view.numel() == 0:
            continue
        # destination: a parameter with room for a strided window of the view's shape
        pad = int(rng.integers(0, 3))
        dest_full = torch.zeros(tuple(s + pad for s in view.shape) if view.dim() else (1 + pad,))

        class One(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.p = torch.nn.Parameter(dest_full.clone())

            def window(self):
                w = self.p.data
                if view.dim() == 0:
                    return w[pad]
                for dim, n in enumerate(view.shape):
                    w = w.narrow(dim, pad, n)
                return w

            def load_weights(self, weights):
                for _name, w in weights:
                    for op in ops:
                        w = apply(w, op)
                    self.window().copy_(w)

        truth = One()
        truth.load_weights([("w", real)])
        model = One()
        cap = capture_geometry(model, [("w", torch.float32, shape)])
        assert cap.unsupported == [] and len(cap.copies) == 1
        # the source is published whole, or cut into two or three shards along a random dim
        keep, shards = [], []
        cut_dim = int(rng.integers(0, nd))
        pieces = int(rng.integers(1, 4))
        edges = sorted({0, shape[cut_dim], *[int(x) for x in rng.integers(0, shape[cut_dim] + 1, pieces - 1)]})
        for lo, hi in zip(edges[:-1], edges[1:]):
            part = real.narrow(cut_dim, lo, hi - lo).contiguous()
            keep.append(part)
            off = [0] * nd
            off[cut_dim] = lo
            shards.append(ShardSpec(tuple(off), tuple(part.shape), f"s{lo}", part.data_ptr(), 4))
        sources = {"w": SourceSpec(shape, torch.float32, 4, shards)}
        table, unsupported, _cv = plan_transfer_2d(cap.copies, sources, lambda n: model.p.data_ptr())
        if unsupported:
            assert len(table) == 0 and float(model.p.detach().abs().sum()) == 0.0
            continue
        accepted += 1
        c_port.scatter2d(table)
        assert torch.equal(model.p.detach(), truth.p.detach()), (shape, ops)
    assert accepted >= 20


def test_tied_and_arena_backed_parameters():
    """Destinations are found by storage: a parameter registered under two names (tied
    embeddings) and parameters that are views into one flat arena (storage offset
    not zero) both resolve to offsets relative to the parameter itself."""
    class Tied(torch.nn.Module):
        def __init__(self):
            super().__init__()
            arena = torch.zeros(4 * 8 + 6 * 8 + 5)
            self.embed = torch.nn.Parameter(torch.zeros(4, 8))
            self.head = self.embed                                  # tied
            self.a = torch.nn.Parameter(torch.zeros(1))
            self.b = torch.nn.Parameter(torch.zeros(1))
            self.a.data = arena[5:5 + 32].view(4, 8)                # views into the arena
            self.b.data = arena[5 + 32:5 + 32 + 48].view(6, 8)

        def load_weights(self, weights):
            for name, w in weights:
                if name == "head":
                    self.head.data.copy_(w)
                elif name == "a":
                    self.a.data.copy_(w)
                elif name == "b_rows":
                    self.b.data[2:5].copy_(w.narrow(0, 1, 3))

    manifest = [("head", torch.float32, (4, 8)), ("a", torch.float32, (4, 8)),
                ("b_rows", torch.float32, (6, 8))]
    model = Tied()
    cap = capture_geometry(model, manifest)
    by = {c.src_name: c for c in cap.copies}
    assert cap.unsupported == [] and by["head"].param_name in ("embed", "head")
    assert (by["a"].param_name, by["a"].dest_offset) == ("a", 0)
    assert (by["b_rows"].param_name, by["b_rows"].dest_offset, by["b_rows"].src_offset) == ("b", 16, 8)
    image, index = _image(manifest, seed=9)
    truth = Tied()
    truth.load_weights((n, _real_tensor(image, index[n], dt)) for n, dt, _s in manifest)
    cap = _run_records(model, image, index, manifest)
    assert not cap.reasons
    for name in ("embed", "a", "b"):
        assert torch.equal(getattr(model, name).data, getattr(truth, name).data), name
    assert model.head is model.embed


def test_scalars_empty_tensors_and_integer_indices():
    """Edge shapes: a 0-d source, a 0-d source viewed as (1,), an empty tensor (no
    record at all) and an integer index that drops a dimension."""
    from modelexpress_b200.planner import ShardSpec, SourceSpec, plan_transfer_2d

    class Edge(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.s0 = torch.nn.Parameter(torch.zeros(()))
            self.s1 = torch.nn.Parameter(torch.zeros(1))
            self.e = torch.nn.Parameter(torch.zeros(0, 4))
            self.v = torch.nn.Parameter(torch.zeros(3))

        def load_weights(self, weights):
            for n, w in weights:
                if n == "s0":
                    self.s0.data.copy_(w)
                elif n == "s1":
                    self.s1.data.copy_(w.view(self.s1.shape))
                elif n == "e":
                    self.e.data.copy_(w)
                elif n == "v":
                    self.v.data.copy_(w[2])

    full = {"s0": torch.tensor(3.5), "s1": torch.tensor(7.25), "e": torch.zeros(0, 4),
            "v": torch.arange(15.0).reshape(5, 3)}
    model = Edge()
    cap = capture_geometry(model, [(n, torch.float32, tuple(t.shape)) for n, t in full.items()])
    assert cap.unsupported == [] and len(cap.copies) == 4
    sources = {n: SourceSpec(tuple(t.shape), torch.float32, 4, [
        ShardSpec((0,) * t.dim(), tuple(t.shape), "s", t.data_ptr(), 4)]) for n, t in full.items()}
    dests = dict(model.named_parameters())
    table, unsupported, converts = plan_transfer_2d(cap.copies, sources, lambda n: dests[n].data_ptr())
    assert not unsupported and not converts and len(table) == 3     # nothing to move for "e"
    c_port.scatter2d(table)
    assert float(model.s0.detach()) == 3.5 and model.s1.tolist() == [7.25] and model.v.tolist() == [6.0, 7.0, 8.0]


def test_transposing_copies_are_staged_as_wide_boxes_and_transposed_on_the_device():
    """A loader that transposes its source (GPT-2's Conv1D weights are stored (in, out)):
    as plain records the copy is one element per row; with a staging buffer it is planned
    as the box it reads, in the source's own row order (wide rows), and transposed by the
    one torch copy that also does the casts.  Same bytes as the loader itself produces,
    also through a 3-D source, a column split and a dtype change."""
    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.conv = torch.nn.Parameter(torch.zeros(128, 96, dtype=torch.bfloat16))      # (out/2, in)
            self.stack = torch.nn.Parameter(torch.zeros(3, 64, 80, dtype=torch.bfloat16))   # (E, out, in)
            self.wide = torch.nn.Parameter(torch.zeros(64, 96, dtype=torch.float32))        # cast as well
            self.plain = torch.nn.Parameter(torch.zeros(96, 256, dtype=torch.bfloat16))

        def load_weights(self, weights):
            for name, w in weights:
                if name == "conv":          # stored (in=96, out=256): this rank's half of the outputs
                    self.conv.data.copy_(w.t().narrow(0, 128, 128))
                elif name == "stack":       # stored (E, in=80, out=64)
                    self.stack.data.copy_(w.transpose(1, 2))
                elif name == "wide":        # stored (in=96, out=64) in bf16, parameter fp32
                    self.wide.data.copy_(w.t())
                elif name == "plain":
                    self.plain.data.copy_(w)

    manifest = [("conv", torch.bfloat16, (96, 256)), ("stack", torch.bfloat16, (3, 80, 64)),
                ("wide", torch.bfloat16, (96, 64)), ("plain", torch.bfloat16, (96, 256))]
    image, index = _image(manifest, seed=5)
    truth = M()
    truth.load_weights((n, _real_tensor(image, index[n], dt)) for n, dt, _s in manifest)
    # without staging: exact, but one element per row
    bare = captured_table(M(), index, {"mem": image.ctypes.data}, device=torch.device("cpu"), min_row_bytes=0)
    narrow = bare.records[bare.records[:, 3] == 2]
    assert len(narrow) and int(narrow[:, 2].sum()) > 20000       # tens of thousands of two-byte rows
    model = M()
    cap = _run_records(model, image, index, manifest)
    assert not cap.reasons and sorted(c.param_name for c in cap.converts) == ["conv", "stack", "wide"]
    assert len(cap.records) <= 8 and int(cap.records[:, 3].min()) >= 128      # a handful of wide rows
    for (n, a), (_n, b) in zip(model.state_dict().items(), truth.state_dict().items()):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), n
