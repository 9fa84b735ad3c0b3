"""Host logic of the product (planner, layout, reshard plan, safetensors index)
checked against the oracle on the CPU: records are executed on host buffers by
the oracle's C loop and compared with the oracle's own result."""

import json
import os

import numpy as np
import pytest

from helpers import NP_OF_TAG, read_full_tensors, run_records_on_host, tiny_dense_config
from modelexpress_b200 import layout, planner, reshard, synth
from modelexpress_b200.safetensors_index import (checkpoint_index, parse_safetensors_header,
                                                 resolve_safetensors_files)
from oracle import ref_port as R
from test_oracle_golden import _chain, _load


@pytest.mark.parametrize("plan_pull", ["library", "python"])
@pytest.mark.parametrize("case", _load("slice_plan.json"), ids=lambda c: c["tag"])
def test_records_expand_to_the_reference_runs(case, plan_pull, monkeypatch):
    if plan_pull == "python":   # the planner's Python statement instead of mxb_plan_pull
        monkeypatch.setattr(planner, "plan_pull_2d", planner.plan_pull_2d_py)
    copy = planner.CopySpec("src", _chain(case["op_chain"]), "p", case["dest_offset"],
                            tuple(case["dest_shape"]), tuple(case["dest_stride"]), "dt")
    shards = [planner.ShardSpec(tuple(o), tuple(s), sess, addr, case["elsize"])
              for o, s, sess, addr in case["shards"]]
    if case["error"]:
        with pytest.raises(planner.UnsupportedReshard):
            planner.plan_pull_2d(copy, case["global_shape"], "dt", case["elsize"], shards, 0)
        return
    parts = planner.plan_pull_2d(copy, case["global_shape"], "dt", case["elsize"], shards, 0)
    got = []
    for sess, recs in parts:
        got += [[sess, s, d, n] for s, d, n in planner.expand_records(recs)]
    assert got == case["segments"]  # same runs, same order as the reference's plan_pull
    assert sum(len(r) for _s, r in parts) <= len(case["segments"]) or not case["segments"]


def test_planner_rejects_what_the_reference_rejects():
    copy = planner.CopySpec("src", (), "w", 0, (4, 4), (4, 1), "f32")
    shard = planner.ShardSpec((0, 0), (4, 4), "s0", 0, 4)
    with pytest.raises(planner.UnsupportedReshard):
        planner.plan_pull_2d(copy, (4, 4), "bf16", 4, [shard], 0)
    with pytest.raises(ValueError):
        planner.plan_pull_2d(copy, (4, 4), "f32", 4, [planner.ShardSpec((0,), (4, 4), "s", 0, 4)], 0)
    bad = planner.CopySpec("src", (("reshape", ((16,),), ()),), "w", 0, (16,), (1,), "f32")
    with pytest.raises(planner.UnsupportedReshard):
        planner.plan_pull_2d(bad, (4, 4), "f32", 4, [shard], 0)


@pytest.fixture(scope="module")
def tiny_ckpt(tmp_path_factory):
    cfg = tiny_dense_config()
    d = str(tmp_path_factory.mktemp("tiny_ckpt"))
    synth.write_checkpoint(d, synth.dense_tensors(cfg), cfg.seed, cfg.files)
    return d


def test_synthetic_checkpoint_is_valid_safetensors(tiny_ckpt):
    from safetensors import safe_open

    files = resolve_safetensors_files(tiny_ckpt)
    assert len(files) == 2
    for path, names in files.items():
        ours = parse_safetensors_header(path)
        theirs = R.parse_safetensors_header(path)
        assert ours == theirs
        with safe_open(path, framework="pt") as f:
            assert sorted(f.keys()) == sorted(ours)
            name = names[0]
            t = f.get_tensor(name)
            raw = np.fromfile(path, dtype=np.uint8)[ours[name]["file_offset"]:][: ours[name]["size"]]
            assert raw.tobytes() == t.contiguous().view(-1).view(__import__("torch").uint8).numpy().tobytes()
    idx = checkpoint_index(tiny_ckpt)
    assert "model.layers.1.self_attn.q_proj.bias" in idx
    norm = read_full_tensors(tiny_ckpt)["model.norm.weight"]
    assert (norm == 0x3F80).all()  # bf16 1.0


def test_header_parser_rejections(tmp_path):
    p = tmp_path / "short.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(RuntimeError, match="Invalid safetensors"):
        parse_safetensors_header(str(p))
    p = tmp_path / "huge.safetensors"
    p.write_bytes((200 * 1024 * 1024).to_bytes(8, "little") + b"{}")
    with pytest.raises(RuntimeError, match="too large"):
        parse_safetensors_header(str(p))
    with pytest.raises(FileNotFoundError):
        resolve_safetensors_files(str(tmp_path / "nothing"))


@pytest.mark.parametrize("tp", [1, 2, 8])
def test_dense_layout_matches_oracle_load_and_shard(tiny_ckpt, tp):
    full = read_full_tensors(tiny_ckpt)
    idx = checkpoint_index(tiny_ckpt)
    index = {n: {"shape": i["shape"], "dtype": i["dtype"]} for n, i in idx.items()}
    for rank in range(tp):
        want = R.load_and_shard(full, rank, tp)
        plan = layout.plan_checkpoint(index, rank, tp)
        assert set(plan.params) == set(want)
        bufs = {n: np.zeros(s.shape, dtype=NP_OF_TAG[s.dtype]) for n, s in plan.params.items()}
        srcs = {n: np.ascontiguousarray(a) for n, a in full.items()}
        recs = [pl.record(srcs[pl.src_name].ctypes.data, bufs[pl.dst_name].ctypes.data)
                for pl in plan.placements]
        run_records_on_host(recs)
        for n in want:
            assert bufs[n].shape == want[n].shape, n
            assert np.array_equal(bufs[n], want[n]), (rank, n)
        assert plan.bytes_placed == sum(a.nbytes for a in want.values())


def test_layout_matches_real_vllm_layers():
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "vllm_layers.npz"))
    tp, h, qh, kvh, hd, inter, voc = (int(x) for x in z["meta"])
    pre = "model.layers.0."
    full = {
        pre + "self_attn.q_proj.weight": z["src/q_proj"], pre + "self_attn.k_proj.weight": z["src/k_proj"],
        pre + "self_attn.v_proj.weight": z["src/v_proj"], pre + "self_attn.q_proj.bias": z["src/q_bias"],
        pre + "self_attn.k_proj.bias": z["src/k_bias"], pre + "self_attn.v_proj.bias": z["src/v_bias"],
        pre + "self_attn.o_proj.weight": z["src/o_proj"], pre + "mlp.gate_proj.weight": z["src/gate_proj"],
        pre + "mlp.up_proj.weight": z["src/up_proj"], pre + "mlp.down_proj.weight": z["src/down_proj"],
        "model.embed_tokens.weight": z["src/embed"],
    }
    names = {"qkv_w": pre + "self_attn.qkv_proj.weight", "qkv_b": pre + "self_attn.qkv_proj.bias",
             "gate_up": pre + "mlp.gate_up_proj.weight", "o": pre + "self_attn.o_proj.weight",
             "down": pre + "mlp.down_proj.weight", "embed": "model.embed_tokens.weight"}
    index = {n: {"shape": list(a.shape), "dtype": "BF16"} for n, a in full.items()}
    srcs = {n: np.ascontiguousarray(a) for n, a in full.items()}
    for rank in range(tp):
        plan = layout.plan_checkpoint(index, rank, tp)
        bufs = {n: np.zeros(s.shape, dtype=np.uint16) for n, s in plan.params.items()}
        run_records_on_host([pl.record(srcs[pl.src_name].ctypes.data, bufs[pl.dst_name].ctypes.data)
                             for pl in plan.placements])
        for short, name in names.items():
            assert np.array_equal(bufs[name], z[f"rank{rank}/{short}"]), (rank, short)
        assert plan.params["model.embed_tokens.weight"].zero_fill == (rank == tp - 1)


def test_layout_errors():
    with pytest.raises(ValueError):
        layout.plan_dense({"a.o_proj.weight": {"shape": [4, 6], "dtype": "BF16"}}, 0, 4)
    with pytest.raises(KeyError):
        layout.plan_dense({"l.self_attn.q_proj.weight": {"shape": [8, 4], "dtype": "BF16"}}, 0, 2)
    with pytest.raises(ValueError):
        layout.plan_dense({}, 3, 2)


def test_moe_layout_places_experts_and_scales():
    cfg = synth.MoEConfig(layers=1, hidden=512, experts=8, moe_intermediate=512, q_lora=128,
                          kv_lora=128, qk_rope=64, qk_nope=64, v_head=64, heads=8, files=1)
    tensors = synth.moe_tensors(cfg)
    index = {n: {"shape": list(s), "dtype": d} for n, s, d, _k in tensors}
    rng = np.random.default_rng(1)
    full = {n: rng.integers(0, 255, size=s, dtype=np.uint8).astype(NP_OF_TAG[d]) if NP_OF_TAG[d] != np.float32
            else rng.random(s, dtype=np.float32) for n, s, d, _k in tensors}
    tp = 4
    for rank in range(tp):
        plan = layout.plan_checkpoint(index, rank, tp)
        bufs = {n: np.zeros(s.shape, dtype=NP_OF_TAG[s.dtype]) for n, s in plan.params.items()}
        run_records_on_host([pl.record(full[pl.src_name].ctypes.data, bufs[pl.dst_name].ctypes.data)
                             for pl in plan.placements])
        p = "model.layers.0.mlp."
        w13, w2 = bufs[p + "experts.w13_weight"], bufs[p + "experts.w2_weight"]
        s13 = bufs[p + "experts.w13_weight_scale_inv"]
        assert w13.shape == (2, 1024, 512) and w2.shape == (2, 512, 512) and s13.shape == (2, 8, 4)
        for slot in range(2):
            e = rank * 2 + slot
            # installer.py:695-754: gate is the low half of w13, up the high half
            assert np.array_equal(w13[slot, :512], full[f"{p}experts.{e}.gate_proj.weight"])
            assert np.array_equal(w13[slot, 512:], full[f"{p}experts.{e}.up_proj.weight"])
            assert np.array_equal(w2[slot], full[f"{p}experts.{e}.down_proj.weight"])
            assert np.array_equal(s13[slot, 4:], full[f"{p}experts.{e}.up_proj.weight_scale_inv"])
        # shared expert: tensor-parallel like a dense MLP, scales split in step
        gu = bufs[p + "shared_experts.gate_up_proj.weight"]
        assert np.array_equal(gu[:128], full[p + "shared_experts.gate_proj.weight"][rank * 128:(rank + 1) * 128])
        gs = bufs[p + "shared_experts.gate_up_proj.weight_scale_inv"]
        assert np.array_equal(gs[1:], full[p + "shared_experts.up_proj.weight_scale_inv"][rank:rank + 1])
        dn = bufs[p + "shared_experts.down_proj.weight"]
        assert np.array_equal(dn, full[p + "shared_experts.down_proj.weight"][:, rank * 128:(rank + 1) * 128])
        ds = bufs[p + "shared_experts.down_proj.weight_scale_inv"]
        assert np.array_equal(ds, full[p + "shared_experts.down_proj.weight_scale_inv"][:, rank:rank + 1])
        a = "model.layers.0.self_attn."
        fq = bufs[a + "fused_qkv_a_proj.weight"]
        assert np.array_equal(fq[:128], full[a + "q_a_proj.weight"])
        assert np.array_equal(fq[128:], full[a + "kv_a_proj_with_mqa.weight"])
        ob = bufs[a + "o_proj.weight"]
        assert np.array_equal(ob, full[a + "o_proj.weight"][:, rank * 128:(rank + 1) * 128])


def test_moe_layout_matches_oracle_on_a_written_checkpoint(tmp_path):
    cfg = synth.MoEConfig(layers=1, hidden=512, experts=8, moe_intermediate=512, q_lora=128,
                          kv_lora=128, qk_rope=64, qk_nope=64, v_head=64, heads=8, files=2)
    d = str(tmp_path)
    synth.write_checkpoint(d, synth.moe_tensors(cfg), cfg.seed, cfg.files)
    full = read_full_tensors(d)
    idx = checkpoint_index(d)
    index = {n: {"shape": i["shape"], "dtype": i["dtype"]} for n, i in idx.items()}
    for rank in (0, 3):
        want = R.load_and_shard_moe(full, rank, 4)
        plan = layout.plan_checkpoint(index, rank, 4)
        assert set(plan.params) == set(want)
        bufs = {n: np.zeros(s.shape, dtype=NP_OF_TAG[s.dtype]) for n, s in plan.params.items()}
        srcs = {n: np.ascontiguousarray(a) for n, a in full.items()}
        run_records_on_host([pl.record(srcs[pl.src_name].ctypes.data, bufs[pl.dst_name].ctypes.data)
                             for pl in plan.placements])
        for n, a in want.items():
            assert bufs[n].shape == a.shape, n
            assert np.array_equal(bufs[n].view(np.uint8), a.view(np.uint8)), (rank, n)


@pytest.mark.parametrize("world,tp", [(8, 8), (4, 2), (2, 4)])
def test_reshard_plan_matches_oracle_regather(tiny_ckpt, world, tp):
    full = read_full_tensors(tiny_ckpt)
    idx = checkpoint_index(tiny_ckpt)
    index = {n: {"shape": i["shape"], "dtype": i["dtype"]} for n, i in idx.items()}
    pieces = R.fsdp_shards(full, world)
    sa = reshard.shard_arena(index, world)
    plans = [layout.plan_checkpoint(index, t, tp) for t in range(tp)]
    pa = reshard.param_arena(plans[0])
    shard_arenas = [np.zeros(sa.total, dtype=np.uint8) for _ in range(world)]
    for s in range(world):
        for n, piece in pieces[s].items():
            b = piece.view(np.uint8)
            shard_arenas[s][sa.offsets[n]: sa.offsets[n] + b.size] = b
    param_arenas = [np.zeros(pa.total, dtype=np.uint8) for _ in range(tp)]
    total = 0
    for s in range(world):
        recs = reshard.plan_reshard(index, world, tp, s, shard_arenas[s].ctypes.data,
                                    [a.ctypes.data for a in param_arenas])
        total += reshard.reshard_bytes(recs)
        run_records_on_host(recs)
    shapes = {n: a.shape for n, a in full.items()}
    for t in range(tp):
        want = R.regather_and_reslice(pieces, shapes, t, tp)
        for n, a in want.items():
            got = param_arenas[t][pa.offsets[n]: pa.offsets[n] + a.nbytes].view(a.dtype).reshape(a.shape)
            assert np.array_equal(got, a), (t, n)
    assert total == sum(p.bytes_placed for p in plans)


def test_clip_records_ragged_split():
    # a 5x6 byte matrix, column block [2:5) of every row, cut at flat bytes [7, 23)
    src = np.arange(30, dtype=np.uint8)
    dst = np.zeros(15, dtype=np.uint8)
    piece = src[7:23].copy()
    recs = reshard.clip_records(2, 0, 5, 3, 6, 3, 7, 23, piece.ctypes.data, dst.ctypes.data)
    run_records_on_host(recs)
    want = np.zeros((5, 3), dtype=np.uint8)
    m = src.reshape(5, 6)
    for r in range(5):
        for c in range(2, 5):
            if 7 <= r * 6 + c < 23:
                want[r, c - 2] = m[r, c]
    assert np.array_equal(dst.reshape(5, 3), want)


@pytest.mark.parametrize("rank", [0, 1])
def test_premerged_gate_up_is_sharded_per_member(rank):
    """tests/test_mdl_tp.py:50-81 of the reference: a checkpoint that ships one
    [gate; up] tensor must shard gate and up independently."""
    src = np.arange(16, dtype=np.float32).reshape(8, 2)
    name = "mlp.gate_up_proj.weight"
    plan = layout.plan_dense({name: {"shape": [8, 2], "dtype": "F32"}}, rank, 2)
    dst = np.zeros(plan.params[name].shape, dtype=np.float32)
    run_records_on_host([pl.record(src.ctypes.data, dst.ctypes.data) for pl in plan.placements])
    gate = src[rank * 2:(rank + 1) * 2]
    up = src[4 + rank * 2: 4 + (rank + 1) * 2]
    assert np.array_equal(dst, np.concatenate((gate, up)))
    # and the same arithmetic as the installer's own helper (fixture)
    writes = R.premerged_writes(4, 2, 8, 2, rank)
    assert [(pl.dst_start, pl.start, pl.size) for pl in plan.placements] == [tuple(w) for w in writes]
    with pytest.raises(ValueError):
        layout.plan_dense({name: {"shape": [10, 2], "dtype": "F32"}}, 0, 2)


def test_dtype_mismatch_is_planned_through_staging():
    """transfer_plan.py:226-256: a served dtype that differs from the destination's is
    pulled into staging of the served dtype and listed for a cast."""
    shard = planner.ShardSpec((0, 0), (4, 8), "s", 1000, 2)
    sources = {"router": planner.SourceSpec((4, 8), "bf16", 2, [shard])}
    copy = planner.CopySpec("router", (("narrow", (0, 1, 2), ()),), "gate", 0, (2, 8), (8, 1), "f32")
    table, unsupported, converts = planner.plan_transfer_2d([copy], sources, lambda n: 0)
    assert unsupported == ["router"] and converts == [] and len(table) == 0
    table, unsupported, converts = planner.plan_transfer_2d([copy], sources, lambda n: 0, convert_base=1 << 20)
    assert unsupported == [] and len(converts) == 1
    assert planner.expand_records(table) == [(1000 + 16, 1 << 20, 32)]
    c = converts[0]
    assert (c.param_name, c.dest_shape, c.src_dtype, c.staging_offset, c.nbytes) == ("gate", (2, 8), "bf16", 0, 32)
    assert planner.convert_staging_bytes([copy], sources) == 32
