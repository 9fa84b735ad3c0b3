"""The CPU oracle (numpy and C restatements) against fixtures produced by the
real reference code (tests/golden/make_golden.py) and the reference tests'
hand-computed vectors."""

import json
import os

import numpy as np
import pytest

from make_golden import golden_bytes
from oracle import c_port as C
from oracle import ref_port as R

G = os.path.join(os.path.dirname(__file__), "golden")


def _load(name):
    with open(os.path.join(G, name)) as f:
        return json.load(f)


def digest_case_bytes(c):
    k = c["kind"]
    if k == "seeded":
        return golden_bytes(c["seed"], c["nbytes"])
    if k == "arange_i32":
        return np.arange(c["n"], dtype=np.int32).view(np.uint8)
    if k == "arange_i16":
        return np.arange(c["n"], dtype=np.int16).view(np.uint8)
    if k == "arange_bf16":
        import torch

        return torch.arange(c["n"], dtype=torch.bfloat16).view(torch.int16).numpy().view(np.uint8)
    if k == "fill_u8":
        return np.full(c["n"], c["value"], dtype=np.uint8)
    raise KeyError(k)


@pytest.mark.parametrize("case", _load("digests.json"), ids=lambda c: f"{c['kind']}-{c.get('nbytes', c.get('n'))}")
def test_digests_match_reference(case):
    b = digest_case_bytes(case)
    assert R.safe_checksum(b) == case["safe_checksum"]
    assert C.safe_checksum(b) == case["safe_checksum"]
    assert C.safe_checksum(b, mt=True) == case["safe_checksum"]
    if case["tensor_digest"] is not None:
        assert R.tensor_digest(b) == case["tensor_digest"]
        assert R.digest_from_scalars(C.digest_scalars(b)) == case["tensor_digest"]
        assert R.digest_from_scalars(C.digest_scalars(b, mt=True)) == case["tensor_digest"]
    # the block hash has no reference counterpart; its two restatements must agree
    assert R.block_hash64(b) == C.block_hash64(b)
    assert np.array_equal(R.block_hashes64(b), C.block_hashes64(b))


def test_known_reference_values():
    # values computed from the reference code when the fixtures were first generated
    assert R.tensor_digest(np.arange(4096, dtype=np.int32)) == "b80e42d0aa211223be9669385be8976b"
    import torch

    a = torch.arange(16, dtype=torch.bfloat16).view(torch.int16).numpy()
    assert R.safe_checksum(a) == "59cd2bf4"


def _chain(js):
    out = []
    for name, args in js:
        a2 = []
        for a in args:
            if isinstance(a, dict) and "slice" in a:
                a2.append(slice(*a["slice"]))
            elif isinstance(a, dict) and "tuple" in a:
                a2.append(tuple(slice(*x["slice"]) if isinstance(x, dict) else x for x in a["tuple"]))
            elif isinstance(a, list):
                a2.append(tuple(a))
            else:
                a2.append(a)
        out.append((name, tuple(a2), ()))
    return tuple(out)


@pytest.mark.parametrize("case", _load("slice_plan.json"), ids=lambda c: c["tag"])
def test_plan_pull_matches_reference(case):
    copy = R.RecordedCopy("src", _chain(case["op_chain"]), "p", case["dest_offset"],
                          tuple(case["dest_shape"]), tuple(case["dest_stride"]), "dt")
    shards = [R.Shard(tuple(o), tuple(s), sess, addr, case["elsize"])
              for o, s, sess, addr in case["shards"]]
    if case["error"]:
        with pytest.raises(R.UnsupportedReshard):
            R.plan_pull(copy, tuple(case["global_shape"]), "dt", case["elsize"], shards)
        return
    segs = R.plan_pull(copy, tuple(case["global_shape"]), "dt", case["elsize"], shards)
    assert [[s.session, s.src_addr, s.dst_byte, s.nbytes] for s in segs] == case["segments"]


def test_plan_pull_hand_computed():
    # tests/test_reshard_refit_slice_plan.py:54-66 of the reference, by hand
    copy = R.RecordedCopy("src", (("narrow", (1, 0, 4), ()),), "row", 0, (4, 4), (4, 1), "f32")
    shard = R.Shard((0, 0), (4, 8), "s0", 2000, 4)
    segs = R.plan_pull(copy, (4, 8), "f32", 4, [shard])
    assert [(s.src_addr - 2000) // 4 for s in segs] == [0, 8, 16, 24]
    assert [s.dst_byte // 4 for s in segs] == [0, 4, 8, 12]
    assert all(s.nbytes == 16 for s in segs)
    with pytest.raises(R.UnsupportedReshard):
        R.plan_pull(copy, (4, 8), "bf16", 4, [shard])
    with pytest.raises(ValueError):
        R.intersect([(0, 4), (0, 4)], [(0, 4)])


def test_installer_arithmetic_matches_reference():
    g = _load("installer.json")
    for c in g["tp_local"]:
        t = np.arange(int(np.prod(c["shape"])), dtype=np.int32).reshape(c["shape"])
        loc = R.tp_local_tensor(t, tuple(c["expected"]), c["tp"], c["rank"])
        assert (None if loc is None else loc.reshape(-1).tolist()) == c["result"]
    for c in g["fused"]:
        res = R.fused_destinations(tuple(c["fused_shape"]),
                                   [(n, tuple(s)) for n, s in c["members"]], c["tp"])
        if c["result"] is None:
            assert res is None
        else:
            assert {k: list(v) for k, v in res.items()} == c["result"]
    for c in g["premerged"]:
        res = R.premerged_writes(c["dst_rows"], 2, c["src_rows"], c["tp"], c["rank"])
        assert (None if res is None else [list(x) for x in res]) == c["result"]


def test_toy_reshard_reconstruction():
    """Reference ToyModel (column / row / fused qkv / norm): the reference's
    captured copies, planned by the oracle, reproduce the reference's segments
    and, moved with the oracle's memmove loop, its loader's ground truth."""
    g = _load("toy_reshard.json")
    shapes = {n: tuple(s) for n, s in g["manifest"]}
    srcs, base = {}, 0.0
    for name, shape in shapes.items():
        n = int(np.prod(shape))
        srcs[name] = (base + np.arange(n, dtype=np.float32)).reshape(shape)
        base += n
    copies = [R.RecordedCopy(c["src_name"], _chain(c["op_chain"]), c["param_name"],
                             c["dest_offset"], tuple(c["dest_shape"]), tuple(c["dest_stride"]), "f32")
              for c in g["copies"]]
    for var in g["variants"]:
        ns = var["nsplit"]
        params = {n: np.zeros(s, dtype=np.float32) for n, s in g["param_shapes"].items()}
        pieces, segs = {}, []
        for c in copies:
            t = srcs[c.src_name]
            per = t.shape[0] // ns
            shards = []
            for s in range(ns):
                key = f"{c.src_name}#{s}"
                pieces.setdefault(key, np.ascontiguousarray(t[s * per:(s + 1) * per]))
                shards.append(R.Shard((s * per,) + (0,) * (t.ndim - 1), pieces[key].shape, key,
                                      pieces[key].ctypes.data, 4))
            segs += R.plan_pull(c, shapes[c.src_name], "f32", 4, shards)
        got = [[s.session, s.src_addr - pieces[s.session].ctypes.data, s.param_name, s.dst_byte, s.nbytes]
               for s in segs]
        assert got == var["segments"]
        runs = [(s.src_addr, params[s.param_name].ctypes.data + s.dst_byte, s.nbytes) for s in segs]
        if ns == 1:
            R.memmove_read([R.ReadDescriptor(s.session, r[0], r[1], r[2]) for s, r in zip(segs, runs)])
        else:
            C.memmove_runs(runs)
        for n, truth in g["truth"].items():
            assert params[n].reshape(-1).tolist() == truth, n


def test_load_and_shard_matches_vllm_layers():
    """Real vLLM parallel layers driven on CPU (fixture): QKV / merged column /
    row / vocab-parallel with a 64-padded vocabulary, TP=4, all ranks."""
    z = np.load(os.path.join(G, "vllm_layers.npz"))
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
    for rank in range(tp):
        got = R.load_and_shard(full, rank, tp)
        for short, name in names.items():
            want = z[f"rank{rank}/{short}"]
            assert got[name].shape == want.shape, (rank, short)
            assert np.array_equal(got[name], want), (rank, short)


def test_regather_and_reslice_equals_load_and_shard():
    rng = np.random.default_rng(3)
    pre = "model.layers.0."
    full = {
        pre + "self_attn.q_proj.weight": rng.integers(0, 65536, (64, 32), dtype=np.uint16),
        pre + "self_attn.k_proj.weight": rng.integers(0, 65536, (16, 32), dtype=np.uint16),
        pre + "self_attn.v_proj.weight": rng.integers(0, 65536, (16, 32), dtype=np.uint16),
        pre + "self_attn.o_proj.weight": rng.integers(0, 65536, (32, 64), dtype=np.uint16),
        pre + "input_layernorm.weight": rng.integers(0, 65536, (32,), dtype=np.uint16),
    }
    shards = R.fsdp_shards(full, 8)
    shapes = {n: a.shape for n, a in full.items()}
    for r in range(8):
        a = R.regather_and_reslice(shards, shapes, r, 8)
        b = R.load_and_shard(full, r, 8)
        assert a.keys() == b.keys()
        for n in a:
            assert np.array_equal(a[n], b[n])


def _expert_case_arrays(case):
    from make_golden import expert_case_tensors

    tensors = expert_case_tensors(case["seed"], case["experts"], case["inter"], case["hidden"], case["block"])
    ep = (case["rank"] if case["ep"] > 1 else 0, case["ep"])
    et = (case["rank"] if case["tp"] > 1 else 0, case["tp"])
    want = {"experts.w13_weight": np.array(case["w13_weight"], dtype=np.uint8),
            "experts.w2_weight": np.array(case["w2_weight"], dtype=np.uint8),
            "experts.w13_weight_scale_inv": np.array(case["w13_scale"], dtype=np.float32),
            "experts.w2_weight_scale_inv": np.array(case["w2_scale"], dtype=np.float32)}
    return tensors, ep, et, want


@pytest.mark.parametrize("case", _load("expert_slots.json"), ids=lambda c: f'{c["tag"]}-r{c["rank"]}')
def test_expert_slots_match_the_reference_loader(case):
    """expert_slots.json is what the reference's MdlLoader (installer.py:695-771) wrote
    into FusedMoE-style w13 / w2 parameters and their block scales, expert-parallel
    and with tensor-parallel experts: the oracle's load_and_shard_moe and the
    product's layout rules (records executed by the oracle's C loop) must give the
    same bytes."""
    from helpers import run_records_on_host
    from modelexpress_b200 import layout

    tensors, ep, et, want = _expert_case_arrays(case)
    got = R.load_and_shard_moe(tensors, 0, 1, ep=ep, expert_tp=et)
    pre = "model.layers.0.mlp."
    for key, w in want.items():
        assert got[pre + key].shape == w.shape, key
        assert np.array_equal(got[pre + key], w), (case["tag"], case["rank"], key)
    # the product's placement rules on the same checkpoint
    index = {n: {"shape": list(a.shape), "dtype": "F8_E4M3" if a.dtype == np.uint8 else "F32"}
             for n, a in tensors.items()}
    plan = layout.plan_moe(index, 0, 1, ep_rank=ep[0], ep_size=ep[1], expert_tp=et)
    bufs = {n: np.zeros(s.shape, dtype=np.uint8 if s.dtype == "F8_E4M3" else np.float32)
            for n, s in plan.params.items()}
    srcs = {n: np.ascontiguousarray(a) for n, a in tensors.items()}
    run_records_on_host([pl.record(srcs[pl.src_name].ctypes.data, bufs[pl.dst_name].ctypes.data)
                         for pl in plan.placements])
    for key, w in want.items():
        assert bufs[pre + key].shape == w.shape, key
        assert np.array_equal(bufs[pre + key], w), (case["tag"], case["rank"], key)
