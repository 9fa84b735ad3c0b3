"""Generate the golden fixtures in this folder from the real reference code.

Run where the reference checkout is present (it is not needed to run the
tests, only to regenerate the fixtures):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py \
        --reference /path/to/modelexpress/modelexpress_client/python

Outputs (all small, committed):
  digests.json      safe_checksum / tensor_digest of seeded byte strings
  slice_plan.json   plan_pull segments for hand-written and random copies
  installer.json    MdlLoader TP-narrow / fused-offset / pre-merged arithmetic
  expert_slots.json MdlLoader.load_weights on FusedMoE-style stand-ins: FP8 expert
                    weights and block scales into w13 / w2 slots, expert-parallel
                    (global -> local expert id) and tensor-parallel inside an expert
  toy_reshard.json  capture_geometry -> plan_transfer -> memmove on the
                    reference's ToyModel (column, row, fused qkv, norm)
  capture_pin.json  the reference's capture_geometry + resolve_slice on
                    tests/hooked_model.py (boxes and landing places per copy)
  shard_table.json  the reference's shard-table wire blob for a small table
  vllm_layers.npz   (only with --vllm) real vLLM parallel-layer weight_loaders
                    driven on CPU with a patched TP rank

Inputs are described by (seed, size) so the tests can rebuild them with
``golden_bytes`` below without the reference.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def golden_bytes(seed: int, n: int) -> np.ndarray:
    """Seeded byte string shared by the generator and the tests."""
    return np.random.default_rng(seed).integers(0, 256, size=n, dtype=np.uint8)


DIGEST_SIZES = [0, 1, 2, 3, 4, 5, 7, 8, 15, 16, 17, 4092, 4095, 4096, 4097, 4100,
                8192, 8192 + 7, 12288 + 2, 65536, 1 << 20, (1 << 20) + 13,
                3 * 4096 * 37 + 4 * 511 + 3]


def make_digests(torch, safe_checksum, tensor_digest):
    cases = []
    for i, n in enumerate(DIGEST_SIZES):
        b = golden_bytes(1000 + i, n)
        t = torch.from_numpy(b.copy())
        try:
            dg = tensor_digest(t)
        except RuntimeError:
            # the reference cannot view a zero-length byte slice as int32, so
            # tensors shorter than one word raise; recorded as null
            dg = None
        cases.append({"kind": "seeded", "seed": 1000 + i, "nbytes": n,
                      "safe_checksum": safe_checksum(t),
                      "tensor_digest": dg})
    # structured inputs the reference tests use
    a = torch.arange(4096, dtype=torch.int32)
    cases.append({"kind": "arange_i32", "n": 4096,
                  "safe_checksum": safe_checksum(a), "tensor_digest": tensor_digest(a)})
    a = torch.arange(8192, dtype=torch.int32)
    cases.append({"kind": "arange_i32", "n": 8192,
                  "safe_checksum": safe_checksum(a), "tensor_digest": tensor_digest(a)})
    a = torch.arange(1024 + 7, dtype=torch.int16)
    cases.append({"kind": "arange_i16", "n": 1024 + 7,
                  "safe_checksum": safe_checksum(a), "tensor_digest": tensor_digest(a)})
    a = torch.arange(16, dtype=torch.bfloat16)
    cases.append({"kind": "arange_bf16", "n": 16,
                  "safe_checksum": safe_checksum(a), "tensor_digest": tensor_digest(a)})
    a = torch.arange(1409, dtype=torch.bfloat16)
    cases.append({"kind": "arange_bf16", "n": 1409,
                  "safe_checksum": safe_checksum(a), "tensor_digest": tensor_digest(a)})
    # all-0xFF: negative int32 words, exercises the signed row sums
    a = torch.full((3 * 4096 + 5,), 255, dtype=torch.uint8)
    cases.append({"kind": "fill_u8", "value": 255, "n": 3 * 4096 + 5,
                  "safe_checksum": safe_checksum(a), "tensor_digest": tensor_digest(a)})
    return cases


def _chain_json(chain):
    out = []
    for name, args, kw in chain:
        jargs = []
        for a in args:
            if isinstance(a, slice):
                jargs.append({"slice": [a.start, a.stop, a.step]})
            elif isinstance(a, tuple):
                jargs.append({"tuple": [
                    {"slice": [x.start, x.stop, x.step]} if isinstance(x, slice) else x
                    for x in a]})
            else:
                jargs.append(a)
        out.append([name, jargs])
    return out


def make_slice_plan(slice_plan, types):
    Shard, plan_pull = slice_plan.Shard, slice_plan.plan_pull
    RecordedCopy = types.RecordedCopy
    rng = np.random.default_rng(7)
    cases = []

    def add(chain, dest_offset, dest_shape, dest_stride, gshape, shards, elsize, tag):
        copy = RecordedCopy("src", chain, "p", dest_offset, tuple(dest_shape),
                            tuple(dest_stride), "dt")
        shard_objs = [Shard(tuple(o), tuple(s), sess, addr, elsize)
                      for (o, s, sess, addr) in shards]
        try:
            segs = plan_pull(copy, tuple(gshape), "dt", elsize, shard_objs)
            result = [[s.session, s.src_addr, s.dst_byte, s.nbytes] for s in segs]
            err = None
        except types.UnsupportedReshard:
            result, err = None, "UnsupportedReshard"
        cases.append({
            "tag": tag, "op_chain": _chain_json(chain), "dest_offset": dest_offset,
            "dest_shape": list(dest_shape), "dest_stride": list(dest_stride),
            "global_shape": list(gshape), "elsize": elsize,
            "shards": [[list(o), list(s), sess, addr] for (o, s, sess, addr) in shards],
            "segments": result, "error": err,
        })

    # the reference's hand-computed cases (tests/test_reshard_refit_slice_plan.py:41-236)
    add((("narrow", (0, 0, 4), ()),), 0, (4, 4), (4, 1), (8, 4),
        [((0, 0), (8, 4), "s0", 1000)], 4, "column_block")
    add((("narrow", (1, 0, 4), ()),), 0, (4, 4), (4, 1), (4, 8),
        [((0, 0), (4, 8), "s0", 2000)], 4, "row_parallel_strided")
    add((), 16, (2, 4), (4, 1), (2, 4), [((0, 0), (2, 4), "s0", 3000)], 4, "fused_offset")
    add((), 0, (4, 8), (8, 1), (4, 8),
        [((0, 0), (4, 4), "a", 100), ((0, 4), (4, 4), "b", 200)], 4, "fan_in")
    add((("narrow", (0, 0, 4), ()),), 0, (4, 4), (4, 1), (8, 4),
        [((4, 0), (4, 4), "s0", 9000)], 4, "disjoint")
    add((("transpose", (0, 1), ()),), 0, (4, 3), (3, 1), (3, 4),
        [((0, 0), (3, 4), "s0", 0)], 4, "transpose")
    add((("permute", (2, 0, 1), ()),), 0, (4, 2, 3), (6, 3, 1), (2, 3, 4),
        [((0, 0, 0), (2, 3, 4), "s0", 0)], 4, "permute3d")
    add((("narrow", (0, 1, 2), ()), ("transpose", (0, 1), ())), 0, (5, 2), (2, 1), (4, 5),
        [((0, 0), (4, 5), "s0", 0)], 4, "narrow_transpose")
    add((("transpose", (0, 1), ()), ("contiguous", (), ())), 0, (4, 4), (4, 1), (4, 4),
        [((0, 0), (4, 4), "s0", 0)], 4, "transpose_contiguous")
    add((("__getitem__", (slice(1, 3),), ()),), 0, (2, 4), (4, 1), (8, 4),
        [((0, 0), (8, 4), "s0", 64)], 2, "getitem_rows")

    # random: 2-D tensors, dim-0 sharded into k pieces, TP narrow on either axis,
    # destination possibly inside a wider fused parameter (row pitch > width)
    for i in range(40):
        tp = int(rng.choice([2, 4, 8]))
        k = int(rng.choice([1, 2, 4, 8]))
        r = int(rng.integers(1, 5)) * tp * k
        c = int(rng.integers(1, 5)) * tp
        rank = int(rng.integers(0, tp))
        elsize = int(rng.choice([1, 2, 4]))
        axis = int(rng.integers(0, 2))
        if axis == 0:
            view = (r // tp, c)
            chain = (("narrow", (0, rank * (r // tp), r // tp), ()),)
        else:
            view = (r, c // tp)
            chain = (("narrow", (1, rank * (c // tp), c // tp), ()),)
        pad = int(rng.integers(0, 3))
        dstride = (view[1] + pad, 1)
        doff = int(rng.integers(0, 9))
        rows_per = r // k
        shards = [((s * rows_per, 0), (rows_per, c), f"t{s}", 4096 * (s + 1))
                  for s in range(k)]
        add(chain, doff, view, dstride, (r, c), shards, elsize, f"rand2d_{i}")
    # random: 3-D expert-style boxes with a 2-D shard grid
    for i in range(12):
        e, r, c = int(rng.integers(2, 5)), int(rng.integers(2, 5)) * 2, int(rng.integers(2, 5)) * 2
        lo = int(rng.integers(0, e - 1))
        chain = (("narrow", (0, lo, 2 if lo + 2 <= e else 1), ()),
                 ("narrow", (2, c // 2, c // 2), ()))
        ne = 2 if lo + 2 <= e else 1
        view = (ne, r, c // 2)
        shards = [((0, 0, 0), (e, r // 2, c), "top", 1 << 16),
                  ((0, r // 2, 0), (e, r // 2, c), "bot", 2 << 16)]
        add(chain, 3, view, (r * (c // 2), c // 2, 1), (e, r, c), shards, 2, f"rand3d_{i}")
    return cases


def make_installer(torch, MdlLoader):
    class _Model:
        def named_parameters(self):
            return []

    out = {"tp_local": [], "fused": [], "premerged": []}
    rng = np.random.default_rng(11)
    for i in range(16):
        tp = int(rng.choice([2, 4, 8]))
        rank = int(rng.integers(0, tp))
        a, b = int(rng.integers(1, 4)) * tp, int(rng.integers(1, 5)) * tp + 1
        axis = int(rng.integers(0, 2))
        shape = (a, b) if axis == 0 else (b, a)
        exp = (a // tp, b) if axis == 0 else (b, a // tp)
        t = torch.arange(shape[0] * shape[1], dtype=torch.int32).reshape(shape)
        ld = MdlLoader(_Model())
        ld._tp_size, ld._tp_rank = tp, rank
        loc = ld._tp_local_tensor(t, exp)
        out["tp_local"].append({"shape": list(shape), "expected": list(exp), "tp": tp,
                                "rank": rank,
                                "result": None if loc is None else loc.reshape(-1).tolist()})
    # ambiguous / incompatible -> None
    ld = MdlLoader(_Model())
    ld._tp_size, ld._tp_rank = 2, 1
    for shape, exp in [((6, 8), (3, 4)), ((5, 4), (3, 4)), ((4, 4), (2, 2))]:
        t = torch.arange(shape[0] * shape[1], dtype=torch.int32).reshape(shape)
        loc = ld._tp_local_tensor(t, exp)
        out["tp_local"].append({"shape": list(shape), "expected": list(exp), "tp": 2,
                                "rank": 1,
                                "result": None if loc is None else loc.reshape(-1).tolist()})
    for tp, fused_shape, members in [
        (8, (768, 64), [("q", (4096, 64)), ("k", (1024, 64)), ("v", (1024, 64))]),
        (1, (6144, 8), [("q", (4096, 8)), ("k", (1024, 8)), ("v", (1024, 8))]),
        (8, (3584, 16), [("gate", (14336, 16)), ("up", (14336, 16))]),
        (4, (48,), [("q", (128,)), ("k", (32,)), ("v", (32,))]),
        (2, (10, 4), [("a", (7, 4)), ("b", (13, 4))]),          # members odd: not divisible
        (2, (12, 4), [("a", (8, 4)), ("b", (8, 4))]),          # total mismatch
        (8, (768, 64), [("q", (512, 64)), ("k", (128, 64)), ("v", (128, 64))]),  # already local
    ]:
        ld = MdlLoader(_Model())
        ld._tp_size, ld._tp_rank = tp, 0
        p = torch.nn.Parameter(torch.zeros(fused_shape), requires_grad=False)
        res = ld._fused_destinations(p, [(i, n, s) for i, (n, s) in enumerate(members)])
        if res is None:
            enc = None
        else:
            enc = {}
            for n, v in res.items():
                # recover (axis, offset, size) from the view's storage offset / shape
                stride = p.stride()
                off = v.storage_offset()
                axis = next((d for d in range(p.ndim) if v.shape[d] != p.shape[d]), 0)
                enc[n] = [axis, off // stride[axis] if stride[axis] else 0, int(v.shape[axis])]
        out["fused"].append({"tp": tp, "fused_shape": list(fused_shape),
                             "members": [[n, list(s)] for n, s in members], "result": enc})
    for tp, rank, dst_rows, src_rows in [(2, 0, 4, 8), (2, 1, 4, 8), (8, 5, 3584, 28672),
                                          (4, 3, 6, 24), (2, 0, 4, 10), (2, 0, 5, 10)]:
        ld = MdlLoader(_Model())
        ld._tp_size, ld._tp_rank = tp, rank
        dest = torch.zeros(dst_rows, 2)
        src = torch.arange(src_rows * 2, dtype=torch.float32).reshape(src_rows, 2)
        w = ld._premerged_writes(dest, 2, src)
        enc = None
        if w is not None:
            enc = [[dv.storage_offset() // 2, sv.storage_offset() // 2, int(dv.shape[0])]
                   for dv, sv in w]
        out["premerged"].append({"tp": tp, "rank": rank, "dst_rows": dst_rows,
                                 "src_rows": src_rows, "result": enc})
    return out


def expert_case_tensors(seed: int, experts: int, inter: int, hidden: int, block: int) -> dict:
    """The checkpoint side of an expert-slot case, rebuilt from its numbers alone:
    per expert gate/up ``[inter, hidden]`` and down ``[hidden, inter]`` as raw FP8
    bytes, block scales ``[inter/block, hidden/block]`` / ``[hidden/block, inter/block]``
    as float32 (small integers over 8, exact in every format)."""
    rng = np.random.default_rng(seed)
    out = {}
    for e in range(experts):
        pre = f"model.layers.0.mlp.experts.{e}."
        for name, shape in (("gate_proj", (inter, hidden)), ("up_proj", (inter, hidden)),
                            ("down_proj", (hidden, inter))):
            # byte values that are finite, distinct FP8 numbers (avoid 0x7f/0xff NaN patterns)
            out[pre + name + ".weight"] = rng.integers(1, 0x70, size=shape, dtype=np.uint8)
            sshape = (shape[0] // block, shape[1] // block)
            out[pre + name + ".weight_scale_inv"] = (rng.integers(1, 64, size=sshape) / 8.0).astype(np.float32)
    return out


def make_expert_slots(torch, MdlLoader):
    """Drive the reference's MdlLoader (engines/vllm/refit/installer.py:86-191, expert
    slots :695-771) on stand-ins shaped like vLLM's FusedMoE parameters, the way the
    reference's own tests do (tests/test_mdl_fp8.py:279-357), and record what lands
    in w13 / w2 and their block scales."""
    F8 = torch.float8_e4m3fn
    cases = []
    for tag, experts, ep, tp, inter, hidden, block, seed in [
        ("ep4_of_8", 8, 4, 1, 4, 6, 2, 101),
        ("ep2_of_6", 6, 2, 1, 8, 4, 2, 102),
        ("ep1_of_3", 3, 1, 1, 4, 4, 1, 103),
        ("tp2_inside_experts", 2, 1, 2, 8, 8, 2, 104),   # the TP2 shape collision of the reference's test
    ]:
        tensors = expert_case_tensors(seed, experts, inter, hidden, block)
        per = experts // ep
        for rank in range(max(ep, tp)):
            ep_rank = rank if ep > 1 else 0
            tp_rank = rank if tp > 1 else 0
            li, lh = inter // tp, hidden   # column split of gate/up rows, row split of down cols
            model = torch.nn.Module()
            model.model = torch.nn.Module()
            model.model.layers = torch.nn.ModuleList([torch.nn.Module()])
            mlp = torch.nn.Module()
            model.model.layers[0].mlp = mlp
            ex = torch.nn.Module()
            mlp.experts = ex

            def par(shape, dtype=torch.float32):
                return torch.nn.Parameter(torch.zeros(shape, dtype=dtype), requires_grad=False)

            ex.w13_weight = par((per, 2 * li, lh), F8)
            ex.w2_weight = par((per, hidden, li), F8)
            ex.w13_weight_scale = par((per, 2 * li // block, lh // block))
            ex.w2_weight_scale = par((per, hidden // block, li // block))
            lo = ep_rank * per
            ex._map_global_expert_id_to_local_expert_id = (
                lambda gid, lo=lo, per=per: gid - lo if lo <= gid < lo + per else -1)

            def load_weights(*, weights):
                raise AttributeError("processed FP8 parameters are not re-entrant")

            model.load_weights = load_weights
            prefix = "model.layers.0.mlp."
            mapping = []
            for e in range(experts):
                mapping += [(prefix + "experts.w13_", prefix + f"experts.{e}.gate_proj.", e, "w1"),
                            (prefix + "experts.w2_", prefix + f"experts.{e}.down_proj.", e, "w2"),
                            (prefix + "experts.w13_", prefix + f"experts.{e}.up_proj.", e, "w3")]
            model.get_expert_mapping = lambda mapping=mapping: mapping
            os.environ["MX_LOAD_MODE"] = "direct"
            os.environ["MX_FP8_LOADERLESS"] = "1"
            ld = MdlLoader(model)
            ld._tp_size, ld._tp_rank = tp, tp_rank
            weights = []
            for e in range(lo, lo + per):       # an expert-parallel rank is fed its own experts
                for name in ("gate_proj", "up_proj", "down_proj"):
                    for suffix in ("weight", "weight_scale_inv"):
                        key = f"{prefix}experts.{e}.{name}.{suffix}"
                        t = torch.from_numpy(tensors[key].copy())
                        weights.append((key, t.view(F8) if suffix == "weight" else t))
            ld.load_weights(weights)
            cases.append({
                "tag": tag, "experts": experts, "ep": ep, "tp": tp, "rank": rank, "inter": inter,
                "hidden": hidden, "block": block, "seed": seed,
                "w13_weight": ex.w13_weight.data.view(torch.uint8).tolist(),
                "w2_weight": ex.w2_weight.data.view(torch.uint8).tolist(),
                "w13_scale": ex.w13_weight_scale.data.tolist(),
                "w2_scale": ex.w2_weight_scale.data.tolist(),
            })
    return cases


def make_toy_reshard(torch, ref_root):
    sys.path.insert(0, ref_root)
    from tests.test_reshard_refit_geometry import ToyModel, _manifest
    from modelexpress.refit.reshard.geometry import capture_geometry
    from modelexpress.refit.reshard.slice_plan import Shard
    from modelexpress.refit.reshard.transfer_plan import (
        SourceInfo, execute_transfer, plan_transfer)
    from modelexpress.refit.reshard.transport import InMemoryReferenceTransport

    shapes = {n: tuple(s) for n, _d, s in _manifest()}
    srcs, base = {}, 0.0
    for name, shape in shapes.items():
        n = int(np.prod(shape))
        srcs[name] = (base + torch.arange(n, dtype=torch.float32)).reshape(shape).contiguous()
        base += n
    truth_model = ToyModel()
    truth_model.load_weights(list(srcs.items()))
    truth = {n: p.detach().clone() for n, p in truth_model.named_parameters()}
    with torch.device("meta"):
        meta = ToyModel()
    capture = capture_geometry(meta, _manifest())
    out = {"manifest": [[n, list(s)] for n, s in shapes.items()], "variants": []}
    out["copies"] = [{"src_name": c.src_name, "op_chain": _chain_json(c.op_chain),
                      "param_name": c.param_name, "dest_offset": c.dest_offset,
                      "dest_shape": list(c.dest_shape), "dest_stride": list(c.dest_stride)}
                     for c in capture.copies]
    out["truth"] = {n: t.reshape(-1).tolist() for n, t in truth.items()}
    out["param_shapes"] = {n: list(t.shape) for n, t in truth.items()}
    # variant A: one whole shard per source; variant B: dim-0 halves
    for nsplit in (1, 2):
        recon = ToyModel()
        for p in recon.parameters():
            torch.nn.init.zeros_(p)
        params = dict(recon.named_parameters())
        sources, keep = {}, []
        for name, t in srcs.items():
            shards = []
            rows = t.shape[0]
            per = rows // nsplit
            for s in range(nsplit):
                piece = t[s * per:(s + 1) * per].contiguous()
                keep.append(piece)
                shards.append(Shard((s * per,) + (0,) * (t.dim() - 1), tuple(piece.shape),
                                    f"{name}#{s}", piece.data_ptr(), 4))
            sources[name] = SourceInfo(tuple(t.shape), torch.float32, 4, shards)
        plan = plan_transfer(capture, sources, max_segments_per_copy=10 ** 9)
        assert plan.fallback == []
        bases = {sh.session: sh.addr for si in sources.values() for sh in si.shards}
        segs = [[s.session, s.src_addr - bases[s.session], s.param_name, s.dst_byte, s.nbytes]
                for s in plan.segments]
        execute_transfer(plan, lambda n: params[n].data_ptr(), InMemoryReferenceTransport())
        for n in truth:
            assert torch.equal(params[n], truth[n]), n
        out["variants"].append({"nsplit": nsplit, "segments": segs})
    return out


def make_capture_pin(torch):
    """The REFERENCE's capture_geometry + resolve_slice on tests/hooked_model.py
    (a meta twin, as the reference's receiver captures): for every recorded copy
    the source box, where it lands and the destination strides in source-dim
    order.  The test runs this repository's capture on the same model and must
    resolve to the same boxes."""
    sys.path.insert(0, os.path.dirname(HERE))
    import hooked_model as H
    from modelexpress.refit.reshard.geometry import capture_geometry
    from modelexpress.refit.reshard.slice_plan import resolve_slice
    from modelexpress.refit.reshard.types import UnsupportedReshard

    with torch.device("meta"):
        twin = H.HookedModel()
    man = H.manifest()
    shapes = {n: s for n, _d, s in man}
    cap = capture_geometry(twin, man, default_weight_loader=H.default_weight_loader)
    out = {"unsupported": list(cap.unsupported), "unattributed": cap.unattributed, "copies": []}
    for c in cap.copies:
        rec = {"src": c.src_name, "param": c.param_name, "dest_offset": int(c.dest_offset),
               "dest_shape": list(c.dest_shape)}
        try:
            box, dstride = resolve_slice(c, shapes[c.src_name])
            rec["box"] = [list(b) for b in box]
            rec["dest_stride_src"] = [int(x) for x in dstride]
        except UnsupportedReshard as e:
            rec["unsupported"] = str(e)
        out["copies"].append(rec)
    return out


def make_shard_table():
    """The reference's shard-table wire blob for a small table (one shard with a
    digest, one without, a replicated 1-D tensor)."""
    from modelexpress.refit.reshard.rendezvous import (PublishedShard, PublishedTensor,
                                                       decode_shard_table, encode_shard_table)

    table = [
        PublishedTensor("model.layers.0.self_attn.q_proj.weight", "torch.bfloat16", 2, (4096, 4096), [
            PublishedShard("trainer-0", 0, 140000000000000, (0, 0), (512, 4096), "00112233445566778899aabbccddeeff"),
            PublishedShard("trainer-1", 1, 140000004194304, (512, 0), (512, 4096), None)]),
        PublishedTensor("model.norm.weight", "torch.float32", 4, (4096,), [
            PublishedShard("trainer-0", 0, 140000008388608, (0,), (4096,), "ffeeddccbbaa99887766554433221100")]),
    ]
    blob = encode_shard_table(table)
    back = decode_shard_table(blob)
    assert [t.name for t in back] == [t.name for t in table]
    return {"blob": blob.decode("utf-8")}


def make_vllm_layers(torch, out_path):
    """Drive real vLLM parallel layers' weight_loaders on CPU with the TP rank
    patched, for a tiny Llama-shaped layer set.  Records full inputs' seeds and
    the per-rank outputs."""
    import vllm  # noqa: F401
    from unittest import mock
    from vllm.config import DeviceConfig, VllmConfig, set_current_vllm_config
    from vllm.model_executor.layers import linear as L
    from vllm.model_executor.layers import vocab_parallel_embedding as V

    TP, H, QH, KVH, HD, I, VOC = 4, 64, 8, 4, 16, 96, 1000  # vocab 1000 pads to 1024
    res = {"meta": np.array([TP, H, QH, KVH, HD, I, VOC], dtype=np.int64),
           "vllm_version": np.array(vllm.__version__)}
    rng = np.random.default_rng(5)

    def full(shape):
        return torch.from_numpy(rng.integers(0, 1 << 16, size=shape, dtype=np.uint16)
                                .astype(np.int32)).to(torch.int32)

    def to_bf16(t_u16):
        return t_u16.to(torch.int16).view(torch.bfloat16) if False else \
            torch.from_numpy(t_u16.numpy().astype(np.uint16)).view(torch.bfloat16)

    srcs = {
        "q_proj": full((QH * HD, H)), "k_proj": full((KVH * HD, H)), "v_proj": full((KVH * HD, H)),
        "o_proj": full((H, QH * HD)), "gate_proj": full((I, H)), "up_proj": full((I, H)),
        "down_proj": full((H, I)), "embed": full((VOC, H)),
        "q_bias": full((QH * HD,)), "k_bias": full((KVH * HD,)), "v_bias": full((KVH * HD,)),
    }
    for k, v in srcs.items():
        res[f"src/{k}"] = v.numpy().astype(np.uint16)
    bf = {k: to_bf16(v) for k, v in srcs.items()}
    cfg = VllmConfig(device_config=DeviceConfig(device="cpu"))
    mods = ["vllm.model_executor.layers.linear",
            "vllm.model_executor.layers.vocab_parallel_embedding",
            "vllm.model_executor.parameter", "vllm.model_executor.utils",
            "vllm.distributed.parallel_state"]
    import importlib
    for rank in range(TP):
        patches = []
        for m in mods:
            mod = importlib.import_module(m)
            for fn, val in (("get_tensor_model_parallel_rank", rank),
                            ("get_tensor_model_parallel_world_size", TP)):
                if hasattr(mod, fn):
                    patches.append(mock.patch.object(mod, fn, lambda v=val: v))
        for p in patches:
            p.start()
        try:
            with set_current_vllm_config(cfg):
                torch.set_default_dtype(torch.bfloat16)
                try:
                    qkv = L.QKVParallelLinear(H, HD, QH, KVH, bias=True)
                    gu = L.MergedColumnParallelLinear(H, [I, I], bias=False)
                    o = L.RowParallelLinear(QH * HD, H, bias=False)
                    down = L.RowParallelLinear(I, H, bias=False)
                    emb = V.VocabParallelEmbedding(VOC, H)
                finally:
                    torch.set_default_dtype(torch.float32)
                for sid, nm in (("q", "q_proj"), ("k", "k_proj"), ("v", "v_proj")):
                    qkv.weight.weight_loader(qkv.weight, bf[nm], sid)
                for sid, nm in (("q", "q_bias"), ("k", "k_bias"), ("v", "v_bias")):
                    qkv.bias.weight_loader(qkv.bias, bf[nm], sid)
                gu.weight.weight_loader(gu.weight, bf["gate_proj"], 0)
                gu.weight.weight_loader(gu.weight, bf["up_proj"], 1)
                o.weight.weight_loader(o.weight, bf["o_proj"])
                down.weight.weight_loader(down.weight, bf["down_proj"])
                emb.weight.weight_loader(emb.weight, bf["embed"])
                for nm, p in (("qkv_w", qkv.weight), ("qkv_b", qkv.bias), ("gate_up", gu.weight),
                              ("o", o.weight), ("down", down.weight), ("embed", emb.weight)):
                    res[f"rank{rank}/{nm}"] = (
                        p.data.contiguous().view(torch.int16).numpy().view(np.uint16).copy())
        finally:
            for p in patches:
                p.stop()
    np.savez_compressed(out_path, **res)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True,
                    help="path to the reference's modelexpress_client/python")
    ap.add_argument("--vllm", action="store_true", help="also drive real vLLM layers")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import torch
    from modelexpress.tensor_utils import safe_checksum
    from modelexpress.refit.reshard.verify import tensor_digest
    from modelexpress.refit.reshard import slice_plan, types
    from modelexpress.engines.vllm.refit import MdlLoader

    def dump(name, obj):
        with open(os.path.join(HERE, name), "w") as f:
            json.dump(obj, f, separators=(",", ":"))
        print("wrote", name)

    dump("digests.json", make_digests(torch, safe_checksum, tensor_digest))
    dump("slice_plan.json", make_slice_plan(slice_plan, types))
    dump("installer.json", make_installer(torch, MdlLoader))
    dump("expert_slots.json", make_expert_slots(torch, MdlLoader))
    dump("toy_reshard.json", make_toy_reshard(torch, args.reference))
    dump("capture_pin.json", make_capture_pin(torch))
    dump("shard_table.json", make_shard_table())
    if args.vllm:
        make_vllm_layers(torch, os.path.join(HERE, "vllm_layers.npz"))
        print("wrote vllm_layers.npz")


if __name__ == "__main__":
    main()
