"""Fan-out and reshard kernels.  On one GPU the ranks are emulated as buffers
of the same device and the launches run one after another (kernels that wait
on each other never share a GPU); with two or more GPUs the real peer path runs."""

import numpy as np
import pytest

from helpers import read_full_tensors, tiny_dense_config
from make_golden import golden_bytes
from oracle import ref_port as R

pytestmark = pytest.mark.gpu


def _spans(torch, tensors):
    return [(t.data_ptr(), t.numel() * t.element_size()) for t in tensors]


@pytest.mark.parametrize("engine", ["vector", "bulk", "dma"])
def test_fanout_single_gpu_loopback(engine, monkeypatch):
    """Root pushes to a 'child' on the same device; then the child's kernel runs
    and finds every chunk counter already satisfied.  Every engine; the ranges
    whose size is not a multiple of 16 are followed by a range of a thousand pieces,
    so that every CTA of the bulk engine reuses each of its shared-memory stages
    after a piece that took a stage without loading into it."""
    import torch

    from modelexpress_b200 import digest
    from modelexpress_b200.runtime import Context

    monkeypatch.setenv("MXB_FANOUT_ENGINE", engine)
    ctx = Context([0])
    sizes = [1 << 20, 4096 + 16, 333 * 16, 100, 5 << 20, 52, 64 << 20, 48]
    src = [torch.from_numpy(golden_bytes(20 + i, n)).cuda() for i, n in enumerate(sizes)]
    dst = [torch.zeros(n, dtype=torch.uint8, device="cuda") for n in sizes]
    torch.cuda.synchronize()
    for chunk in (1 << 20, 64 << 10):
        for d in dst:
            d.zero_()
        torch.cuda.synchronize()
        # the store kernel also with 256 KiB pieces (what a one-hop push uses)
        piece = 256 << 10 if (engine == "vector" and chunk == 1 << 20) else 64 << 10
        root = ctx.fanout(_spans(torch, src), chunk, 0, piece)
        leaf = ctx.fanout(_spans(torch, dst), chunk, 0, piece)
        root.add_child(_spans(torch, dst), leaf.counters)
        for _ in range(2):  # counters are cumulative: a second broadcast needs no reset
            root.run(True, 2000)
            assert root.wait() > 0
            leaf.run(False, 2000)
            leaf.wait()
        for s, d in zip(src, dst):
            assert torch.equal(s, d)
        a = digest.digest_many(src)
        b = digest.digest_many(dst)
        assert a == b
        root.close()
        leaf.close()
    ctx.close()


@pytest.mark.parametrize("engine", ["vector", "bulk"])
def test_fanout_wait_runs_out_cleanly(engine):
    """A node whose parent never delivers: the bounded wait ends, the call
    reports a timeout and the context keeps working."""
    import torch

    from modelexpress_b200._lib import MxbTimeout
    from modelexpress_b200.runtime import Context

    ctx = Context([0])
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    node = ctx.fanout(_spans(torch, [buf]), 1 << 16, 0)
    node.set_engine(engine)
    node.run(False, 50)
    with pytest.raises(MxbTimeout):
        node.wait()
    with pytest.raises(TimeoutError):
        node.run(False, 50)
        node.wait()
    # still usable
    src = torch.from_numpy(golden_bytes(1, 1 << 16)).cuda()
    torch.cuda.synchronize()
    ctx.scatter([(src.data_ptr(), buf.data_ptr(), 1, 1 << 16, 1 << 16, 1 << 16)], 0)
    assert torch.equal(src, buf)
    node.close()
    ctx.close()


def test_manifest_matching_rules():
    from modelexpress_b200.fanout import (ManifestMismatchError, TensorDescriptor, match_manifests,
                                          topology)

    s = [TensorDescriptor("a", 100, 64, 0, "bf16"), TensorDescriptor("b", 200, 32, 0, "bf16")]
    t = [TensorDescriptor("b", 900, 32, 1, "bf16"), TensorDescriptor("a", 800, 64, 1, "bf16")]
    assert match_manifests(s, t) == [("b", 200, 900, 32), ("a", 100, 800, 64)]
    with pytest.raises(ManifestMismatchError):
        match_manifests(s, [TensorDescriptor("a", 1, 65, 1, "bf16")])
    with pytest.raises(ManifestMismatchError):
        match_manifests(s, [TensorDescriptor("a", 1, 64, 1, "f16")])
    with pytest.raises(ManifestMismatchError):
        match_manifests(s, [TensorDescriptor("c", 1, 64, 1, "bf16")])
    assert topology("chain", 4) == [[1], [2], [3], []]
    assert topology("tree", 5) == [[1, 2], [3, 4], [], [], []]
    assert topology("flat", 3, root=1) == [[], [0, 2], []]


@pytest.mark.parametrize("kind,engine", [("chain", "vector"), ("tree", "vector"), ("flat", "vector"),
                                         ("chain", "bulk"), ("tree", "bulk"), ("flat", "dma"), ("chain", "dma")])
def test_fanout_across_gpus(kind, engine):
    import torch

    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    from modelexpress_b200.fanout import Broadcast
    from modelexpress_b200.runtime import Context

    devs = list(range(min(n, 4)))
    ctx = Context(devs)
    # large enough on average (>= 4 MiB per range) for the copy-engine push to be taken when asked for
    sizes = [3 << 20, 4096 + 16, 7 << 20, 160, 24 << 20]
    bufs = []
    for i, d in enumerate(devs):
        if i == 0:
            bufs.append([torch.from_numpy(golden_bytes(50 + j, s)).to(f"cuda:{d}") for j, s in enumerate(sizes)])
        else:
            bufs.append([torch.zeros(s, dtype=torch.uint8, device=f"cuda:{d}") for s in sizes])
    for d in devs:
        torch.cuda.synchronize(d)
    bc = Broadcast(ctx, devs, [_spans(torch, b) for b in bufs], 1 << 20, kind, engine=engine)
    for _ in range(2):
        for b in bufs[1:]:
            for t in b:
                t.zero_()
        for d in devs:
            torch.cuda.synchronize(d)
        bc.run(5000)
    for b in bufs[1:]:
        for s, t in zip(bufs[0], b):
            assert torch.equal(s.cpu(), t.cpu())
    bc.close()
    ctx.close()


def _reshard_case(torch, tmp_path, devices):
    from modelexpress_b200 import layout, reshard, synth
    from modelexpress_b200.runtime import Context
    from modelexpress_b200.safetensors_index import checkpoint_index

    cfg = tiny_dense_config()
    d = str(tmp_path)
    synth.write_checkpoint(d, synth.dense_tensors(cfg), cfg.seed, 1)
    full = read_full_tensors(d)
    idx = checkpoint_index(d)
    index = {n: {"shape": i["shape"], "dtype": i["dtype"]} for n, i in idx.items()}
    world = tp = 8
    pieces = R.fsdp_shards(full, world)
    sa = reshard.shard_arena(index, world)
    pa = reshard.param_arena(layout.plan_checkpoint(index, 0, tp))
    ctx = Context(sorted(set(devices)))
    shard_t, param_t = [], []
    for s in range(world):
        host = np.zeros(sa.total, dtype=np.uint8)
        for n, piece in pieces[s].items():
            b = piece.view(np.uint8)
            host[sa.offsets[n]: sa.offsets[n] + b.size] = b
        shard_t.append(torch.from_numpy(host).to(f"cuda:{devices[s]}"))
        param_t.append(torch.zeros(pa.total, dtype=torch.uint8, device=f"cuda:{devices[s]}"))
    for dv in set(devices):
        torch.cuda.synchronize(dv)
    moved = 0
    for s in range(world):  # every source rank pushes its pieces to every destination
        recs = reshard.plan_reshard(index, world, tp, s, shard_t[s].data_ptr(),
                                    [p.data_ptr() for p in param_t])
        moved += reshard.reshard_bytes(recs)
        ctx.scatter(recs, devices[s])
    shapes = {n: a.shape for n, a in full.items()}
    for t in range(tp):
        want = R.regather_and_reslice(pieces, shapes, t, tp)
        host = param_t[t].cpu().numpy()
        for n, a in want.items():
            got = host[pa.offsets[n]: pa.offsets[n] + a.nbytes].view(a.dtype).reshape(a.shape)
            assert np.array_equal(got, a), (t, n)
    assert moved == sum(a.nbytes for a in R.load_and_shard(full, 0, tp).values()) * tp
    ctx.close()


def test_reshard_emulated_ranks_one_gpu(tmp_path):
    import torch

    _reshard_case(torch, tmp_path, [0] * 8)


def test_reshard_across_gpus(tmp_path):
    import torch

    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    _reshard_case(torch, tmp_path, [i % n for i in range(8)])


def test_module_manifest_follows_reference_rules():
    import torch

    from modelexpress_b200.fanout import manifest_from_module

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Parameter(torch.zeros(4, 8, device="cuda"))
            self.tied = self.a                                  # same data_ptr: listed once
            base = torch.zeros(8, 8, device="cuda")
            self.register_buffer("strided", base[:, ::2])       # non-contiguous -> storage bytes
            self.register_buffer("empty", torch.zeros(0, device="cuda"))
            self.register_buffer("cpu_buf", torch.zeros(3))     # not on the accelerator

    rows = manifest_from_module(M())
    names = [r.name for r in rows]
    assert names == ["a", "strided.__storage", "empty"]
    assert rows[0].size == 4 * 8 * 4 and rows[1].size == 8 * 8 * 4 and rows[2].size == 0


def test_strict_verify_catches_a_misplaced_shard():
    """nixl_staged_transfer.py:529-549: digests of every published box are recomputed
    from the assembled tensor; one launch for all of them."""
    import torch

    from modelexpress_b200 import planner, verify

    full = torch.arange(64 * 1024, dtype=torch.int32, device="cuda").reshape(64, 1024)
    boxes = {s: full[s * 16:(s + 1) * 16].contiguous() for s in range(4)}
    dig = verify.published_digests(boxes)
    shards = [planner.ShardSpec((s * 16, 0), (16, 1024), f"t{s}", 0, 4, dig[s]) for s in range(4)]
    sources = {"w": planner.SourceSpec((64, 1024), "i32", 4, shards)}
    assert verify.verify_sources({"w": full.reshape(-1)}, sources) == 4
    bad = full.clone()
    bad[16:32], bad[32:48] = full[32:48].clone(), full[16:32].clone()   # right bytes, wrong place
    with pytest.raises(RuntimeError, match="digest mismatch for source 'w' at offset \\(16, 0\\)"):
        verify.verify_sources({"w": bad}, sources)
    shards[2].digest = None
    with pytest.raises(RuntimeError, match="did not publish"):
        verify.verify_sources({"w": full}, sources)
    with pytest.raises(ValueError, match="rank mismatch"):
        verify.shard_region(full, (64, 1024), (1,), (2, 3))
    region = verify.shard_region(full.reshape(-1), (64, 1024), (1, 2), (2, 3))
    assert torch.equal(region, full[1:3, 2:5])


def test_reshard_receiver_prepare_once_update_every_step():
    """The refit cycle of refit/reshard/receiver.py:447-1043 on one GPU: four
    emulated trainer ranks publish row shards (with digests) of every HF tensor,
    the receiver captures the engine's loader once and replays one resident table
    per step.  Parameters must equal what the loader makes of the assembled full
    tensors, for the first step and after the trainers rewrote their shards in
    place; a shard that no longer matches its published digest stops the step
    before a byte is written."""
    import torch

    from modelexpress_b200.refit import (PublishedTensor, ReshardReceiver, decode_shard_table,
                                         encode_shard_table, merge_shard_tables,
                                         publish_local_shards)
    from modelexpress_b200.verify import published_digests

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")

    class Engine(torch.nn.Module):
        def __init__(self, rank):
            super().__init__()
            self.rank = rank
            self.qkv = torch.nn.Parameter(torch.zeros(256 + 64 + 64, 512, dtype=torch.bfloat16))
            self.down = torch.nn.Parameter(torch.zeros(512, 384, dtype=torch.bfloat16))
            self.router = torch.nn.Parameter(torch.zeros(4, 512, dtype=torch.float32))
            self.norm = torch.nn.Parameter(torch.zeros(512, dtype=torch.bfloat16))

        def load_weights(self, weights):
            r = self.rank
            for name, w in weights:
                if name in ("q", "k", "v"):
                    rows = {"q": 256, "k": 64, "v": 64}[name]
                    at = {"q": 0, "k": 256, "v": 320}[name]
                    self.qkv.data.narrow(0, at, rows).copy_(w.narrow(0, r * rows, rows))
                elif name == "down":
                    self.down.data.copy_(w[:, r * 384:(r + 1) * 384])
                elif name == "router":
                    self.router.data.copy_(w)
                elif name == "norm":
                    self.norm.data.copy_(w)

    shapes = {"q": (512, 512), "k": (128, 512), "v": (128, 512), "down": (512, 768),
              "router": (4, 512), "norm": (512,)}
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    world = 4
    # trainer rank t owns rows [t*R/4, (t+1)*R/4) of every tensor, in its own buffer
    shards = {n: [torch.randn((s[0] // world,) + s[1:], device="cuda", generator=g).to(torch.bfloat16)
                  for _ in range(world)] for n, s in shapes.items()}

    def tables():
        # each trainer rank publishes its own table (digests from one launch), which
        # travels as the wire blob and is decoded and merged on the receiving side
        blobs = []
        for t in range(world):
            blobs.append(encode_shard_table(publish_local_shards(
                {n: (shards[n][t], shapes[n],
                     (t * (shapes[n][0] // world),) + (0,) * (len(shapes[n]) - 1)) for n in shapes},
                f"trainer{t}")))
        decoded = [decode_shard_table(b) for b in blobs]
        assert decoded[1][0].shards[0].digest == published_digests({"x": shards["q"][1]})["x"]
        # a replica of rank 0 publishing the same geometry again must not add reads
        return merge_shard_tables(decoded + [decoded[0]])

    def truth(rank):
        m = Engine(rank).cuda()
        m.load_weights((n, torch.cat(shards[n], 0)) for n in shapes)
        return m

    for rank in (0, 1):
        model = Engine(rank).cuda()
        rx = ReshardReceiver(model, device="cuda:0")
        plan = rx.prepare(tables())
        assert plan["converts"] == ["router"] and plan["sources_unused"] == []
        assert plan["copies"] == 6 and plan["coverage"] > 0.99
        st = rx.update_weights(1, verify=True)
        assert st["shards_verified"] == world * len(shapes) and st["bytes"] == plan["bytes_per_step"]
        want = truth(rank)
        for (n, a), (_n, b) in zip(model.state_dict().items(), want.state_dict().items()):
            assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), (rank, n)
        # next step: the trainers rewrite their shards in place, same addresses
        for n in shapes:
            for t in range(world):
                shards[n][t].copy_(torch.randn(shards[n][t].shape, device="cuda", generator=g))
        torch.cuda.synchronize()
        rx.update_weights(2)
        want = truth(rank)
        for (n, a), (_n, b) in zip(model.state_dict().items(), want.state_dict().items()):
            assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), (rank, n)
        # the published digests are those of step 1: the strict gate refuses step 3 untouched
        before = {n: p.detach().clone() for n, p in model.state_dict().items()}
        with pytest.raises(RuntimeError, match="digest mismatch"):
            rx.update_weights(3, verify=True)
        for n, p in model.state_dict().items():
            assert torch.equal(p, before[n]), n
        rx.close()

    # fail closed: a source the loader computes on cannot be planned
    class Casting(Engine):
        def load_weights(self, weights):
            for name, w in weights:
                if name == "norm":
                    self.norm.data.copy_(w.float() * 2)

    with pytest.raises(RuntimeError, match="cannot plan"):
        ReshardReceiver(Casting(0).cuda(), device="cuda:0").prepare(tables())
    with pytest.raises(ValueError, match="inconsistent shape/dtype"):
        merge_shard_tables([[PublishedTensor("q", "torch.bfloat16", 2, (512, 512), [])],
                            [PublishedTensor("q", "torch.bfloat16", 2, (256, 512), [])]])


@pytest.mark.gpu
@pytest.mark.parametrize("fused", ["1", "0"])
def test_update_weights_returns_with_the_bytes_in_place(fused, monkeypatch):
    """update_weights must not return before the kernels have finished: a payload of
    several hundred MB with a dtype-changing source (read in place and cast by the
    convert kernel, or staged in the served dtype and cast afterwards) is compared
    right after the call returns, and the reported read time must be that of the
    copy, not of its enqueue."""
    import torch

    monkeypatch.setenv("MXB_RESHARD_FUSED_CASTS", fused)

    from modelexpress_b200.planner import ShardSpec, SourceSpec
    from modelexpress_b200.refit import IncompleteRefit, ReshardReceiver

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    rows, cols = 16384, 8192                      # 256 MiB of bf16

    class Engine(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.big = torch.nn.Parameter(torch.zeros(rows, cols, dtype=torch.bfloat16))
            self.gate = torch.nn.Parameter(torch.zeros(2048, cols, dtype=torch.float32))   # cast on the way in
            self.untouched = torch.nn.Parameter(torch.ones(4096, dtype=torch.bfloat16))

        def load_weights(self, weights):
            for name, w in weights:
                if name == "big":
                    self.big.data.copy_(w)
                elif name == "gate":
                    self.gate.data.copy_(w)

    g = torch.Generator(device="cuda")
    g.manual_seed(11)
    big = torch.randn(rows, cols, device="cuda", generator=g).to(torch.bfloat16)
    gate = torch.randn(2048, cols, device="cuda", generator=g).to(torch.bfloat16)
    sources = {
        "big": SourceSpec((rows, cols), torch.bfloat16, 2,
                          [ShardSpec((0, 0), (rows, cols), "t0", big.data_ptr(), 2)]),
        "gate": SourceSpec((2048, cols), torch.bfloat16, 2,
                           [ShardSpec((0, 0), (2048, cols), "t0", gate.data_ptr(), 2)]),
    }
    model = Engine().cuda()
    rx = ReshardReceiver(model, device="cuda:0")
    plan = rx.prepare(sources)
    assert plan["converts"] == ["gate"] and plan["params_missed"] == ["untouched"]
    assert plan["fused_casts"] == (["gate"] if fused == "1" else [])
    assert plan["bytes_per_step"] == big.numel() * 2 + gate.numel() * 2
    assert (rx._staging.numel() <= 1) == (fused == "1")      # nothing is staged when the cast is fused
    for step in range(3):
        model.big.data.zero_()
        model.gate.data.zero_()
        torch.cuda.synchronize()
        st = rx.update_weights(step)
        # no synchronize here: what the call returned must already be true
        assert torch.equal(model.big.data, big), step
        assert torch.equal(model.gate.data, gate.float()), step
        assert st["read_s"] > 50e-6 and st["gbps"] < 20000, st     # a copy of 288 MiB, not an enqueue
        big.add_(1.0)
        gate.mul_(0.5)
        torch.cuda.synchronize()
    rx.close()
    # the coverage gate: 'untouched' keeps its old value, which an opted-in complete refit refuses
    import os

    os.environ["MXB_RESHARD_REQUIRE_FULL_COVERAGE"] = "1"
    os.environ["MXB_RESHARD_COVERAGE_FLOOR"] = "0.999999"
    try:
        with pytest.raises(IncompleteRefit, match="untouched"):
            ReshardReceiver(model, device="cuda:0").prepare(sources)
    finally:
        del os.environ["MXB_RESHARD_REQUIRE_FULL_COVERAGE"], os.environ["MXB_RESHARD_COVERAGE_FLOOR"]
