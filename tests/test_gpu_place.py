"""Checkpoint placement through the staging ring against the oracle's load-and-shard."""

import numpy as np
import pytest

from helpers import read_full_tensors, tiny_dense_config
from oracle import ref_port as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ckpts(tmp_path_factory):
    import torch

    from modelexpress_b200 import synth

    assert torch.cuda.is_available()
    tiny = str(tmp_path_factory.mktemp("tiny"))
    cfg = tiny_dense_config()
    synth.write_checkpoint(tiny, synth.dense_tensors(cfg), cfg.seed, cfg.files)
    # the CPU-runnable benchmark configuration exactly as stated: 4 layers, hidden 1024,
    # intermediate 2816, 16 q / 4 kv heads of 64, vocabulary 32000, untied lm_head, one file
    small = str(tmp_path_factory.mktemp("small"))
    scfg = synth.SMALL_LLAMA
    assert (scfg.layers, scfg.hidden, scfg.intermediate, scfg.q_heads, scfg.kv_heads, scfg.head_dim,
            scfg.vocab, scfg.seed) == (4, 1024, 2816, 16, 4, 64, 32000, 0)
    synth.write_checkpoint(small, synth.dense_tensors(scfg), scfg.seed, 1)
    return tiny, small


def _as_np(t):
    import torch

    t = t.detach().cpu().contiguous()
    if t.element_size() == 2:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.element_size() == 1:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def _check(placed, want):
    assert set(placed.params) == set(want)
    for n, a in want.items():
        got = _as_np(placed.params[n])
        assert got.shape == a.shape, n
        assert np.array_equal(got, a), n


@pytest.mark.parametrize("mode", ["copy_engine", "zero_copy"])
@pytest.mark.parametrize("tp", [1, 8])
def test_tiny_checkpoint_every_rank(ckpts, tp, mode):
    from modelexpress_b200.loader import place_checkpoint
    from modelexpress_b200.runtime import PLACE_COPY_ENGINE, PLACE_ZERO_COPY, Context

    tiny, _ = ckpts
    full = read_full_tensors(tiny)
    ctx = Context([0])
    ring = ctx.ring(8 << 20, 4, 0)  # 2 MiB slots: tensors span several chunks
    m = PLACE_COPY_ENGINE if mode == "copy_engine" else PLACE_ZERO_COPY
    try:
        for rank in range(tp):
            placed = place_checkpoint(tiny, rank, tp, "cuda:0", ring=ring, host_threads=4, mode=m)
            _check(placed, R.load_and_shard(full, rank, tp))
            assert placed.stats.bytes_placed == placed.plan.bytes_placed
            assert placed.stats.chunks >= 1 and placed.stats.launches == placed.stats.chunks
    finally:
        ring.close()
        ctx.close()


def test_small_llama_tp1_byte_exact(ckpts):
    """The reference-runnable configuration: TP=1 load onto one GPU, checked
    byte for byte and by both reference digests per tensor."""
    from modelexpress_b200 import digest
    from modelexpress_b200.loader import place_checkpoint

    _, small = ckpts
    full = read_full_tensors(small)
    assert len(full) == 39 and sum(a.nbytes for a in full.values()) == 221_267_968
    placed = place_checkpoint(small, 0, 1, "cuda:0", ring_bytes=64 << 20, ring_slots=4, host_threads=4)
    want = R.load_and_shard(full, 0, 1)
    _check(placed, want)
    assert placed.stats.bytes_placed == 221_267_968
    names = sorted(want)
    res = digest.digest_many([placed.params[n] for n in names])
    for n, r in zip(names, res):
        assert r["safe_checksum"] == R.safe_checksum(want[n]), n
        assert r["tensor_digest"] == R.tensor_digest(want[n]), n


@pytest.mark.parametrize("mode", ["copy_engine", "zero_copy"])
def test_pinned_host_image_is_read_in_place(ckpts, mode):
    """Files kept mapped and page-locked (pin="pages"): the copy engine (or, in
    zero-copy mode, the kernel) reads the slices where they lie, no byte goes
    through the ring, and the shards are the oracle's for every rank."""
    from modelexpress_b200.loader import HostImages, place_checkpoint
    from modelexpress_b200.runtime import PLACE_COPY_ENGINE, PLACE_ZERO_COPY, Context

    tiny, _ = ckpts
    full = read_full_tensors(tiny)
    ctx = Context([0])
    ring = ctx.ring(8 << 20, 4, 0)
    images = HostImages()
    m = PLACE_COPY_ENGINE if mode == "copy_engine" else PLACE_ZERO_COPY
    try:
        for tp in (1, 8):
            for rank in range(tp):
                placed = place_checkpoint(tiny, rank, tp, "cuda:0", ring=ring, host_threads=4, mode=m,
                                          pin="pages", images=images)
                _check(placed, R.load_and_shard(full, rank, tp))
                assert placed.stats.bytes_direct == placed.stats.bytes_placed == placed.plan.bytes_placed
        assert images.pinned_bytes > 0
        # a second load of the same rank pins nothing new
        before = images.pinned_bytes
        placed = place_checkpoint(tiny, 0, 8, "cuda:0", ring=ring, mode=m, pin="pages", images=images)
        assert images.pinned_bytes == before and placed.timings["pin"] < 0.05
    finally:
        ring.close()
        images.close()
        ctx.close()


def test_pin_after_the_first_load_and_mixed_sources(ckpts):
    """pin="pages_after": the first load goes through the ring, later ones find the
    ranges pinned.  A call whose sources are partly pinned, partly pageable places both."""
    import time

    from modelexpress_b200.loader import HostImages, place_checkpoint
    from modelexpress_b200.runtime import Context

    _, small = ckpts
    full = read_full_tensors(small)
    want = R.load_and_shard(full, 1, 4)
    ctx = Context([0])
    ring = ctx.ring(32 << 20, 4, 0)
    images = HostImages()
    try:
        first = place_checkpoint(small, 1, 4, "cuda:0", ring=ring, host_threads=4, pin="pages_after", images=images)
        _check(first, want)
        assert first.stats.bytes_direct == 0
        for t in ctx._background:
            t.join()
        assert images.pinned_bytes > 0
        second = place_checkpoint(small, 1, 4, "cuda:0", ring=ring, host_threads=4, pin="pages_after", images=images)
        _check(second, want)
        assert second.stats.bytes_direct == second.stats.bytes_placed
        for t in ctx._background:
            t.join()
        # another rank of the same files: its column/vocab slices are new (pageable), the
        # row-parallel tensors were pinned whole by rank 1 -> a mixed call
        third = place_checkpoint(small, 2, 4, "cuda:0", ring=ring, host_threads=4, pin="off")
        _check(third, R.load_and_shard(full, 2, 4))
        mixed = place_checkpoint(small, 2, 4, "cuda:0", ring=ring, host_threads=4, pin="pages_after", images=images)
        _check(mixed, R.load_and_shard(full, 2, 4))
        assert 0 < mixed.stats.bytes_direct < mixed.stats.bytes_placed
    finally:
        for t in ctx._background:
            t.join()
        ring.close()
        images.close()
        ctx.close()


def test_kept_packed_image_replays_without_the_files(ckpts, tmp_path):
    """pin="keep": the first load gathers into a page-locked image of the rank's packed
    bytes; later loads replay it (no gather, no file read), also into parameters at
    other addresses."""
    import shutil

    import torch

    from modelexpress_b200.loader import HostImages, allocate_params, place_checkpoint
    from modelexpress_b200.runtime import Context

    _, small = ckpts
    work = str(tmp_path / "ckpt")
    shutil.copytree(small, work)
    full = read_full_tensors(work)
    ctx = Context([0])
    ring = ctx.ring(32 << 20, 4, 0)
    images = HostImages()
    try:
        for rank in (0, 3):
            want = R.load_and_shard(full, rank, 4)
            first = place_checkpoint(work, rank, 4, "cuda:0", ring=ring, host_threads=4, pin="keep", images=images)
            _check(first, want)
            assert first.stats.bytes_direct == 0 and first.stats.seconds_gather > 0
            for v in first.params.values():
                v.zero_()
            again = place_checkpoint(work, rank, 4, "cuda:0", ring=ring, params=first.params, pin="keep",
                                     images=images)
            _check(again, want)
            assert again.stats.bytes_direct == again.stats.bytes_placed and again.stats.seconds_gather == 0
            # other destination tensors (other addresses): the image is retargeted, not rebuilt
            other = allocate_params(again.plan, "cuda:0")
            pad = torch.empty(4096 + 16 * rank, dtype=torch.uint8, device="cuda")  # shift the allocator
            moved = place_checkpoint(work, rank, 4, "cuda:0", ring=ring, params=other, pin="keep", images=images)
            _check(moved, want)
            assert moved.stats.seconds_gather == 0
            del pad
        assert images.packed_bytes > 0
        # a destination at another 16-byte phase cannot reuse the packing: a new image is made
        plan = moved.plan
        skew = {}
        for n, spec in plan.params.items():
            numel = 1
            for e in spec.shape:
                numel *= int(e)
            raw = torch.zeros(numel * 2 + 8, dtype=torch.uint8, device="cuda")
            skew[n] = raw[8: 8 + numel * 2].view(torch.bfloat16).reshape(tuple(spec.shape))
        skewed = place_checkpoint(work, 3, 4, "cuda:0", ring=ring, params=skew, host_threads=4, pin="keep",
                                  images=images)
        _check(skewed, R.load_and_shard(full, 3, 4))
        assert skewed.stats.seconds_gather > 0
    finally:
        images.close()
        ring.close()
        ctx.close()


def test_vocab_padding_rows_are_zero(tmp_path):
    import torch

    from modelexpress_b200 import synth
    from modelexpress_b200.loader import place_checkpoint

    cfg = synth.DenseConfig("pad", 1, 128, 256, 4, 4, 32, 1000, False, 3, 1)  # 1000 pads to 1024
    d = str(tmp_path)
    synth.write_checkpoint(d, synth.dense_tensors(cfg), cfg.seed, 1)
    full = read_full_tensors(d)
    for rank in (0, 3):
        placed = place_checkpoint(d, rank, 4, "cuda:0", ring_bytes=8 << 20, ring_slots=2, host_threads=2)
        _check(placed, R.load_and_shard(full, rank, 4))
    emb = placed.params["model.embed_tokens.weight"]
    assert emb.shape == (256, 128) and bool((emb[232:] == 0).all())


def test_strategy_contract(ckpts):
    """load_strategy/base.py:37-76 contract: LoadResult on success, StrategyFailed
    (mutated=False) on an expected miss."""
    import torch

    from modelexpress_b200.layout import plan_checkpoint
    from modelexpress_b200.loader import (B200ScatterStrategy, LoadResult, StrategyFailed,
                                          allocate_params)
    from modelexpress_b200.safetensors_index import checkpoint_index

    tiny, _ = ckpts

    class Adapter:
        def __init__(self, params):
            self.params = params

        def tp_layout(self, result):
            return 1, 2

        def named_destinations(self, result):
            return self.params

    class Cfg:
        model = tiny

    class Ctx:
        model_config = Cfg()
        device_id = 0
        adapter = None

    idx = checkpoint_index(tiny)
    plan = plan_checkpoint({n: {"shape": i["shape"], "dtype": i["dtype"]} for n, i in idx.items()}, 1, 2)
    params = allocate_params(plan, "cuda:0")
    strat = B200ScatterStrategy(ring_bytes=8 << 20, ring_slots=2, host_threads=2)
    ctx = Ctx()
    assert strat.name == "b200_scatter" and not strat.is_available(ctx)
    ctx.adapter = Adapter(params)
    assert strat.is_available(ctx)
    res = strat.load(LoadResult(value="model", model="model"), ctx)
    assert res.metadata["b200_scatter"]["bytes_placed"] == plan.bytes_placed
    want = R.load_and_shard(read_full_tensors(tiny), 1, 2)
    for n, a in want.items():
        assert np.array_equal(_as_np(params[n]), a), n
    Cfg.model = "/nonexistent"
    with pytest.raises(StrategyFailed) as ei:
        strat.load(LoadResult(value="m"), ctx)
    assert ei.value.mutated is False
    strat.rollback(ctx)


def test_fp8_moe_slice_expert_parallel_placement(tmp_path):
    """DeepSeek-V3-style block-FP8 slice: experts expert-parallel into w13/w2 slots with
    their scale blocks, MLA and shared expert tensor-parallel; thousands of small
    records in a handful of launches."""
    import torch

    from modelexpress_b200 import synth
    from modelexpress_b200.loader import place_checkpoint

    cfg = synth.MoEConfig(layers=2, hidden=512, experts=16, moe_intermediate=1024, q_lora=256,
                          kv_lora=128, qk_rope=64, qk_nope=64, v_head=64, heads=16, files=2)
    d = str(tmp_path)
    synth.write_checkpoint(d, synth.moe_tensors(cfg), cfg.seed, cfg.files)
    full = read_full_tensors(d)
    for rank in (0, 5):
        placed = place_checkpoint(d, rank, 8, "cuda:0", ring_bytes=32 << 20, ring_slots=4, host_threads=4)
        want = R.load_and_shard_moe(full, rank, 8)
        assert set(placed.params) == set(want)
        for n, a in want.items():
            got = placed.params[n].detach().cpu().contiguous().view(torch.uint8).numpy()
            assert got.size == a.nbytes, n
            assert np.array_equal(got.reshape(-1), a.view(np.uint8).reshape(-1)), (rank, n)
        assert placed.stats.launches <= 2 * placed.stats.chunks


@pytest.mark.parametrize("mode", ["copy_engine", "zero_copy"])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_ring_random_items_any_alignment(seed, mode):
    """Host -> device items with odd sizes, odd destination phases, pitches that are not
    multiples of 16 and rows larger than a ring slot (split by bytes across chunks),
    against the oracle's memmove loop."""
    import torch

    from make_golden import golden_bytes
    from modelexpress_b200.runtime import PLACE_COPY_ENGINE, PLACE_ZERO_COPY, Context
    from oracle import c_port as C

    rng = np.random.default_rng(seed)
    src = golden_bytes(500 + seed, 24 << 20)
    items_rel, dpos = [], 0
    for _ in range(50):
        kind = int(rng.integers(0, 5))
        if kind == 0:    # a row larger than the 1 MiB slot
            rows, rb = 1, int(rng.integers(1 << 20, 3 << 20))
            sp = dp = rb
        elif kind == 1:  # row-parallel style
            rows, rb = int(rng.integers(2, 600)), 16 * int(rng.integers(1, 200))
            sp, dp = rb * int(rng.integers(2, 6)), rb + 16 * int(rng.integers(0, 3))
        elif kind == 2:  # ragged everything
            rows, rb = int(rng.integers(1, 300)), int(rng.integers(1, 3000))
            sp, dp = rb + int(rng.integers(0, 40)), rb + int(rng.integers(0, 40))
        elif kind == 3:  # multi-row item taller than a slot
            rows, rb = int(rng.integers(700, 1500)), 2048
            sp, dp = 4096, 2048 + 16 * int(rng.integers(0, 2))
        else:            # tiny
            rows, rb = 1, int(rng.integers(1, 64))
            sp = dp = rb
        span_s = (rows - 1) * sp + rb
        span_d = (rows - 1) * dp + rb
        s0 = int(rng.integers(0, src.size - span_s))
        d0 = dpos + int(rng.integers(0, 33))
        items_rel.append((s0, d0, rows, rb, sp, dp))
        dpos = d0 + span_d
    ctx = Context([0])
    ring = ctx.ring(4 << 20, 4, 0)  # 1 MiB slots
    dst_d = torch.full((dpos + 64,), 0x5A, dtype=torch.uint8, device="cuda")
    dst_h = np.full(dpos + 64, 0x5A, dtype=np.uint8)
    torch.cuda.synchronize()
    items = [(src.ctypes.data + s, dst_d.data_ptr() + d, r, rb, sp, dp) for s, d, r, rb, sp, dp in items_rel]
    st = ring.place(items, 3, PLACE_COPY_ENGINE if mode == "copy_engine" else PLACE_ZERO_COPY)
    C.scatter2d([(src.ctypes.data + s, dst_h.ctypes.data + d, r, rb, sp, dp) for s, d, r, rb, sp, dp in items_rel])
    assert np.array_equal(dst_d.cpu().numpy(), dst_h)
    assert st.bytes_placed == sum(r * rb for _s, _d, r, rb, _sp, _dp in items_rel)
    assert st.chunks > 10
    ring.close()
    ctx.close()


def test_sglang_loader_signature_with_stand_ins(ckpts):
    """engines/sglang/loader.py:61-86: keyword-only load_model(model=, model_config=,
    device_config=) on an already initialised model."""
    import torch

    from modelexpress_b200.engines.sglang.loader import MxModelLoader
    from modelexpress_b200.layout import plan_checkpoint
    from modelexpress_b200.loader import torch_dtype
    from modelexpress_b200.safetensors_index import checkpoint_index

    tiny, _ = ckpts
    idx = checkpoint_index(tiny)
    plan = plan_checkpoint({n: {"shape": i["shape"], "dtype": i["dtype"]} for n, i in idx.items()}, 2, 4)

    class Model(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.names = {}
            for i, (n, s) in enumerate(plan.params.items()):
                p = torch.nn.Parameter(torch.zeros(tuple(s.shape), dtype=torch_dtype(s.dtype), device="cuda"),
                                       requires_grad=False)
                self.register_parameter(f"p{i}", p)
                self.names[f"p{i}"] = n

        def named_parameters(self, *a, **k):
            for n, p in super().named_parameters(*a, **k):
                yield self.names[n], p

    class ModelConfig:
        model_path = tiny

    class DeviceConfig:
        gpu_id = 0

    model = Model()
    torch.cuda.synchronize()
    loader = MxModelLoader(object(), tp_rank=2, tp_size=4)
    out = loader.load_model(model=model, model_config=ModelConfig(), device_config=DeviceConfig())
    assert out is model and not model.training
    # the stand-in has no load_weights to dry-run, so the layout rules planned this load
    assert loader.last_strategy == "b200_scatter"
    want = R.load_and_shard(read_full_tensors(tiny), 2, 4)
    got = dict(model.named_parameters())
    for n, a in want.items():
        assert np.array_equal(_as_np(got[n]), a), n
    ModelConfig.model_path = "/nonexistent"
    with pytest.raises(RuntimeError, match="No loading strategy succeeded"):
        MxModelLoader(object(), tp_rank=0, tp_size=1).load_model(
            model=model, model_config=ModelConfig(), device_config=DeviceConfig())


@pytest.mark.parametrize("rank", [0, 1])
def test_mdl_loader_warm_install(rank):
    """tests/test_mdl_tp.py:50-81 and test_mdl_fp8-style fused members on the GPU:
    global HF tensors -> this rank's fused / pre-merged / row-parallel parameters in one
    launch; the second cycle with the same buffers is 'warm' (no re-planning)."""
    import torch

    from modelexpress_b200.installer import MdlLoader

    class Model(torch.nn.Module):
        def __init__(self):
            super().__init__()
            z = lambda *s: torch.nn.Parameter(torch.zeros(*s, dtype=torch.bfloat16, device="cuda"),
                                              requires_grad=False)
            self.qkv = z(12, 8)          # (8 + 2*8) / 2 rows... q 16 rows, k 4, v 4 global, tp=2
            self.gate_up = z(8, 8)       # pre-merged [gate; up], 16 rows global
            self.o = z(8, 8)             # row-parallel: [8, 16] global
            self.norm = z(8)

        def named_parameters(self, *a, **k):
            yield "l.self_attn.qkv_proj.weight", self.qkv
            yield "l.mlp.gate_up_proj.weight", self.gate_up
            yield "l.self_attn.o_proj.weight", self.o
            yield "l.input_layernorm.weight", self.norm

    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
    w = {"l.self_attn.q_proj.weight": mk(16, 8), "l.self_attn.k_proj.weight": mk(4, 8),
         "l.self_attn.v_proj.weight": mk(4, 8), "l.mlp.gate_up_proj.weight": mk(16, 8),
         "l.self_attn.o_proj.weight": mk(8, 16), "l.input_layernorm.weight": mk(8)}
    model = Model()
    torch.cuda.synchronize()
    mdl = MdlLoader(model, tp_rank=rank, tp_size=2)

    def check():
        q, k, v = (w[f"l.self_attn.{m}_proj.weight"] for m in "qkv")
        want_qkv = torch.cat((q[rank * 8:(rank + 1) * 8], k[rank * 2:(rank + 1) * 2], v[rank * 2:(rank + 1) * 2]))
        gu = w["l.mlp.gate_up_proj.weight"]
        want_gu = torch.cat((gu[rank * 4:(rank + 1) * 4], gu[8 + rank * 4: 8 + (rank + 1) * 4]))
        assert torch.equal(model.qkv, want_qkv)
        assert torch.equal(model.gate_up, want_gu)
        assert torch.equal(model.o, w["l.self_attn.o_proj.weight"][:, rank * 8:(rank + 1) * 8])
        assert torch.equal(model.norm, w["l.input_layernorm.weight"])

    mdl.load_weights(list(w.items()))
    assert mdl.last_cycle == "cold" and mdl.cycles == 1
    check()
    for t in w.values():                      # a new version of the weights in the same buffers
        t.copy_(mk(*t.shape))
    mdl.load_weights(list(w.items()))
    assert mdl.last_cycle == "warm" and mdl.cycles == 2
    check()
    assert mdl.covered_params == {n for n, _ in model.named_parameters()}
    with pytest.raises(KeyError):
        MdlLoader(model, 0, 2).load_weights([("l.unknown.weight", mk(4, 4))])
    mdl.close()


def test_place_captured_converts_batches_and_engine_leftovers(tmp_path):
    """``place_captured`` on a hand-made engine model: a fused, tensor-parallel
    loader, a checkpoint tensor served in bf16 for an fp32 parameter (staged and
    cast on the device), a transposed expert stack (staged as the boxes it reads and
    transposed on the device), a scalar the loader reads with
    ``.item()`` (handed to the loader itself afterwards), one source per dry-run
    batch so that capture and placement interleave.  Every parameter must equal
    what the same ``load_weights`` produces from the real tensors."""
    import torch

    from modelexpress_b200 import synth
    from modelexpress_b200.loader import StrategyFailed, place_captured

    class Engine(torch.nn.Module):
        def __init__(self, rank):
            super().__init__()
            self.rank = rank
            self.qkv = torch.nn.Parameter(torch.zeros(256 + 64 + 64, 512, dtype=torch.bfloat16))
            self.down = torch.nn.Parameter(torch.zeros(512, 384, dtype=torch.bfloat16))
            self.experts = torch.nn.Parameter(torch.zeros(4, 96, 512, dtype=torch.bfloat16))
            self.router = torch.nn.Parameter(torch.zeros(4, 512, dtype=torch.float32))
            self.embed = torch.nn.Parameter(torch.ones(1024, 512, dtype=torch.bfloat16))
            self.scale = torch.nn.Parameter(torch.zeros(1, dtype=torch.float32))

        def load_weights(self, weights):
            r = self.rank
            for name, w in weights:
                if name in ("q", "k", "v"):
                    rows = {"q": 256, "k": 64, "v": 64}[name]
                    at = {"q": 0, "k": 256, "v": 320}[name]
                    self.qkv.data.narrow(0, at, rows).copy_(w.narrow(0, r * rows, rows))
                elif name == "down":
                    self.down.data.copy_(w[:, r * 384:(r + 1) * 384])
                elif name == "experts":          # stored (E, hidden, inter)
                    for e, we in enumerate(w.unbind(0)):
                        self.experts.data[e].copy_(we.t().narrow(0, r * 96, 96))
                elif name == "router":
                    self.router.data.copy_(w)
                elif name == "embed":
                    self.embed.data[: w.shape[0]].copy_(w)
                    self.embed.data[w.shape[0]:].fill_(0)
                elif name == "scale":
                    self.scale.data.fill_(w.item())

    tensors = [("q", (512, 512), "BF16", "matrix"), ("k", (128, 512), "BF16", "matrix"),
               ("scale", (1,), "F32", "matrix"), ("v", (128, 512), "BF16", "matrix"),
               ("down", (512, 768), "BF16", "matrix"), ("experts", (4, 512, 192), "BF16", "matrix"),
               ("router", (4, 512), "BF16", "matrix"), ("embed", (1000, 512), "BF16", "matrix")]
    d = str(tmp_path)
    synth.write_checkpoint(d, tensors, 77, 2)
    full = read_full_tensors(d)
    for rank in (0, 1):
        truth = Engine(rank).cuda()
        truth.load_weights((n, torch.from_numpy(a.copy()).view(
            torch.bfloat16 if a.dtype == np.uint16 else torch.float32)) for n, a in full.items())
        model = Engine(rank).cuda()
        got = place_captured(model, d, "cuda:0", first_batch=1, ring_bytes=8 << 20, ring_slots=4,
                             host_threads=2, min_row_bytes=0)
        assert got.engine_loaded == ["scale"] and "item" in got.reasons["scale"]
        assert got.converted == ["experts"] * 4 + ["router"]
        assert got.written_params == {"qkv", "down", "experts", "router", "embed"}
        assert got.copies == 3 + 1 + 4 + 1 + 1 and got.stats.chunks >= 4
        torch.cuda.synchronize()
        for (n, a), (_n, b) in zip(model.state_dict().items(), truth.state_dict().items()):
            assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), (rank, n)
    # the default settings: the same, in doubling batches
    model = Engine(1).cuda()
    got = place_captured(model, d, "cuda:0", ring_bytes=8 << 20, ring_slots=4, host_threads=2)
    assert got.engine_loaded == ["scale"] and got.converted == ["experts"] * 4 + ["router"]
    torch.cuda.synchronize()
    for (n, a), (_n, b) in zip(model.state_dict().items(), truth.state_dict().items()):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), n
    # a caller that wants every byte through the kernel is told before anything is written
    model = Engine(0).cuda()
    with pytest.raises(StrategyFailed) as e:
        place_captured(model, d, "cuda:0", on_unsupported="raise", ring_bytes=8 << 20, ring_slots=4)
    assert not e.value.mutated and float(model.qkv.detach().abs().sum()) == 0.0


def test_captured_load_keeps_images_and_replays_into_a_new_model(tmp_path):
    """place_captured(pin="keep"): the first load dry-runs the engine's loader and gathers
    into kept images; the next load of the same files, even into another model object
    of the same shapes, skips both and replays; parameters are what the loader itself
    makes of the real tensors."""
    import torch
    from safetensors.torch import save_file

    import hooked_model as H
    from modelexpress_b200.loader import HostImages, place_captured
    from modelexpress_b200.runtime import Context

    g = torch.Generator().manual_seed(13)
    tensors = {n: torch.randn(shape, generator=g, dtype=dt) for n, dt, shape in H.manifest()}
    d = str(tmp_path)
    save_file(tensors, f"{d}/model.safetensors")
    truth = H.HookedModel()
    truth.load_weights(tensors.items())
    want = {n: t.clone() for n, t in truth.state_dict().items()}
    ctx = Context([0])
    ring = ctx.ring(8 << 20, 4, 0)
    images = HostImages()
    try:
        for attempt in range(3):
            model = H.HookedModel().cuda()       # a new object (new addresses) every time
            got = place_captured(model, d, "cuda:0", ring=ring, host_threads=2, pin="keep", images=images)
            for n, t in model.state_dict().items():
                assert torch.equal(t.cpu(), want[n]), (attempt, n)
            assert got.engine_loaded == []
            if attempt == 0:
                assert got.stats.seconds_gather > 0 and got.timings["capture"] > 0
            else:
                assert got.stats.seconds_gather == 0 and got.timings["capture"] == 0.0
                assert got.stats.bytes_direct == got.stats.bytes_placed
        assert images.packed_bytes > 0
    finally:
        images.close()
        ring.close()
        ctx.close()
