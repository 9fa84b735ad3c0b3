"""The fan-out strategy at the plugin seam: a serving peer (another process, reached
over CUDA IPC) publishes its tensors, a starting replica receives them.

Source and target share one GPU here, so the target launches its receiving kernel only
after the source reported its push done (``wait_for_push``): kernels that wait on one
another must not depend on being scheduled together.  The failure paths are made on the
host: a source that never answers, a manifest that does not match; the one device-side
wait that runs out waits on counters nothing will ever raise and returns a status."""

import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _spawn(rendezvous, source_id, seed, mode):
    p = subprocess.Popen([sys.executable, os.path.join(HERE, "fanout_source_proc.py"), rendezvous, source_id,
                          str(seed), mode], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    line = p.stdout.readline().strip()
    assert line == "ready", line
    return p


def _stop(p):
    try:
        p.stdin.write("bye\n")
        p.stdin.flush()
        p.wait(timeout=30)
    except Exception:
        p.kill()


class _Ctx:
    device_id = 0
    adapter = None
    model_config = None


def _model(torch):
    from fanout_source_proc import seeded_tensors

    shapes = seeded_tensors(0, "cpu")
    m = torch.nn.Module()
    m.tensors = torch.nn.ParameterDict()
    params = {}
    for name, t in shapes.items():
        params[name] = torch.zeros_like(t, device="cuda")
    return params


@pytest.mark.gpu
def test_receive_from_a_serving_peer_then_misses_and_timeouts(tmp_path):
    import torch

    from fanout_source_proc import seeded_tensors
    from modelexpress_b200.fanout import B200FanoutStrategy
    from modelexpress_b200.loader import LoadResult, StrategyFailed

    assert torch.cuda.is_available()
    rendezvous = str(tmp_path)

    class Adapter:
        def __init__(self, dests):
            self.dests = dests

        def named_destinations(self, result):
            return self.dests

    ctx = _Ctx()
    # nobody has published: an expected miss
    strat = B200FanoutStrategy(rendezvous, timeout_ms=3000, wait_for_push=True)
    assert strat.name == "b200_fanout" and strat.is_available(ctx)
    dests = _model(torch)
    ctx.adapter = Adapter(dests)
    with pytest.raises(StrategyFailed) as e:
        strat.load(LoadResult(value=None, model=None), ctx)
    assert e.value.mutated is False

    # a silent source (published, never pushes) sorts before the live one: the host-side wait
    # for its push runs out (nothing written: not mutated), the next candidate delivers
    silent = _spawn(rendezvous, "a_silent", 5, "silent")
    live = _spawn(rendezvous, "b_live", 5, "serve")
    try:
        strat = B200FanoutStrategy(rendezvous, timeout_ms=1500, wait_for_push=True)
        res = strat.load(LoadResult(value=None, model=None), ctx)
        meta = res.metadata["b200_fanout"]
        assert meta["source_id"] == "b_live" and meta["tensors"] == len(dests)
        want = seeded_tensors(5, "cuda")
        for n, t in want.items():
            assert torch.equal(dests[n].view(torch.uint8), t.view(torch.uint8)), n
        assert live.stdout.readline().strip() == "served 1"
        # the request to the silent source was withdrawn when the wait ran out
        assert not [f for f in os.listdir(rendezvous) if ".request." in f]

        # a target whose tensor differs in size: refused before anything moves
        bad = dict(dests)
        bad["norm.weight"] = torch.zeros(128, dtype=torch.bfloat16, device="cuda")
        ctx.adapter = Adapter(bad)
        with pytest.raises(StrategyFailed) as e:
            B200FanoutStrategy(rendezvous, timeout_ms=500, wait_for_push=True).load(
                LoadResult(value=None, model=None), ctx)
        assert e.value.mutated is False and "norm.weight" in str(e.value)

        # the device-side wait: the receiving kernel is launched at once and waits for chunks the
        # silent source never sends; the bounded wait ends with a status, the parameters count as
        # touched (mutated), and the context stays usable
        os.remove(os.path.join(rendezvous, "b_live.manifest.json"))
        ctx.adapter = Adapter(dests)
        with pytest.raises(StrategyFailed) as e:
            B200FanoutStrategy(rendezvous, timeout_ms=100, wait_for_push=False).load(
                LoadResult(value=None, model=None), ctx)
        assert e.value.mutated is True and "did not complete" in str(e.value)
        from modelexpress_b200 import digest

        assert digest.safe_checksum(dests["norm.weight"]) == digest.safe_checksum(want["norm.weight"])
    finally:
        _stop(silent)
        _stop(live)


def test_retry_reinitialises_after_a_mutating_failure(monkeypatch, tmp_path):
    """rdma_strategy.py:209-247 on the host: at most three candidates; after a failure that
    may have written into the model the adapter's reinit_for_retry runs before the next
    candidate, and the strategy continues on the model it returned."""
    import json

    from modelexpress_b200 import fanout
    from modelexpress_b200.loader import LoadResult, StrategyFailed

    for sid in ("s1", "s2", "s3", "s4"):
        with open(tmp_path / f"{sid}.manifest.json", "w") as f:
            json.dump({"source_id": sid, "status": "READY" if sid != "s2" else "LOADING", "tensors": []}, f)
    calls, reinits = [], []

    class Adapter:
        def named_destinations(self, result):
            return {"from": result.value}

        def reinit_for_retry(self, result):
            reinits.append(result.value)
            return LoadResult(value=result.value + "'", model=None)

    class Ctx:
        device_id = 0
        adapter = Adapter()

    def fake_receive(self, manifest, dests, ctx):
        calls.append((manifest["source_id"], dests["from"]))
        if manifest["source_id"] == "s1":
            raise StrategyFailed("chunks missing", mutated=True)
        if manifest["source_id"] == "s3":
            raise StrategyFailed("manifest mismatch", mutated=False)
        return {"source_id": manifest["source_id"]}

    monkeypatch.setattr(fanout.B200FanoutStrategy, "_receive", fake_receive)
    strat = fanout.B200FanoutStrategy(str(tmp_path))
    out = strat.load(LoadResult(value="m", model=None), Ctx())
    # s2 is not READY; s1 mutated -> reinit -> s3 on the fresh model (expected miss) -> s4 succeeds
    assert calls == [("s1", "m"), ("s3", "m'"), ("s4", "m'")] and reinits == ["m"]
    assert out.value == "m'" and out.metadata["b200_fanout"]["source_id"] == "s4"
    # every candidate failing: the error says whether the model was touched
    monkeypatch.setattr(fanout.B200FanoutStrategy, "_receive",
                        lambda self, m, d, c: (_ for _ in ()).throw(StrategyFailed("x", mutated=m["source_id"] == "s3")))
    with pytest.raises(StrategyFailed) as e:
        fanout.B200FanoutStrategy(str(tmp_path)).load(LoadResult(value="m", model=None), Ctx())
    assert e.value.mutated is True and str(e.value).count("x") == 3


@pytest.mark.gpu
def test_push_into_a_target_whose_parameters_live_in_a_published_arena(tmp_path):
    """The target allocated its parameters through torch inside ``use_arena`` and published the
    arena: its request names every tensor by the arena's socket and an offset, and the serving
    process maps the whole arena once (descriptors over the socket) instead of opening one IPC
    handle per allocation.  Same push, same digests."""
    import torch

    from fanout_source_proc import seeded_tensors
    from modelexpress_b200 import fanout
    from modelexpress_b200.arena import Arena, lookup, publish_arena, use_arena, withdraw_arena
    from modelexpress_b200.fanout import B200FanoutStrategy
    from modelexpress_b200.loader import LoadResult

    rendezvous = str(tmp_path)
    arena = Arena(0, 4 << 30)
    shapes = seeded_tensors(0, "cpu")
    with use_arena(arena):
        dests = {n: torch.zeros_like(t, device="cuda") for n, t in shapes.items()}
    sock = publish_arena(arena, os.path.join(rendezvous, "target-arena.sock"))
    try:
        assert all(lookup(t.data_ptr(), t.numel() * t.element_size()) is not None for t in dests.values())
        rows = fanout._export_rows(fanout._tensor_rows(dests, 0))
        assert all(r["arena"] == sock and r["handle"] == "" for r in rows if r["size"])

        class Adapter:
            def named_destinations(self, result):
                return dests

        ctx = _Ctx()
        ctx.adapter = Adapter()
        live = _spawn(rendezvous, "arena_src", 8, "serve256")
        try:
            res = B200FanoutStrategy(rendezvous, timeout_ms=5000, wait_for_push=True).load(
                LoadResult(value=None, model=None), ctx)
            assert res.metadata["b200_fanout"]["tensors"] == len(dests)
            for n, t in seeded_tensors(8, "cuda").items():
                assert torch.equal(dests[n].view(torch.uint8), t.view(torch.uint8)), n
            assert live.stdout.readline().strip() == "served 1"
        finally:
            _stop(live)
    finally:
        withdraw_arena(sock)
        del dests
        torch.cuda.synchronize()
        arena.close()
